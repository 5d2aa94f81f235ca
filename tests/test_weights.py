"""Weights by name: the safetensors container, the dtype policy, the one error
that lists everything wrong, and the random model folder."""
import json
import os
import struct

import pytest
import torch

from tiny_configs import TINY_A, TINY_B
from zlm_b200 import WeightError, write_random_model
from zlm_b200.parts.model import DecoderModel
from zlm_b200.registry import config_from_dict, config_from_folder
from zlm_b200.weights import SafetensorsError, SafetensorsFile, load_weights, random_tensors, write_safetensors


def expected(cfg):
    return DecoderModel(cfg.to_model_spec()).param_specs()


def test_names_are_the_checkpoints():
    names = set(expected(config_from_dict(TINY_B)))
    assert "model.embed_tokens.weight" in names and "model.norm.weight" in names and "lm_head.weight" in names
    for s in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
              "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
              "self_attn.q_norm.weight", "self_attn.k_norm.weight", "mlp.gate_proj.weight",
              "mlp.up_proj.weight", "mlp.down_proj.weight"):
        assert f"model.layers.2.{s}" in names
    assert len(names) == 3 + 11 * 3


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.arange(12, dtype=torch.float32).reshape(3, 4),
         "b": torch.randn(5, 2).to(torch.bfloat16), "c": torch.tensor([1, 2, 3], dtype=torch.int32),
         "d": torch.randn(2, 2).to(torch.float16), "e": torch.empty(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"format": "pt"})
    f = SafetensorsFile(p)
    assert sorted(f.names()) == sorted(t) and f.metadata == {"format": "pt"}
    for n, v in t.items():
        got = f.tensor(n)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)


def test_truncated_and_malformed_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": torch.zeros(100)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-50])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="not JSON"):
        SafetensorsFile(p)


def test_random_folder_loads_back(tmp_path):
    cfg = config_from_dict(TINY_A)
    write_random_model(str(tmp_path), cfg, seed=5)
    assert config_from_folder(str(tmp_path)) == cfg
    exp = expected(cfg)
    w32 = load_weights(str(tmp_path), exp, torch.float32, "cpu")
    wbf = load_weights(str(tmp_path), exp, torch.bfloat16, "cpu")
    assert "lm_head.weight" not in w32                       # tied: the table serves as head
    again = random_tensors(exp, 5)
    for n, t in w32.items():
        assert t.dtype == torch.float32 and torch.equal(t, again[n])
    # bfloat16: matrices narrowed, norm vectors stay 32-bit because the file stores them so
    assert wbf["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert wbf["model.layers.0.input_layernorm.weight"].dtype == torch.float32
    assert wbf["model.layers.0.self_attn.q_norm.weight"].dtype == torch.float32
    # distributions: N(0, 0.02) and 1 + N(0, 0.02)
    e = w32["model.embed_tokens.weight"]
    assert abs(float(e.std()) - 0.02) < 0.002 and abs(float(e.mean())) < 0.002
    assert abs(float(w32["model.norm.weight"].mean()) - 1.0) < 0.02
    # another seed gives other weights; the same seed the same
    assert not torch.equal(random_tensors(exp, 6)["model.norm.weight"], again["model.norm.weight"])


def test_bf16_file_stays_bf16_and_widens_for_fp32(tmp_path):
    cfg = config_from_dict(TINY_A)
    write_random_model(str(tmp_path), cfg, seed=1, dtype=torch.bfloat16)
    exp = expected(cfg)
    wbf = load_weights(str(tmp_path), exp, torch.bfloat16, "cpu")
    assert all(t.dtype == torch.bfloat16 for t in wbf.values())
    w32 = load_weights(str(tmp_path), exp, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["model.norm.weight"], wbf["model.norm.weight"].float())


def test_one_error_lists_everything(tmp_path):
    cfg = config_from_dict(TINY_B)
    exp = expected(cfg)
    t = random_tensors(exp, 0)
    del t["model.layers.1.self_attn.k_norm.weight"]
    del t["lm_head.weight"]
    t["model.layers.0.mlp.up_proj.weight"] = torch.zeros(160, 95)
    t["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    t["model.norm.weight"] = torch.ones(96, dtype=torch.int32)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg.to_dict(), f)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightError) as ei:
        load_weights(str(tmp_path), exp, torch.float32, "cpu")
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.k_norm.weight"]
    assert e.unexpected == ["model.layers.7.mlp.up_proj.weight"]
    assert e.wrong_shape == [("model.layers.0.mlp.up_proj.weight", (160, 95), (160, 96))]
    assert e.wrong_dtype == [("model.norm.weight", "torch.int32")]
    msg = str(e)
    for s in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "is [160, 95], expected [160, 96]"):
        assert s in msg


def test_tied_checkpoint_may_carry_a_head_copy(tmp_path):
    cfg = config_from_dict(TINY_A)
    exp = expected(cfg)
    t = random_tensors(exp, 0)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    w = load_weights(str(tmp_path), exp, torch.float32, "cpu")
    assert "lm_head.weight" not in w


def test_sharded_checkpoint_and_duplicates(tmp_path):
    cfg = config_from_dict(TINY_A)
    exp = expected(cfg)
    t = random_tensors(exp, 0)
    names = sorted(t)
    a, b = {n: t[n] for n in names[:7]}, {n: t[n] for n in names[7:]}
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), a)
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), b)
    wm = {n: "model-00001-of-00002.safetensors" for n in a}
    wm.update({n: "model-00002-of-00002.safetensors" for n in b})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    w = load_weights(str(tmp_path), exp, torch.float32, "cpu")
    assert all(torch.equal(w[n], t[n]) for n in t)
    b[names[0]] = t[names[0]]
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), b)
    with pytest.raises(WeightError, match="appears in"):
        load_weights(str(tmp_path), exp, torch.float32, "cpu")
    with pytest.raises(WeightError, match="neither model.safetensors"):
        load_weights(str(tmp_path / "empty"), exp, torch.float32, "cpu")
