"""The order of layers as data, on the GPU: a schedule that runs layer 0 twice (weights shared, a
cache for each run) and whose last entry reads the keys and values that an earlier entry wrote
instead of writing its own (its mixer then projects queries only).  Tiny models in 32-bit and
bfloat16, and Qwen3-0.6B's layer sizes at a prompt long enough for the tensor-core products and
the tiled attention, each compared with a plain whole-sequence forward of the same schedule put
together here from the plain implementation's parts; whole, cut into steps and decoded."""
from dataclasses import replace

import pytest
import torch

import plain_qwen3 as P
from helpers import SHARP, TINY, assert_close, plain_sizes, random_prompts, reference_tensors
from test_layer_sizes_gpu import SIZES, TOL_8B

pytestmark = pytest.mark.gpu

SCHEDULE = ((0, None), (1, None), (0, None), (1, 1))      # (layer, the entry whose cache it reads)


def plain_scheduled(tensors, sizes, ids, schedule=SCHEDULE):
    """The plain forward (tests/plain_qwen3.py: decoder_layer, attention_block) in the order of
    ``schedule``; an entry that reads entry e's cache attends to the keys and values that entry
    e computed from its own input."""
    T = len(ids)
    pos = torch.arange(T)
    nq, nkv, hd, eps, theta = (sizes[n] for n in ("num_heads", "num_kv_heads", "head_dim", "eps", "rope_theta"))
    h = P.embed(tensors["model.embed_tokens.weight"], ids)
    kept = {}
    for e, (layer, cache_of) in enumerate(schedule):
        p = f"model.layers.{layer}."
        x = P.rms_norm(h, tensors[p + "input_layernorm.weight"], eps)
        q = P.linear(x, tensors[p + "self_attn.q_proj.weight"]).reshape(T, nq, hd)
        q = P.rope_half_split(P.head_rms_norm(q, tensors[p + "self_attn.q_norm.weight"], eps), pos, theta)
        if cache_of is None:
            k = P.linear(x, tensors[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd)
            k = P.rope_half_split(P.head_rms_norm(k, tensors[p + "self_attn.k_norm.weight"], eps), pos, theta)
            kept[e] = (k, P.linear(x, tensors[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd))
        k, v = kept[e if cache_of is None else cache_of]
        o = P.causal_attention(q, k, v, P.layer_window(sizes, layer)).reshape(T, nq * hd)
        h = h + P.linear(o, tensors[p + "self_attn.o_proj.weight"])
        h = h + P.feed_forward(P.rms_norm(h, tensors[p + "post_attention_layernorm.weight"], eps), tensors, layer)
    h = P.rms_norm(h, tensors["model.norm.weight"], eps)
    return P.linear(h, tensors["model.embed_tokens.weight"] if sizes["tied"] else tensors["lm_head.weight"])


def scheduled_engine(cfg, tensors, dtype, **kw):
    from zlm_b200 import Engine
    from zlm_b200.config import ScheduleEntry
    from zlm_b200.engine import parse_dtype
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.weights.loader import target_dtype
    spec = replace(cfg.to_model_spec(), schedule=tuple(ScheduleEntry(l, cache_of=c) for l, c in SCHEDULE))

    class Scheduled:
        eos_token_ids = ()

        def to_model_spec(self):
            return spec

    dt = parse_dtype(dtype)
    specs = DecoderModel(spec).param_specs()
    dev = {n: t.to("cuda").to(target_dtype(specs[n], t.dtype, dt)) for n, t in tensors.items()}
    return Engine(Scheduled(), dev, dt, "cuda:0", **kw)


def whole_cut_and_decoded(eng, prompt, want, dtype, tol, cuts, n_decode):
    from zlm_b200 import StepEntry
    from zlm_b200.sampling import SamplingParams
    n = len(prompt) - n_decode
    s = eng.new_sequence()
    got = eng.step([StepEntry(s, prompt, list(range(len(prompt))))]).clone()
    assert_close(got, want, dtype, f"schedule whole {dtype}", tol)
    eng.release(s)
    s = eng.new_sequence()            # the slot of the sequence before, used again
    parts, at = [], 0
    for c in list(cuts) + [n]:
        parts.append(eng.step([StepEntry(s, prompt[at:c], list(range(c - at)))]).clone())
        at = c
    assert_close(torch.cat(parts), want[:n], dtype, f"schedule in steps {dtype}", tol)
    for t in range(n, len(prompt)):
        eng.decoder.step([s], [prompt[t]], SamplingParams())
        assert_close(eng.decoder.last_logits.clone(), want[t:t + 1], dtype, f"schedule decode {t} {dtype}", tol)
    eng.release(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_layer_run_twice_and_a_cache_read_by_two_entries(name, dtype):
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    from zlm_b200.weights import random_tensors
    cfg = config_from_dict(TINY[name])
    tensors = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 21, "cpu", torch.float32)
    for n in tensors:
        if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
            tensors[n] = tensors[n] * SHARP[dtype]
    eng = scheduled_engine(cfg, tensors, dtype, max_tokens=512, max_batch=2)
    # three entries write (two runs of layer 0 and layer 1), one only reads
    assert sorted(e for g in eng.cache.groups for e in g.entries) == [0, 1, 2]
    n = min(150, cfg.max_position_embeddings)
    (prompt,) = random_prompts(cfg.vocab_size, [n], seed=5)
    want = plain_scheduled(reference_tensors(tensors, dtype), plain_sizes(cfg), prompt)
    assert float((want - P.forward(reference_tensors(tensors, dtype), plain_sizes(cfg), prompt)).abs().max()) > 1e-3
    whole_cut_and_decoded(eng, prompt, want, dtype, None, cuts=(64, 65, n - 20), n_decode=12)
    assert eng.rt.k.status(sync=True) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_schedule_at_layer_sizes_that_take_the_tensor_core_kernels(dtype):
    """420 tokens of Qwen3-0.6B's layer sizes: the fused query-only projection (norm and rotation
    in the product's epilogue, nothing written to the cache) and the tiled attention over pages
    that another entry wrote."""
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    from zlm_b200.weights import random_tensors
    cfg = config_from_dict(dict(SIZES["0.6B"], vocab_size=2056))
    tensors = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 6, "cpu", torch.float32)
    eng = scheduled_engine(cfg, tensors, dtype, max_tokens=1024, max_batch=2)
    (prompt,) = random_prompts(cfg.vocab_size, [420], seed=2)
    want = plain_scheduled(reference_tensors(tensors, dtype), plain_sizes(cfg), prompt)
    whole_cut_and_decoded(eng, prompt, want, dtype, TOL_8B[dtype], cuts=(390, 400), n_decode=8)
    if dtype == "bfloat16":
        assert eng.rt.k.gemm_tc_status() == 0
    assert eng.rt.k.status(sync=True) == 0
