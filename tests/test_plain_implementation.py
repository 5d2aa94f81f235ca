"""The plain implementation checked against itself: float64 against float32,
each part against a second way of writing the same formula, and the sampler's
properties that the reference tests (src/runtime/sampler.zig:69-127)."""
import math

import pytest
import torch

import plain_qwen3 as P
from tiny_configs import TINY, plain_sizes
from zlm_b200.parts.model import DecoderModel
from zlm_b200.registry import config_from_dict
from zlm_b200.weights import random_tensors


def model(name, seed=0):
    cfg = config_from_dict(TINY[name])
    return cfg, random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), seed)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_float64_agrees_with_float32(name):
    cfg, t = model(name)
    ids = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    l32 = P.forward(t, plain_sizes(cfg), ids)
    l64 = P.forward({n: v.double() for n, v in t.items()}, plain_sizes(cfg), ids)
    assert l32.shape == (40, cfg.vocab_size)
    assert float((l32.double() - l64).abs().max()) < 5e-6


@pytest.mark.parametrize("name", ["A", "C"])
def test_a_position_depends_only_on_its_prefix(name):
    cfg, t = model(name)
    ids = torch.randint(0, cfg.vocab_size, (50,), generator=torch.Generator().manual_seed(2)).tolist()
    whole = P.forward(t, plain_sizes(cfg), ids)
    part = P.forward(t, plain_sizes(cfg), ids[:31])
    assert float((whole[:31] - part).abs().max()) < 1e-5


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    inv = 1.0 / math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(P.rms_norm(x, w, 1e-6), torch.tensor([[3 * inv * 2, 4 * inv * 0.5]]))


def test_rope_is_a_rotation_of_half_split_pairs():
    x = torch.randn(5, 3, 8, generator=torch.Generator().manual_seed(3))
    pos = torch.tensor([0, 1, 7, 100, 1000])
    y = P.rope_half_split(x, pos, 10000.0)
    assert torch.equal(y[0], x[0])                                 # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # pair (i, i+4) of position 7 by hand
    inv = 10000.0 ** (-2 * 1 / 8)
    a = 7 * inv
    x0, x1 = x[2, 1, 1], x[2, 1, 5]
    assert math.isclose(float(y[2, 1, 1]), float(x0 * math.cos(a) - x1 * math.sin(a)), abs_tol=1e-5)
    assert math.isclose(float(y[2, 1, 5]), float(x0 * math.sin(a) + x1 * math.cos(a)), abs_tol=1e-5)
    # the score of a rotated pair depends on the distance only
    q, k = torch.randn(1, 1, 8), torch.randn(1, 1, 8)
    s = lambda pq, pk: float((P.rope_half_split(q, torch.tensor([pq]), 1e4) * P.rope_half_split(k, torch.tensor([pk]), 1e4)).sum())
    assert math.isclose(s(10, 3), s(107, 100), abs_tol=1e-4)
    # partial rotation leaves the rest alone
    z = P.rope_half_split(x, pos, 10000.0, n_rot=4)
    assert torch.equal(z[..., 2:4], x[..., 2:4]) and torch.equal(z[..., 6:], x[..., 6:])


def test_attention_against_a_masked_dense_softmax():
    g = torch.Generator().manual_seed(4)
    T, nq, nkv, hd = 12, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, generator=g) for n in (nq, nkv, nkv))
    for window in (0, 5):
        got = P.causal_attention(q, k, v, window)
        kk, vv = k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1)
        s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(hd)
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        mask = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
        s = s.masked_fill(~mask, float("-inf"))
        want = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv)
        assert torch.allclose(got, want, atol=1e-5)


def test_swiglu_closed_form():
    g, u = torch.tensor([0.0, 1.0, -2.0]), torch.tensor([3.0, 2.0, 1.0])
    want = [0.0, 2 / (1 + math.exp(-1)), -2 / (1 + math.exp(2))]
    assert torch.allclose(P.swiglu(g, u), torch.tensor(want))


def test_sampler_properties():
    l = torch.tensor([0.1, 2.0, 2.0, -1.0, 1.5])
    assert P.argmax(l) == 1                                           # ties -> lowest index
    assert P.sample(l, 0.0, 0, 1.0, 0.7) == 1                         # temperature 0 is greedy
    assert all(P.sample(l, 0.8, 1, 1.0, u) == 1 for u in (0.0, 0.5, 0.999))   # top_k = 1 is greedy
    assert all(P.sample(l, 0.8, 0, 1e-9, u) == 1 for u in (0.0, 0.999))        # tiny top_p keeps the best
    idx, w = P.kept_set(l, 1.0, 0, 1.0)
    assert sorted(idx) == [0, 1, 2, 3, 4] and idx[:2] == [1, 2]       # top_p = 1 keeps the support
    idx, _ = P.kept_set(l, 1.0, 3, 1.0)
    assert idx == [1, 2, 4]
    idx, w = P.kept_set(l, 1.0, 0, 0.5)
    assert idx == [1, 2]                                               # 2 * e^0 / total = 0.61 >= 0.5 after two
    assert P.sample(l, 1.0, 0, 1.0, 0.0) == 1 and P.sample(l, 1.0, 0, 1.0, 0.9999) == 3
    counts = [0] * 5
    for i in range(2000):
        counts[P.sample(l, 1.0, 0, 1.0, (i + 0.5) / 2000)] += 1
    p = torch.softmax(l, 0)
    assert all(abs(c / 2000 - float(pi)) < 0.002 for c, pi in zip(counts, p))


def test_greedy_generate_stops_without_emitting_the_stop_token():
    cfg, t = model("A", seed=3)
    out = P.greedy_generate(t, plain_sizes(cfg), [1, 2, 3], 5)
    assert len(out) == 5
    k = next((i for i in range(5) if out[i] not in out[:i] and i > 0), 0)     # a token's first appearance
    assert P.greedy_generate(t, plain_sizes(cfg), [1, 2, 3], 5, stop_ids=[out[k]]) == out[:k]
    unused = next(v for v in range(cfg.vocab_size) if v not in out)
    assert P.greedy_generate(t, plain_sizes(cfg), [1, 2, 3], 5, stop_ids=[unused]) == out
