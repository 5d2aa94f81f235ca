"""The sampling kernel against the plain sampler: the kept set is the reference's
(sorted, top-k, nucleus; src/runtime/sampler.zig:30-58), the draw walks it in
index order with the uniform that the kernel derives from (seed, request, position)."""
import math

import pytest
import torch

import plain_qwen3 as P
from zlm_b200.sampling import uniform_for

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from zlm_b200.kernels import get_kernels
    return get_kernels()


def expected_token(logits, temperature, top_k, top_p, u):
    """(token, distance of r to the nearest boundary relative to the kept weight)."""
    idx, w = P.kept_set(logits, temperature, top_k, top_p)
    order = sorted(range(len(idx)), key=lambda j: idx[j])
    total = sum(w)
    r = u * total
    cum, pick, gap = 0.0, None, 1.0
    for j in order:
        cum += w[j]
        gap = min(gap, abs(cum - r) / total)
        if pick is None and r < cum:
            pick = idx[j]
    return (pick if pick is not None else idx[order[-1]]), gap


@pytest.mark.parametrize("form", ["cluster", "block"])
@pytest.mark.parametrize("V", [50, 1543, 151936])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.0, 40, 1.0), (0.7, 0, 0.9), (1.3, 50, 0.5),
                                                     (0.5, 1, 1.0), (1.0, 0, 1e-6)])
def test_draws_match_the_plain_sampler(K, V, temperature, top_k, top_p, form):
    R = 6
    g = torch.Generator().manual_seed(V + top_k)
    logits = torch.randn((R, V), generator=g) * 3.0
    logits[1, 7] = logits[1, 3] = logits[1].max() + 1.0          # a tie at the top
    logits[2] = torch.round(logits[2])                           # many ties everywhere
    req = torch.tensor([0, 5, 2, 9, 1, 3], dtype=torch.int32)
    pos = torch.tensor([10, 11, 500, 3, 77, 4095], dtype=torch.int32)
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    K.sample(out, logits.cuda(), temperature, top_k, top_p, 1234, req.cuda(), pos.cuda(), form=form)
    got = out.cpu().tolist()
    for r in range(R):
        u = uniform_for(1234, int(req[r]), int(pos[r]))
        want, gap = expected_token(logits[r], temperature, top_k, top_p, u)
        kept, _ = P.kept_set(logits[r], temperature, top_k, top_p)
        assert got[r] in kept, f"row {r}: token {got[r]} is outside the kept set of {len(kept)}"
        assert got[r] == want or gap < 1e-5, f"row {r}: got {got[r]}, want {want} (gap {gap:.2e})"


def test_the_two_forms_draw_the_same_tokens(K):
    """The cluster form (8 blocks per row) and the one-block form keep the same set and walk
    it in the same order; their 64-bit sums are grouped differently, so a draw may differ
    only where the uniform falls within rounding of a boundary."""
    R, V = 64, 40000
    g = torch.Generator().manual_seed(11)
    logits = (torch.randn((R, V), generator=g) * 2.5).cuda()
    logits[3] = torch.round(logits[3])
    req = torch.arange(R, dtype=torch.int32).cuda()
    pos = torch.arange(100, 100 + R, dtype=torch.int32).cuda()
    for temperature, top_k, top_p in [(0.9, 0, 1.0), (1.1, 64, 0.9), (0.6, 0, 0.7)]:
        a = torch.empty(R, dtype=torch.int32, device="cuda")
        b = torch.empty_like(a)
        K.sample(a, logits, temperature, top_k, top_p, 5, req, pos, form="cluster")
        K.sample(b, logits, temperature, top_k, top_p, 5, req, pos, form="block")
        assert int((a != b).sum()) <= 1, (a != b).nonzero().tolist()
    with pytest.raises(Exception, match="too long for the cluster form"):
        K.sample(torch.empty(1, dtype=torch.int32, device="cuda"), torch.zeros((1, 300000), device="cuda"), 1.0, 0, 1.0, 1,
                 req[:1].contiguous(), pos[:1].contiguous(), form="cluster")


def test_one_and_tiny_p_are_greedy_and_rows_do_not_see_each_other(K):
    V = 3001
    logits = torch.randn((4, V), generator=torch.Generator().manual_seed(1))
    req = torch.arange(4, dtype=torch.int32).cuda()
    pos = torch.full((4,), 9, dtype=torch.int32).cuda()
    out = torch.empty(4, dtype=torch.int32, device="cuda")
    best = logits.argmax(-1).tolist()
    K.sample(out, logits.cuda(), 0.9, 1, 1.0, 7, req, pos)
    assert out.cpu().tolist() == best
    K.sample(out, logits.cuda(), 0.9, 0, 1e-7, 7, req, pos)
    assert out.cpu().tolist() == best
    # the same (request, position) draws the same token whatever else is in the batch
    K.sample(out, logits.cuda(), 1.0, 0, 1.0, 7, req, pos)
    alone = torch.empty(1, dtype=torch.int32, device="cuda")
    K.sample(alone, logits[2:3].cuda(), 1.0, 0, 1.0, 7, req[2:3].contiguous(), pos[2:3].contiguous())
    assert int(alone[0]) == int(out[2])


def test_frequencies_follow_the_distribution(K):
    V, N = 37, 4000
    l = torch.randn(V, generator=torch.Generator().manual_seed(2)) * 1.5
    logits = l[None, :].repeat(N, 1).cuda()
    req = torch.zeros(N, dtype=torch.int32).cuda()
    pos = torch.arange(N, dtype=torch.int32).cuda()
    out = torch.empty(N, dtype=torch.int32, device="cuda")
    K.sample(out, logits, 0.9, 12, 0.95, 99, req, pos)
    idx, w = P.kept_set(l, 0.9, 12, 0.95)
    p = {i: wi / sum(w) for i, wi in zip(idx, w)}
    counts = torch.bincount(out.cpu().long(), minlength=V).tolist()
    assert sum(counts[i] for i in range(V) if i not in p) == 0
    for i, pi in p.items():
        assert abs(counts[i] / N - pi) < 4 * math.sqrt(pi * (1 - pi) / N) + 1e-3
