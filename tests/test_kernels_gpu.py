"""Each CUDA kernel alone against its plain torch reference (tests/cpu_kernels.py),
at sizes other than the tiny models': widths and vocabularies that are no power
of two, head sizes in steps of 16, odd head counts and groups."""
import math

import pytest
import torch

from cpu_kernels import PAGE, PlainKernels

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def K():
    from zlm_b200.kernels import get_kernels
    return get_kernels()


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(got, want, dtype, atol=None, rtol=None):
    atol = atol if atol is not None else (1e-5 if dtype == torch.float32 else 2e-2)
    rtol = rtol if rtol is not None else (1e-5 if dtype == torch.float32 else 2e-2)
    torch.testing.assert_close(got.float().cpu(), want.float().cpu(), atol=atol, rtol=rtol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(K, dtype):
    V, H, T = 301, 72, 9
    table = rnd((V, H), DT[dtype], 1)
    ids = torch.tensor([0, 300, 7, 7, 150, 1, 299, 33, 2], dtype=torch.int32)
    want = torch.empty(T, H)
    PlainKernels().embed(want, table, ids)
    got = torch.empty(T, H, device="cuda")
    K.embed(got, table.cuda(), ids.cuda())
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("w_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [72, 1000, 4096])
def test_rmsnorm(K, out_dtype, w_dtype, H):
    T = 5
    x = rnd((T, H), torch.float32, 2, 3.0)
    w = (1 + rnd((H,), torch.float32, 3, 0.1)).to(DT[w_dtype])
    rows = torch.tensor([4, 0, 2], dtype=torch.int32)
    for r in (None, rows):
        R = T if r is None else 3
        want = torch.empty(R, H, dtype=DT[out_dtype])
        PlainKernels().rmsnorm(want, x, w, 1e-5, r)
        got = torch.empty(R, H, dtype=DT[out_dtype], device="cuda")
        K.rmsnorm(got, x.cuda(), w.cuda(), 1e-5, None if r is None else r.cuda())
        close(got, want, DT[out_dtype], atol=1e-5 if out_dtype == "float32" else 4e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(K, dtype):
    T, I = 7, 200
    gu = rnd((T, 2 * I), DT[dtype], 4, 4.0)
    want = torch.empty(T, I, dtype=DT[dtype])
    PlainKernels().swiglu(want, gu)
    got = torch.empty(T, I, dtype=DT[dtype], device="cuda")
    K.swiglu(got, gu.cuda())
    close(got, want, DT[dtype], atol=1e-5 if dtype == "float32" else 5e-2)


@pytest.mark.parametrize("T,N,K_", [(1, 70, 50), (3, 129, 77), (64, 64, 16), (65, 200, 1000), (130, 67, 33)])
def test_linear_f32(K, T, N, K_):
    x, w = rnd((T, K_), torch.float32, 5), rnd((N, K_), torch.float32, 6, 0.1)
    want = x.double() @ w.double().t()
    got = torch.empty(T, N, device="cuda")
    K.linear(got, x.cuda(), w.cuda())
    close(got, want, torch.float32, atol=1e-5, rtol=1e-5)
    base = rnd((T, N), torch.float32, 7)
    acc = base.clone().cuda()
    K.linear(acc, x.cuda(), w.cuda(), accumulate=True)
    close(acc, base.double() + want, torch.float32, atol=1e-5, rtol=1e-5)


def test_linear_f32_is_batch_invariant(K):
    x, w = rnd((70, 300), torch.float32, 8), rnd((90, 300), torch.float32, 9)
    whole = torch.empty(70, 90, device="cuda")
    K.linear(whole, x.cuda(), w.cuda())
    for t in (0, 13, 69):
        one = torch.empty(1, 90, device="cuda")
        K.linear(one, x[t:t + 1].contiguous().cuda(), w.cuda())
        assert torch.equal(one[0], whole[t])


@pytest.mark.parametrize("T", [1, 2, 3, 4, 5, 8, 9, 16, 17, 33, 64, 65, 128, 300])
@pytest.mark.parametrize("N,K_", [(72, 40), (200, 1000), (1024, 512), (151, 4096)])
def test_linear_bf16(K, T, N, K_):
    x, w = rnd((T, K_), torch.bfloat16, 10), rnd((N, K_), torch.bfloat16, 11, 0.05)
    want = x.double() @ w.double().t()
    for out_dtype in (torch.bfloat16, torch.float32):
        got = torch.empty(T, N, dtype=out_dtype, device="cuda")
        K.linear(got, x.cuda(), w.cuda())
        close(got, want, out_dtype, atol=1e-3 if out_dtype == torch.float32 else 3e-2, rtol=1e-2)
    base = rnd((T, N), torch.float32, 12)
    acc = base.clone().cuda()
    K.linear(acc, x.cuda(), w.cuda(), accumulate=True)
    close(acc, base.double() + want, torch.float32, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("T", [1, 8, 11, 16])
@pytest.mark.parametrize("N,K_", [(6144, 1024), (5000 + 9, 1000), (6144, 4096), (9600, 640), (5120, 3072)])
def test_linear_bf16_gemv_blocks_of_four_warps(K, T, N, K_):
    """More outputs than one round of the wide blocks holds: the product runs blocks of four warps
    where the estimate says so (it does for each of these sizes at one token tile or at two).  All
    output modes, a ragged number of outputs and a ragged K, and the fused gate/up epilogue; one
    output far from the others' size, so that a block that read another block's rows shows."""
    from zlm_b200.kernels import interleave_gate_up
    assert 4 in (K.lib.zlm_gemv_plan_warps(N, K_, 148, 2, 5), K.lib.zlm_gemv_plan_warps(N, K_, 148, 2, 4))
    x, w = rnd((T, K_), torch.bfloat16, 13), rnd((N, K_), torch.bfloat16, 14, 0.03)
    w[N - 3] *= 30.0
    want = x.double() @ w.double().t()
    for out_dtype in (torch.bfloat16, torch.float32):
        got = torch.full((T, N), 7.0, dtype=out_dtype, device="cuda")
        K.linear(got, x.cuda(), w.cuda(), impl="gemv")
        close(got, want, out_dtype, atol=1e-3 if out_dtype == torch.float32 else 3e-2, rtol=1e-2)
    base = rnd((T, N), torch.float32, 15)
    acc = base.clone().cuda()
    K.linear(acc, x.cuda(), w.cuda(), accumulate=True, impl="gemv")
    close(acc, base.double() + want, torch.float32, atol=1e-3, rtol=1e-3)
    I = (N // 32) * 16
    gate, up = w[:I], w[I:2 * I]
    g, u = x.double() @ gate.double().t(), x.double() @ up.double().t()
    got = torch.full((T, I), 7.0, dtype=torch.bfloat16, device="cuda")
    K.linear_swiglu(got, x.cuda(), interleave_gate_up(gate.cuda(), up.cuda()), impl="gemv")
    close(got, (g / (1 + torch.exp(-g))) * u, torch.bfloat16, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("T", [1, 7, 8, 13, 16])
@pytest.mark.parametrize("K_,seg", [(1024, 128), (2048, 256), (3072, 384), (5120, 640), (7168, 128), (4096, 512),
                                    (12288, 512), (1000, 512), (4104, 512)])
def test_linear_bf16_gemv_segments(K, T, K_, seg):
    """The weight-streaming product at every width of a warp's share of K (chosen so that K
    spreads evenly over the warps; 512 where K is a multiple of 4096 or ragged), one and two
    token tiles, a ragged number of outputs, all output modes and the fused gate/up epilogue."""
    from zlm_b200.kernels import interleave_gate_up
    assert K.lib.zlm_gemv_segment(K_) == seg
    N = 208 + 9
    x, w = rnd((T, K_), torch.bfloat16, 13), rnd((N, K_), torch.bfloat16, 14, 0.03)
    want = x.double() @ w.double().t()
    for out_dtype in (torch.bfloat16, torch.float32):
        got = torch.full((T, N), 7.0, dtype=out_dtype, device="cuda")
        K.linear(got, x.cuda(), w.cuda(), impl="gemv")
        close(got, want, out_dtype, atol=1e-3 if out_dtype == torch.float32 else 3e-2, rtol=1e-2)
    base = rnd((T, N), torch.float32, 15)
    acc = base.clone().cuda()
    K.linear(acc, x.cuda(), w.cuda(), accumulate=True, impl="gemv")
    close(acc, base.double() + want, torch.float32, atol=1e-3, rtol=1e-3)
    gate, up = w[:104], w[104:208]
    g, u = x.double() @ gate.double().t(), x.double() @ up.double().t()
    got = torch.full((T, 104), 7.0, dtype=torch.bfloat16, device="cuda")
    K.linear_swiglu(got, x.cuda(), interleave_gate_up(gate.cuda(), up.cuda()), impl="gemv")
    close(got, (g / (1 + torch.exp(-g))) * u, torch.bfloat16, atol=3e-2, rtol=3e-2)


def test_linear_bf16_refuses_odd_inner_size(K):
    from zlm_b200.kernels import KernelError
    x, w = rnd((4, 36), torch.bfloat16, 1).cuda(), rnd((8, 36), torch.bfloat16, 2).cuda()
    with pytest.raises(KernelError, match="multiple of 8"):
        K.linear(torch.empty(4, 8, dtype=torch.bfloat16, device="cuda"), x, w)


def make_paged(nkv, hd, lens, dtype, seed, n_pages=64):
    """A pool filled at random, a shuffled block table, and per-sequence slots that
    are not 0, 1, 2 ... so that a wrong slot or page shows."""
    g = torch.Generator().manual_seed(seed)
    pool = (torch.randn((n_pages, 2, nkv, PAGE, hd), generator=g)).to(dtype)
    slots = [3, 0, 5, 1, 4][:len(lens)]
    table = torch.zeros((6, 16), dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).tolist()
    for s, n in zip(slots, lens):
        for lp in range((n + PAGE - 1) // PAGE):
            table[s, lp] = perm.pop()
    return pool, table, slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,hd,n_rot,norm", [(4, 2, 16, 16, True), (6, 2, 48, 48, True), (5, 5, 80, 32, False),
                                                  (8, 1, 128, 128, True), (3, 1, 256, 0, True)])
def test_qk_norm_rope_write(K, dtype, nq, nkv, hd, n_rot, norm):
    dt = DT[dtype]
    lens = [70, 5, 130]
    pool, table, slots = make_paged(nkv, hd, lens, dt, 20)
    # new tokens: the last 3 positions of each sequence
    pos = torch.tensor([p for n in lens for p in range(n - 3, n)], dtype=torch.int32)
    slot = torch.tensor([s for s in slots for _ in range(3)], dtype=torch.int32)
    T = pos.numel()
    qkv = rnd((T, (nq + 2 * nkv) * hd), dt, 21, 2.0)
    qw = (1 + rnd((hd,), torch.float32, 22, 0.2)) if norm else None
    kw = (1 + rnd((hd,), torch.float32, 23, 0.2)) if norm else None
    i = torch.arange(n_rot // 2, dtype=torch.float64)
    inv = (10000.0 ** (-2.0 * i / hd)).float() if n_rot else None
    want_qkv, want_pool = qkv.clone(), pool.clone()
    PlainKernels().qk_norm_rope_write(want_qkv, qw, kw, 1e-6, inv, n_rot, pos, slot, table, want_pool, nq, nkv, hd)
    got_qkv, got_pool = qkv.cuda(), pool.cuda()
    c = lambda t: None if t is None else t.cuda()
    K.qk_norm_rope_write(got_qkv, c(qw), c(kw), 1e-6, c(inv), n_rot, pos.cuda(), slot.cuda(), table.cuda(),
                         got_pool, nq, nkv, hd)
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=5e-2, rtol=2e-2)
    close(got_qkv[:, :nq * hd], want_qkv[:, :nq * hd], dt, **tol)
    close(got_pool, want_pool, dt, **tol)
    # nothing but the new tokens' places changed
    changed = (got_pool.cpu() != pool).any(-1).sum().item()
    assert changed <= T * 2 * nkv


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,hd,window", [(4, 2, 16, 0), (6, 2, 48, 24), (5, 5, 80, 0), (8, 1, 128, 100),
                                              (3, 1, 256, 0), (32, 8, 128, 0)])
def test_attention_over_the_cache(K, dtype, nq, nkv, hd, window):
    """Decode-like (one query per sequence) and prefill-like (several queries) rows
    over sequences that span pages; one far key is made to stand out."""
    dt = DT[dtype]
    lens = [300, 5, 129, 64]
    pool, table, slots = make_paged(nkv, hd, lens, dt, 30)
    pos_list, slot_list = [], []
    for n, s in zip(lens, slots):
        for p in ([n - 1] if n != 129 else list(range(120, 129))):
            pos_list.append(p)
            slot_list.append(s)
    pos = torch.tensor(pos_list, dtype=torch.int32)
    slot = torch.tensor(slot_list, dtype=torch.int32)
    T = pos.numel()
    q = rnd((T, nq * hd), dt, 31)
    # make key 17 of the first sequence (far from its query at 299) dominate head 0
    page = int(table[slots[0], 17 // PAGE])
    scale = 1.0 / math.sqrt(hd)
    q0 = q[0, :hd].float()
    pool[page, 0, 0, 17 % PAGE, :] = (q0 * (30.0 / (float(q0 @ q0) * scale))).to(dt)   # score 30
    want = torch.empty(T, nq * hd, dtype=dt)
    PlainKernels().attention(want, q, pool, table, pos, slot, nq, nkv, hd, scale, window)
    got = torch.empty(T, nq * hd, dtype=dt, device="cuda")
    K.attention(got, q.cuda(), pool.cuda(), table.cuda(), pos.cuda(), slot.cuda(), nq, nkv, hd, scale, window)
    close(got, want, dt, atol=2e-5 if dtype == "float32" else 3e-2, rtol=1e-4 if dtype == "float32" else 3e-2)
    if window == 0:
        # the far key really carries the first row's head 0
        v17 = pool[page, 1, 0, 17 % PAGE, :].float()
        assert (got[0, :hd].float().cpu() - v17).abs().max() < 0.05 * v17.abs().max() + 0.05


def test_argmax_ties_to_lowest_index(K):
    V = 1543
    logits = rnd((5, V), torch.float32, 40)
    logits[1, 700] = logits[1, 1400] = 50.0
    logits[2, :] = 0.0
    logits[3, V - 1] = 99.0
    logits[4, 0] = 99.0
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    K.argmax(out, logits.cuda())
    want = torch.empty(5, dtype=torch.int32)
    PlainKernels().argmax(want, logits)
    assert out.cpu().tolist() == want.tolist() == [int(logits[0].argmax()), 700, 0, V - 1, 0]


class FakePlan:
    """What the attention kernel wants to know about a step."""

    def __init__(self):
        self.is_decode = True
        self.bufs = {}

    def scratch(self, name, shape, dtype):
        self.bufs[name] = torch.empty(shape, dtype=dtype, device="cuda")
        return self.bufs[name]


@pytest.mark.parametrize("len_bucket", [16, 64, 1024])
@pytest.mark.parametrize("nq,nkv,hd,window", [(4, 2, 16, 0), (6, 2, 48, 24), (5, 5, 80, 0), (8, 1, 128, 100),
                                              (32, 8, 128, 0), (16, 1, 64, 0), (6, 3, 32, 70)])
def test_attention_decode_kernel(K, nq, nkv, hd, window, len_bucket):
    """The split-KV decode kernel (one query per sequence) for several numbers of
    splits, with a far key that dominates one head and a sequence that ends exactly
    at a page's edge."""
    from zlm_b200.kernels import decode_splits
    dt = torch.bfloat16
    lens = [700, 5, 129, 64, 65]
    pool, table, slots = make_paged(nkv, hd, lens, dt, 50, n_pages=40)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    slot = torch.tensor(slots, dtype=torch.int32)
    T = pos.numel()
    q = rnd((T, nq * hd), dt, 51)
    scale = 1.0 / math.sqrt(hd)
    far = 17 if window == 0 else 700 - window          # the oldest key the query may see
    page = int(table[slots[0], far // PAGE])
    qh = q[0, (nq - 1) * hd:].float()                  # last head -> last kv head
    pool[page, 0, nkv - 1, far % PAGE, :] = (qh * (30.0 / (float(qh @ qh) * scale))).to(dt)
    want = torch.empty(T, nq * hd, dtype=dt)
    PlainKernels().attention(want, q, pool, table, pos, slot, nq, nkv, hd, scale, window)
    got = torch.empty(T, nq * hd, dtype=dt, device="cuda")
    plan = FakePlan()
    K.attention(got, q.cuda(), pool.cuda(), table.cuda(), pos.cuda(), slot.cuda(), nq, nkv, hd, scale, window, plan,
                len_bucket=len_bucket)
    assert (decode_splits(T, nkv, len_bucket, K.sm_count * 3)[0] > 1) == bool(plan.bufs)
    close(got, want, dt, atol=3e-2, rtol=3e-2)
    vfar = pool[page, 1, nkv - 1, far % PAGE, :].float()
    assert (got[0, (nq - 1) * hd:].float().cpu() - vfar).abs().max() < 0.05 * vfar.abs().max() + 0.05


class PrefillPlan:
    """A step of several sequences with several new tokens each, as the engine's
    StepContext describes it."""
    is_decode = False

    def __init__(self, slots, starts, news):
        cu = [0]
        for n in news:
            cu.append(cu[-1] + n)
        self.R, self.max_new = len(slots), max(news)
        self.cu_seqlens = torch.tensor(cu, dtype=torch.int32).cuda()
        self.seq_slot = torch.tensor(slots, dtype=torch.int32).cuda()
        self.seq_start = torch.tensor(starts, dtype=torch.int32).cuda()


@pytest.mark.parametrize("impl", ["mma", None, "tc1", "tc2"])
@pytest.mark.parametrize("nq,nkv,hd,window", [(4, 2, 16, 0), (6, 2, 48, 24), (5, 5, 80, 0), (8, 1, 128, 100),
                                              (32, 8, 128, 0), (6, 3, 32, 70), (4, 1, 64, 64), (3, 3, 128, 0),
                                              (4, 2, 128, 17)])
def test_attention_prefill_kernel(K, nq, nkv, hd, window, impl):
    """Tiles of query tokens over the paged cache: whole prompts, a chunk that
    continues a cached prefix, a single token, tile and page edges; a far key
    dominates one head of the last query of the first sequence."""
    dt = torch.bfloat16
    lens = [300, 5, 129, 64, 65]          # lengths after the step
    news = [300, 5, 70, 1, 65]            # of which new in this step
    pool, table, slots = make_paged(nkv, hd, lens, dt, 60, n_pages=40)
    starts = [l - n for l, n in zip(lens, news)]
    pos = torch.tensor([p for s, n in zip(starts, news) for p in range(s, s + n)], dtype=torch.int32)
    slot = torch.tensor([sl for sl, n in zip(slots, news) for _ in range(n)], dtype=torch.int32)
    T = pos.numel()
    q = rnd((T, nq * hd), dt, 61)
    scale = 1.0 / math.sqrt(hd)
    far = 17 if window == 0 else 300 - window
    page = int(table[slots[0], far // PAGE])
    qh = q[299, (nq - 1) * hd:].float()
    pool[page, 0, nkv - 1, far % PAGE, :] = (qh * (30.0 / (float(qh @ qh) * scale))).to(dt)
    want = torch.empty(T, nq * hd, dtype=dt)
    PlainKernels().attention(want, q, pool, table, pos, slot, nq, nkv, hd, scale, window)
    got = torch.empty(T, nq * hd, dtype=dt, device="cuda")
    plan = PrefillPlan(slots, starts, news)
    # None: the tcgen05 kernel where it takes the shape (head size 128), with one or two heads of a
    # kv group per block as it chooses; "tc1" / "tc2" force that number
    plan.attention_impl = impl if impl == "mma" else None
    K.set_prefill_attention_heads({"tc1": 1, "tc2": 2}.get(impl, 0))
    try:
        K.attention(got, q.cuda(), pool.cuda(), table.cuda(), pos.cuda(), slot.cuda(), nq, nkv, hd, scale, window, plan)
    finally:
        K.set_prefill_attention_heads(0)
    assert K.gemm_tc_status() == 0
    close(got, want, dt, atol=3e-2, rtol=3e-2)
    vfar = pool[page, 1, nkv - 1, far % PAGE, :].float()
    assert (got[299, (nq - 1) * hd:].float().cpu() - vfar).abs().max() < 0.05 * vfar.abs().max() + 0.05


@pytest.mark.parametrize("T,N,K_", [(128, 256, 64), (130, 300, 72), (200, 151, 1000), (128, 8, 64), (1, 40, 24),
                                    (300, 1000, 520), (512, 768, 2048)])
def test_linear_bf16_tcgen05(K, T, N, K_):
    """The TMA + tcgen05 product at aligned and ragged shapes (tails in T, N and K are
    zero-filled by the tensor maps), in all three output modes; no bounded wait gave up."""
    x, w = rnd((T, K_), torch.bfloat16, 70), rnd((N, K_), torch.bfloat16, 71, 0.05)
    want = x.double() @ w.double().t()
    for out_dtype in (torch.bfloat16, torch.float32):
        got = torch.full((T, N), 7.0, dtype=out_dtype, device="cuda")
        K.linear(got, x.cuda(), w.cuda(), impl="tc")
        close(got, want, out_dtype, atol=1e-3 if out_dtype == torch.float32 else 3e-2, rtol=1e-2)
    base = rnd((T, N), torch.float32, 72)
    acc = base.clone().cuda()
    K.linear(acc, x.cuda(), w.cuda(), accumulate=True, impl="tc")
    close(acc, base.double() + want, torch.float32, atol=1e-3, rtol=1e-3)
    assert K.gemm_tc_status() == 0


@pytest.mark.parametrize("form,width", [("single", 256), ("single", 240), ("single", 224), ("pair", 256),
                                        ("pair", 240), ("pair", 224), ("pair", 128), (None, 0)])
@pytest.mark.parametrize("T,N,K_", [(385, 300, 72), (700, 2064, 264), (1000, 1000, 520)])
def test_linear_bf16_tcgen05_many_tokens(K, T, N, K_, form, width):
    """The persistent many-token product in both forms (one block per tile; a pair of
    blocks per tile, cta_group::2) at every tile width, several tiles per block, ragged
    in T, N and K, all output modes and the fused gate/up epilogue."""
    from zlm_b200.kernels import interleave_gate_up
    x, w = rnd((T, K_), torch.bfloat16, 75), rnd((N, K_), torch.bfloat16, 76, 0.05)
    want = x.double() @ w.double().t()
    K.set_gemm_form(form, width)
    try:
        for out_dtype in (torch.bfloat16, torch.float32):
            got = torch.full((T, N), 7.0, dtype=out_dtype, device="cuda")
            K.linear(got, x.cuda(), w.cuda(), impl="tc")
            close(got, want, out_dtype, atol=1e-3 if out_dtype == torch.float32 else 3e-2, rtol=1e-2)
        base = rnd((T, N), torch.float32, 77)
        acc = base.clone().cuda()
        K.linear(acc, x.cuda(), w.cuda(), accumulate=True, impl="tc")
        close(acc, base.double() + want, torch.float32, atol=1e-3, rtol=1e-3)
        # the output as columns of a wider tensor: what lies beside them stays as it was (the
        # epilogue's boxes are clipped at the product's own width, not at the row's)
        for out_dtype in (torch.bfloat16, torch.float32):
            wide = torch.full((T, N + 24), 7.0, dtype=out_dtype, device="cuda")
            K.linear(wide[:, 8:8 + N], x.cuda(), w.cuda(), accumulate=out_dtype == torch.float32, impl="tc")
            close(wide[:, 8:8 + N], want + (7.0 if out_dtype == torch.float32 else 0.0), out_dtype,
                  atol=1e-3 if out_dtype == torch.float32 else 3e-2, rtol=1e-2)
            assert bool((wide[:, :8] == 7.0).all()) and bool((wide[:, 8 + N:] == 7.0).all())
        if N % 16 == 0:
            gate, up = w[:N // 2], w[N // 2:]
            g, u = x.double() @ gate.double().t(), x.double() @ up.double().t()
            got = torch.full((T, N // 2), 7.0, dtype=torch.bfloat16, device="cuda")
            K.linear_swiglu(got, x.cuda(), interleave_gate_up(gate.cuda(), up.cuda()), impl="tc")
            close(got, (g / (1 + torch.exp(-g))) * u, torch.bfloat16, atol=3e-2, rtol=3e-2)
    finally:
        K.set_gemm_form(None, 0)
    assert K.gemm_tc_status() == 0


@pytest.mark.parametrize("T,N,K_", [(40, 19040, 1032), (300, 8000, 1024), (17, 24576, 520), (100, 37904, 264)])
def test_linear_bf16_tcgen05_few_tokens_many_tiles(K, T, N, K_):
    """The few-token product with more tiles than SMs: the persistent form, whose blocks walk
    several tiles, computes as many full rounds of tiles in one piece and cuts the rest along K
    (shares added up by the second kernel, from some output on); one or several token tiles;
    all output modes and the fused gate/up epilogue; the same bits on a second run."""
    from zlm_b200.kernels import interleave_gate_up
    x, w = rnd((T, K_), torch.bfloat16, 86), rnd((N, K_), torch.bfloat16, 87, 0.05)
    want = x.double() @ w.double().t()
    outs = []
    for rep in range(2):
        for out_dtype in (torch.bfloat16, torch.float32):
            got = torch.full((T, N), 7.0, dtype=out_dtype, device="cuda")
            K.linear(got, x.cuda(), w.cuda(), impl="tc")
            close(got, want, out_dtype, atol=1e-3 if out_dtype == torch.float32 else 3e-2, rtol=1e-2)
            outs.append(got)
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
    base = rnd((T, N), torch.float32, 88)
    acc = base.clone().cuda()
    K.linear(acc, x.cuda(), w.cuda(), accumulate=True, impl="tc")
    close(acc, base.double() + want, torch.float32, atol=1e-3, rtol=1e-3)
    gate, up = w[:N // 2], w[N // 2:]
    g, u = x.double() @ gate.double().t(), x.double() @ up.double().t()
    got = torch.full((T, N // 2), 7.0, dtype=torch.bfloat16, device="cuda")
    K.linear_swiglu(got, x.cuda(), interleave_gate_up(gate.cuda(), up.cuda()), impl="tc")
    close(got, (g / (1 + torch.exp(-g))) * u, torch.bfloat16, atol=3e-2, rtol=3e-2)
    assert K.gemm_tc_status() == 0


@pytest.mark.parametrize("form", ["single", "pair"])
def test_linear_bf16_tcgen05_groups_of_token_tiles(K, form):
    """A product whose token tiles are walked in more than one group (a group's activations
    are sized to stay in L2: with K = 16384 that is 8 tiles of 256 tokens, 16 of 128), the
    last group not full."""
    T, N, K_ = 2400, 300, 16384
    x, w = rnd((T, K_), torch.bfloat16, 78), rnd((N, K_), torch.bfloat16, 79, 0.02)
    want = (x.cuda().double() @ w.cuda().double().t()).cpu()
    K.set_gemm_form(form, 0)
    try:
        got = torch.full((T, N), 7.0, dtype=torch.float32, device="cuda")
        K.linear(got, x.cuda(), w.cuda(), impl="tc")
    finally:
        K.set_gemm_form(None, 0)
    close(got, want, torch.float32, atol=2e-3, rtol=1e-3)
    assert K.gemm_tc_status() == 0


def test_linear_bf16_kernels_agree(K):
    """The three bf16 products give the same numbers up to the order of their sums."""
    x, w = rnd((16, 512), torch.bfloat16, 73), rnd((384, 512), torch.bfloat16, 74, 0.05)
    outs = []
    for impl in ("gemv", "mma", "tc"):
        o = torch.empty(16, 384, dtype=torch.float32, device="cuda")
        K.linear(o, x.cuda(), w.cuda(), impl=impl)
        outs.append(o.cpu())
    torch.testing.assert_close(outs[0], outs[1], atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(outs[0], outs[2], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("T", [1, 3, 8, 16, 17, 40, 64, 100, 128, 300, 500])
@pytest.mark.parametrize("I,K_", [(64, 40), (200, 1000), (1536, 512)])
def test_linear_swiglu_fused(K, T, I, K_):
    """silu(x . gate) * (x . up) in the product's epilogue, for every kernel that has
    the epilogue, against the plain formula on the same bf16 inputs."""
    from zlm_b200.kernels import interleave_gate_up
    x = rnd((T, K_), torch.bfloat16, 80)
    gate, up = rnd((I, K_), torch.bfloat16, 81, 0.08), rnd((I, K_), torch.bfloat16, 82, 0.08)
    g, u = x.double() @ gate.double().t(), x.double() @ up.double().t()
    want = (g / (1 + torch.exp(-g))) * u
    w = interleave_gate_up(gate.cuda(), up.cuda())
    assert torch.equal(w[:8].cpu(), gate[:8]) and torch.equal(w[8:16].cpu(), up[:8]) and torch.equal(w[16:24].cpu(), gate[8:16])
    impls = [None, "tc", "mma"] + (["gemv"] if T <= 16 else [])
    for impl in impls:
        got = torch.full((T, I), 7.0, dtype=torch.bfloat16, device="cuda")
        K.linear_swiglu(got, x.cuda(), w, impl=impl)
        close(got, want, torch.bfloat16, atol=3e-2, rtol=3e-2)
    assert K.gemm_tc_status() == 0


@pytest.mark.parametrize("T", [17, 33, 64, 65, 129, 384, 385])
def test_linear_bf16_tcgen05_few_tokens(K, T):
    """The swapped-operand form (W is the 128-row operand) for decode-sized batches."""
    N, K_ = 712, 520
    x, w = rnd((T, K_), torch.bfloat16, 83), rnd((N, K_), torch.bfloat16, 84, 0.05)
    want = x.double() @ w.double().t()
    got = torch.full((T, N), 7.0, dtype=torch.bfloat16, device="cuda")
    K.linear(got, x.cuda(), w.cuda(), impl="tc")
    close(got, want, torch.bfloat16, atol=3e-2, rtol=1e-2)
    base = rnd((T, N), torch.float32, 85)
    acc = base.clone().cuda()
    K.linear(acc, x.cuda(), w.cuda(), accumulate=True, impl="tc")
    close(acc, base.double() + want, torch.float32, atol=1e-3, rtol=1e-3)
    lg = torch.empty((T, N), dtype=torch.float32, device="cuda")
    K.linear(lg, x.cuda(), w.cuda(), impl="tc")
    close(lg, want, torch.float32, atol=1e-3, rtol=1e-3)
    assert K.gemm_tc_status() == 0


@pytest.mark.parametrize("T", [17, 40, 64, 100])
def test_shares_of_a_few_token_product_are_added_up_by_the_kernel_that_reads_it_next(K, T):
    """A few-token product that cuts K into shares may leave them to the norm (a product into
    the fp32 stream) or to the norm / rotation / cache write (the q/k/v projection): the same
    bits as with the product's own second kernel.  Anything else that touches the output gets
    the product finished first."""
    H, Kin = 1024, 2048                    # 8 tiles of 128 outputs on 148 SMs: K is cut
    x, w = rnd((T, Kin), torch.bfloat16, 201).cuda(), rnd((H, Kin), torch.bfloat16, 202, 0.05).cuda()
    nw = (1 + rnd((H,), torch.float32, 203, 0.1)).cuda()
    base = rnd((T, H), torch.float32, 204).cuda()
    # 1. into the stream, then the norm
    want_x = base.clone()
    K.linear(want_x, x, w, accumulate=True)
    want_n = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    K.rmsnorm(want_n, want_x, nw, 1e-6)
    got_x = base.clone()
    K.linear(got_x, x, w, accumulate=True, defer=True)
    assert K._shares is not None, "this product was expected to be cut into shares"
    got_n = torch.empty_like(want_n)
    K.rmsnorm(got_n, got_x, nw, 1e-6)
    assert K._shares is None
    assert torch.equal(got_n, want_n) and torch.equal(got_x, want_x)
    # 2. the same, but the next reader is not the whole-stream norm: the product is finished first
    rows = torch.tensor([T - 1, 0, 3], dtype=torch.int32, device="cuda")
    got_x = base.clone()
    K.linear(got_x, x, w, accumulate=True, defer=True)
    some = torch.empty((3, H), dtype=torch.bfloat16, device="cuda")
    K.rmsnorm(some, got_x, nw, 1e-6, rows)
    assert K._shares is None and torch.equal(got_x, want_x) and torch.equal(some, want_n[rows.long()])
    got_x = base.clone()
    K.linear(got_x, x, w, accumulate=True, defer=True)
    K.flush_shares()
    assert torch.equal(got_x, want_x)
    # 3. a q/k/v projection, then norm, rotation and cache write
    nq, nkv, hd = 4, 2, 128
    lens = [T - 9, 9]
    pool, table, slots = make_paged(nkv, hd, [n + 70 for n in lens], torch.bfloat16, 205)
    pos = torch.cat([torch.arange(70, 70 + n) for n in lens]).to(torch.int32).cuda()
    slot = torch.cat([torch.full((n,), sl) for sl, n in zip(slots, lens)]).to(torch.int32).cuda()
    wq = rnd(((nq + 2 * nkv) * hd, Kin), torch.bfloat16, 206, 0.05).cuda()
    qw, kw = (1 + rnd((hd,), torch.float32, 207, 0.1)).cuda(), (1 + rnd((hd,), torch.float32, 208, 0.1)).cuda()
    inv = torch.pow(torch.tensor(10000.0), -torch.arange(0, hd, 2).float() / hd).cuda()
    outs = []
    for defer in (False, True):
        qkv = torch.empty((T, (nq + 2 * nkv) * hd), dtype=torch.bfloat16, device="cuda")
        p = pool.clone().cuda()
        K.linear(qkv, x, wq, defer=defer)
        assert (K._shares is not None) == defer
        K.qk_norm_rope_write(qkv, qw, kw, 1e-6, inv, hd, pos, slot, table.cuda(), p, nq, nkv, hd)
        assert K._shares is None
        outs.append((qkv[:, : nq * hd].clone(), p))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert K.status(sync=True) == 0


@pytest.mark.parametrize("T", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("H,Kin,N", [(1024, 2048, 3072), (1000, 520, 6144 + 16), (4096, 1024, 6144)])
def test_a_norm_between_two_streaming_products_without_a_kernel_of_its_own(K, T, H, Kin, N):
    """A streaming product into the stream that was told which norm follows leaves that norm's rows
    (but for their scale) and the rows' sums of squares; ``rmsnorm`` then launches nothing, and the
    streaming products that read its output scale their own sums.  Compared with the plain formula,
    with the three kernels run one after the other, and with the norm's output read by something else
    (it is then computed after all, the same bits as the norm's kernel).  One row of the stream is
    made a hundred times larger than the others, so that a scale taken from another row shows."""
    from zlm_b200.kernels import interleave_gate_up
    x, w = rnd((T, Kin), torch.bfloat16, 301).cuda(), rnd((H, Kin), torch.bfloat16, 302, 0.05).cuda()
    nw = (1 + rnd((H,), torch.float32, 303, 0.1)).cuda()
    base = rnd((T, H), torch.float32, 304)
    base[T // 2] *= 100.0
    base = base.cuda()
    w2 = rnd((N, H), torch.bfloat16, 305, 1.6 / H ** 0.5).cuda()      # outputs of the same size at every width
    eps = 1e-5
    # the three kernels one after the other
    want_x = base.clone()
    K.linear(want_x, x, w, accumulate=True)
    want_n = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    K.rmsnorm(want_n, want_x, nw, eps)
    before = K._launches
    # the plain formula on the same stream (fp64)
    xs = want_x.double()
    normed = xs * torch.rsqrt((xs * xs).mean(-1, keepdim=True) + eps) * nw.double()
    plain = normed @ w2.double().t()

    def lazily():
        got_x = base.clone()
        K.expect_norm(nw)
        K.linear(got_x, x, w, accumulate=True, defer=True)
        assert K._norm_halves is not None and torch.equal(got_x, want_x)
        got_n = torch.full((T, H), 7.0, dtype=torch.bfloat16, device="cuda")
        K.norm_output_read_by_products(True)
        n0 = K._launches
        K.rmsnorm(got_n, got_x, nw, eps)
        assert K._lazy is not None and K._launches == n0, "the norm was expected to be left to the products"
        return got_x, got_n

    # bf16 outputs, fp32 outputs (with the argmax's candidates), added into another stream, gate/up
    got_x, got_n = lazily()
    y = torch.empty((T, N), dtype=torch.bfloat16, device="cuda")
    K.linear(y, got_n, w2)
    close(y, plain, torch.bfloat16, atol=3e-2, rtol=2e-2)
    lg = torch.empty((T, N), dtype=torch.float32, device="cuda")
    K.linear(lg, got_n, w2)                                  # the same norm serves several products
    close(lg, plain, torch.float32, atol=2e-2, rtol=1e-2)    # (the bound is that of bf16 rows times weight)
    best = torch.empty(T, dtype=torch.int32, device="cuda")
    K.argmax(best, lg, fresh=True)                           # from the candidates that the product left
    assert torch.equal(best.cpu().long(), lg.argmax(-1).cpu())
    other = rnd((T, N), torch.float32, 306).cuda()
    acc = other.clone()
    K.linear(acc, got_n, w2, accumulate=True)
    close(acc, other.double() + plain, torch.float32, atol=2e-2, rtol=1e-2)
    I = N // 2
    act = torch.empty((T, I), dtype=torch.bfloat16, device="cuda")
    K.linear_swiglu(act, got_n, interleave_gate_up(w2[:I].contiguous(), w2[I:].contiguous()))
    g, u = plain[:, :I], plain[:, I:]
    close(act, (g / (1 + torch.exp(-g))) * u, torch.bfloat16, atol=3e-2, rtol=3e-2)
    assert K._lazy is not None
    # and against the three kernels: the scale is applied to the sum instead of to every term
    y3 = torch.empty((T, N), dtype=torch.float32, device="cuda")
    K.linear(y3, want_n, w2)
    close(lg, y3, torch.float32, atol=2e-2, rtol=1e-2)
    # something else reads the norm's output: it is computed first, the kernel's own bits
    copy = torch.empty((T, H // 2), dtype=torch.bfloat16, device="cuda")
    K.swiglu(copy, got_n)
    assert K._lazy is None and torch.equal(got_n, want_n)
    # the stream is written before anyone read the norm: forgotten, nothing launched for it
    got_x, got_n = lazily()
    n0 = K._launches
    K.linear(got_x, x, w, accumulate=True)
    assert K._lazy is None and K._launches == n0 + 1
    # without the arrangement's word on the readers, and for chosen rows, the norm runs as ever
    got_x = base.clone()
    K.expect_norm(nw)
    K.linear(got_x, x, w, accumulate=True, defer=True)
    got_n = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    K.rmsnorm(got_n, got_x, nw, eps)
    assert K._lazy is None and K._norm_halves is None and torch.equal(got_n, want_n)
    got_x = base.clone()
    K.expect_norm(nw)
    K.linear(got_x, x, w, accumulate=True, defer=True)
    K.norm_output_read_by_products(True)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
    some = torch.empty((2, H), dtype=torch.bfloat16, device="cuda")
    K.rmsnorm(some, got_x, nw, eps, rows)
    assert K._lazy is None and torch.equal(some, want_n[rows.long()])
    # another norm's weight than the one announced: as ever
    got_x = base.clone()
    K.expect_norm(nw)
    K.linear(got_x, x, w, accumulate=True, defer=True)
    K.norm_output_read_by_products(True)
    nw2 = nw.clone()
    K.rmsnorm(got_n, got_x, nw2, eps)
    assert K._lazy is None and torch.equal(got_n, want_n)
    assert K.status(sync=True) == 0


@pytest.mark.parametrize("T,nq,nkv,hd,Kin,norm,rope,width", [
    (500, 4, 2, 128, 256, True, True, 0), (700, 6, 3, 64, 192, True, True, 0), (390, 8, 0, 128, 128, True, True, 0),
    (450, 3, 1, 32, 96, False, True, 0), (600, 4, 4, 128, 320, True, False, 0), (1100, 5, 1, 128, 512, True, True, 128),
    (513, 16, 8, 128, 1024, True, True, 256)])
def test_projection_with_norm_rotation_and_cache_write_in_its_epilogue(K, T, nq, nkv, hd, Kin, norm, rope, width):
    """The fused q/k/v projection (norm, rotation and cache write in the tcgen05 product's
    epilogue) against the plain product followed by the plain norm / rotation / write: q, and
    every key and value where the tokens' positions put them in the paged pool; pages that
    no token of the step writes must keep their content.  Two sequences with a cached prefix
    each, so that positions do not start at zero and slots differ."""
    dt = torch.bfloat16
    N = (nq + 2 * nkv) * hd
    x = rnd((T, Kin), dt, 70)
    w = rnd((N, Kin), dt, 71, scale=0.3)
    q_w = (1.0 + rnd((hd,), torch.float32, 72, scale=0.1)) if norm else None
    k_w = (1.0 + rnd((hd,), torch.float32, 73, scale=0.1)) if (norm and nkv) else None
    half = hd // 2
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / hd).float()
    starts, news = [70, 3], [T - T // 3, T // 3]
    lens = [s + n for s, n in zip(starts, news)]
    pool, table, slots = make_paged(max(nkv, 1), hd, lens, dt, 74, n_pages=sum((n + PAGE - 1) // PAGE for n in lens) + 4)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, news)]).to(torch.int32)
    slot = torch.cat([torch.full((n,), sl) for sl, n in zip(slots, news)]).to(torch.int32)
    if not K.qkv_rope_supported(x.cuda(), w.cuda(), nq, nkv, hd, hd if rope else 0):
        pytest.fail("the fused projection refuses a shape it is documented to take")
    # plain: product (rounded to bf16 as the unfused path stores it), then norm / rotation / write
    P = PlainKernels()
    qkv = torch.empty((T, N), dtype=dt)
    P.linear(qkv, x, w)
    want_pool = pool.clone()
    P.qk_norm_rope_write(qkv, q_w, k_w, 1e-6, inv if rope else None, hd if rope else 0, pos, slot,
                         table if nkv else None, want_pool if nkv else None, nq, nkv, hd)
    got_pool = pool.clone().cuda()
    q = torch.empty((T, nq * hd), dtype=dt, device="cuda")
    cs = None
    if rope:
        cs = torch.empty((2, half, T), dtype=torch.float32, device="cuda")
        K.rope_table(cs, inv.cuda(), hd, pos.cuda())
        a = inv[:, None] * pos.float()[None, :]
        torch.testing.assert_close(cs.cpu(), torch.stack([torch.cos(a), torch.sin(a)]), atol=2e-6, rtol=1e-5)
    K.set_gemm_form("pair" if width else None, width)
    try:
        K.linear_qkv_rope(q, x.cuda(), w.cuda(), None if q_w is None else q_w.cuda(), None if k_w is None else k_w.cuda(),
                          1e-6, cs, pos.cuda(), slot.cuda(), table.cuda() if nkv else None, got_pool if nkv else None,
                          nq, nkv, hd)
    finally:
        K.set_gemm_form(None, 0)
    assert K.gemm_tc_status() == 0
    close(q, qkv[:, : nq * hd], dt, atol=3e-2, rtol=3e-2)
    if nkv:
        close(got_pool, want_pool, dt, atol=3e-2, rtol=3e-2)
        written = torch.zeros(pool.shape[0], dtype=torch.bool)
        for p_, s_ in zip(pos.tolist(), slot.tolist()):
            written[int(table[s_, p_ // PAGE])] = True
        assert torch.equal(got_pool.cpu()[~written], pool[~written]), "a page that no token writes was touched"


@pytest.mark.parametrize("R,H,w_dtype", [(512, 64, "float32"), (700, 1000, "bfloat16"), (1500, 4096, "float32"),
                                         (600, 5120, "float32"), (2100, 8192, "bfloat16"), (513, 2052, "float32")])
def test_rmsnorm_of_many_rows(K, R, H, w_dtype):
    """Steps of 512 rows and more with bf16 output run the row-walking kernel (a block takes rows
    r, r + blocks, ...; more rows than blocks here, and a last round that is not full); rows of
    very different sizes, so that a row normed with another row's sum shows."""
    x = rnd((R, H), torch.float32, 90) * (0.01 + torch.arange(R, dtype=torch.float32)[:, None] % 37)
    w = (1 + rnd((H,), torch.float32, 91, 0.1)).to(DT[w_dtype])
    assert K.lib.zlm_rmsnorm_walks_rows(1, R, H, 0) == 1
    want = torch.empty(R, H, dtype=torch.bfloat16)
    PlainKernels().rmsnorm(want, x, w, 1e-6)
    got = torch.empty(R, H, dtype=torch.bfloat16, device="cuda")
    K.rmsnorm(got, x.cuda(), w.cuda(), 1e-6)
    close(got, want, torch.bfloat16, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("T,V,Kin", [(1, 1000, 64), (8, 151936, 128), (5, 50021, 72), (3, 40, 200)])
def test_argmax_from_the_candidates_the_head_product_leaves(K, T, V, Kin):
    """The few-token product with fp32 output leaves every block's best (value, index) per token;
    ``argmax(..., fresh=True)`` picks among them.  Ties (equal rows of the weight) must go to the
    lowest index, in one block and across blocks; a later write into the same tensor by another
    path must not be answered from stale candidates."""
    x = rnd((T, Kin), torch.bfloat16, 95)
    w = rnd((V, Kin), torch.bfloat16, 96, scale=0.3)
    w[V - 3] = w[7] = w[min(V - 1, 16 + 7)] = w[2] * 3.0           # a tie of four; which row wins differs by token
    logits = torch.empty((T, V), dtype=torch.float32, device="cuda")
    K.linear(logits, x.cuda(), w.cuda())
    got = torch.empty(T, dtype=torch.int32, device="cuda")
    K.argmax(got, logits, fresh=True)
    plain = torch.empty(T, dtype=torch.int32, device="cuda")
    K.argmax(plain, logits)                                        # the two-kernel path over the logits themselves
    want = torch.empty(T, dtype=torch.int32)
    PlainKernels().argmax(want, logits.cpu())
    assert got.cpu().tolist() == plain.cpu().tolist() == want.tolist()
    # the tensor is written again by something else: fresh candidates there are none
    logits.copy_(torch.flip(logits, dims=[1]))
    K.linear(logits, x.cuda(), w.cuda(), impl="mma")
    logits[:, V // 2] = 1e9
    K.argmax(got, logits, fresh=True)
    assert got.cpu().tolist() == [V // 2] * T
