"""The persistent decode kernel: each operation of its program alone against the
stand-alone kernel of the same name (bit for bit: it is built to add in the same
order), whole decode steps against the same steps launched kernel by kernel (bit
for bit) and against the plain implementation, and what it refuses."""
import pytest
import torch

from helpers import SHARP, assert_close, make_model, plain_logits, random_prompts, reference_tensors

pytestmark = pytest.mark.gpu


def kernels():
    from zlm_b200.kernels import get_kernels
    return get_kernels()


def run_ops(record):
    """Records operations with ``record(recorder)`` and runs them as one program."""
    from zlm_b200.engine.stream import StepRecorder, StreamProgram, stream_blocks
    k = kernels()
    blocks = stream_blocks(k)
    assert blocks > 0, "the persistent decode kernel cannot run on this device"
    rec = StepRecorder(k, blocks)
    record(rec)
    prog = StreamProgram(k, rec, "cuda:0")
    prog.run()
    torch.cuda.synchronize()
    assert k.stream_status() == 0
    return prog


@pytest.mark.parametrize("T,N,K", [(1, 64, 64), (3, 100, 72), (8, 1000, 520), (5, 4096, 4096), (8, 148 * 16 + 5, 1032),
                                   (2, 7, 4104), (8, 333, 12288)])
@pytest.mark.parametrize("mode", ["store", "accumulate", "store_f32"])
def test_product_equals_the_gemv(T, N, K, mode):
    k = kernels()
    g = torch.Generator(device="cuda").manual_seed(T * 1000 + N + K)
    x = torch.randn(T, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    if mode == "store":
        want = torch.zeros(T, N, device="cuda", dtype=torch.bfloat16)
        got = torch.zeros_like(want)
        acc = False
    else:
        base = torch.randn(T, N, device="cuda", generator=g)
        want, got = base.clone(), base.clone()
        acc = mode == "accumulate"
    k.linear(want, x, w, accumulate=acc, impl="gemv")
    run_ops(lambda r: r.linear(got, x, w, accumulate=acc))
    assert torch.equal(got, want), f"max diff {(got.float() - want.float()).abs().max().item()}"
    # and it is the product: against fp32 arithmetic on the same bf16 values
    ref = x.float() @ w.float().T
    if mode != "store":
        ref = ref + (base if acc else 0)
    torch.testing.assert_close(got.float(), ref, atol=2e-2 * max(1.0, ref.abs().max().item()), rtol=2e-2)


@pytest.mark.parametrize("T,I,K", [(1, 16, 64), (4, 104, 72), (8, 12288, 4096), (7, 1000, 520)])
def test_fused_gate_up_equals_the_gemv(T, I, K):
    from zlm_b200.kernels import interleave_gate_up
    k = kernels()
    g = torch.Generator(device="cuda").manual_seed(I + K)
    x = torch.randn(T, K, device="cuda", generator=g).bfloat16()
    gate = (torch.randn(I, K, device="cuda", generator=g) * 0.05).bfloat16()
    up = (torch.randn(I, K, device="cuda", generator=g) * 0.05).bfloat16()
    w = interleave_gate_up(gate, up)
    want = torch.zeros(T, I, device="cuda", dtype=torch.bfloat16)
    got = torch.zeros_like(want)
    k.linear_swiglu(want, x, w, impl="gemv")
    run_ops(lambda r: r.linear_swiglu(got, x, w))
    assert torch.equal(got, want)


def test_strided_operands_and_a_chain_of_products():
    """A product that reads a column view and one that reads what the first wrote: the
    barrier between them orders the blocks."""
    k = kernels()
    g = torch.Generator(device="cuda").manual_seed(5)
    big = torch.randn(6, 1024, device="cuda", generator=g).bfloat16()
    x = big[:, 256:768]                                   # row stride 1024, 512 columns
    w1 = (torch.randn(2000, 512, device="cuda", generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(300, 2000, device="cuda", generator=g) * 0.05).bfloat16()
    mid_w = torch.zeros(6, 2000, device="cuda", dtype=torch.bfloat16)
    mid_g = torch.zeros_like(mid_w)
    out_w = torch.zeros(6, 300, device="cuda")
    out_g = torch.zeros_like(out_w)
    k.linear(mid_w, x, w1, impl="gemv")
    k.linear(out_w, mid_w, w2, impl="gemv")

    def rec(r):
        r.linear(mid_g, x, w1)
        r.linear(out_g, mid_g, w2)
    for _ in range(3):                                    # a program can be run again and again
        out_g.zero_()
        prog = run_ops(rec)
    assert prog.n_ops == 2
    assert torch.equal(mid_g, mid_w) and torch.equal(out_g, out_w)


def test_norm_rope_attention_ops_equal_their_kernels():
    """rmsnorm, q/k norm + rotation + cache write, attention with its combine: one program
    against the three stand-alone kernels on the same inputs."""
    from test_kernels_gpu import FakePlan, make_paged
    from zlm_b200.engine.stream import stream_blocks
    k = kernels()
    nq, nkv, hd, H = 6, 2, 48, 200
    R = 5
    lens = [70, 3, 129, 64, 200]
    g = torch.Generator(device="cuda").manual_seed(11)
    hidden = torch.randn(R, H, device="cuda", generator=g)
    norm_w = 1 + 0.1 * torch.randn(H, device="cuda", generator=g)
    qn = (1 + 0.1 * torch.randn(hd, device="cuda", generator=g))
    kn = (1 + 0.1 * torch.randn(hd, device="cuda", generator=g))
    inv_freq = (10000.0 ** (-torch.arange(0, hd, 2, device="cuda").float() / hd)).contiguous()
    pool, table, slots = make_paged(nkv, hd, lens, torch.bfloat16, 3)
    pool, table = pool.cuda(), table.cuda()
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    slot = torch.tensor(slots, dtype=torch.int32, device="cuda")
    qkv0 = torch.randn(R, (nq + 2 * nkv) * hd, device="cuda", generator=g).bfloat16()
    plan = FakePlan(4)
    plan.attention_blocks = stream_blocks(k)
    outs = []
    for which in ("kernels", "program"):
        pool_c, qkv = pool.clone(), qkv0.clone()
        normed = torch.zeros(R, H, device="cuda", dtype=torch.bfloat16)
        out = torch.zeros(R, nq * hd, device="cuda", dtype=torch.bfloat16)

        def ops(r):
            r.rmsnorm(normed, hidden, norm_w, 1e-5)
            r.qk_norm_rope_write(qkv, qn, kn, 1e-6, inv_freq, hd, pos, slot, table, pool_c, nq, nkv, hd)
            r.attention(out, qkv[:, : nq * hd], pool_c, table, pos, slot, nq, nkv, hd, hd ** -0.5, 0, plan)
        if which == "kernels":
            ops(k)
        else:
            run_ops(ops)
        torch.cuda.synchronize()
        outs.append((normed, qkv, pool_c, out))
    for a, b, what in zip(outs[0], outs[1], ("rmsnorm", "q after rotation", "cache", "attention")):
        assert torch.equal(a, b), what


def _decode_logits(eng, prompts, steps, tokens_seed):
    """Prefill, then ``steps`` decode steps of fixed tokens through the decode runner; the
    logits of every step."""
    from zlm_b200 import StepEntry
    from zlm_b200.sampling import SamplingParams
    slots = [eng.new_sequence() for _ in prompts]
    eng.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
    g = torch.Generator().manual_seed(tokens_seed)
    out, fed = [], []
    for _ in range(steps):
        toks = torch.randint(0, eng.spec.vocab_size, (len(prompts),), generator=g).tolist()
        eng.decoder.step(slots, toks, SamplingParams())
        out.append(eng.decoder.last_logits.clone())
        fed.append(toks)
    for s in slots:
        eng.release(s)
    return out, fed


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_steps_equal_the_kernel_by_kernel_steps(tmp_path, name):
    """The same decode steps as one program and as a CUDA graph of stand-alone kernels: the
    logits are the same bits (with the attention cut the same way in both)."""
    from zlm_b200 import Engine
    folder, cfg, tensors = make_model(tmp_path, name, seed=3, sharp=SHARP["bfloat16"])
    eng = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=4096)
    assert eng.decoder.can_stream and not eng.decoder.use_stream     # it has to be asked for
    eng.decoder.use_stream = True
    eng.decoder.attention_blocks = eng.decoder.stream_blocks
    lengths = [5, 70, 1, 33, 64, 100, 17][: 7 if name != "A" else 5]
    lengths = [min(n, cfg.max_position_embeddings - 40) for n in lengths]
    prompts = random_prompts(cfg.vocab_size, lengths, seed=4)
    got, _ = _decode_logits(eng, prompts, 30, 9)
    assert eng.rt.k.stream_status() == 0
    assert eng.decoder.launches_per_step <= 4, "a streamed step is the program and the choice of tokens"
    eng.decoder.use_stream = False
    want, _ = _decode_logits(eng, prompts, 30, 9)
    for i, (a, b) in enumerate(zip(got, want)):
        assert torch.equal(a, b), f"step {i}: max diff {(a - b).abs().max().item()}"
    eng.cache.check()


@pytest.mark.parametrize("name", ["B", "C"])
def test_steps_against_the_plain_implementation(tmp_path, name):
    """Decode steps of an unequal batch through the persistent kernel (its own attention
    cut), every step's logits against whole sequences through the plain implementation."""
    from zlm_b200 import Engine
    folder, cfg, tensors = make_model(tmp_path, name, seed=5, sharp=SHARP["bfloat16"])
    ref = reference_tensors(tensors, "bfloat16")
    eng = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=2048)
    eng.decoder.use_stream = True
    lengths = [3, 60, 64, 1, 90, 31, 7, 128]
    prompts = random_prompts(cfg.vocab_size, lengths, seed=6)
    steps = 12
    got, fed = _decode_logits(eng, prompts, steps, 2)
    assert eng.rt.k.stream_status() == 0
    for r, p in enumerate(prompts):
        seq = list(p) + [fed[i][r] for i in range(steps)]
        want = plain_logits(ref, cfg, seq)[len(p):]
        mine = torch.stack([got[i][r] for i in range(steps)])
        assert_close(mine, want, "bfloat16", f"{name} row {r}")


def test_what_is_not_a_program_falls_back(tmp_path):
    """More than 8 rows, or 32-bit: the step runs kernel by kernel and gives the same
    results as before; nothing is refused."""
    from zlm_b200 import Engine
    folder, cfg, tensors = make_model(tmp_path, "B", seed=3, sharp=1.0)
    eng = Engine.from_pretrained(folder, dtype="float32", max_tokens=2048)
    assert not eng.decoder.can_stream
    eng = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=2048)
    eng.decoder.use_stream = True
    prompts = random_prompts(cfg.vocab_size, [4] * 9, seed=1)
    got, _ = _decode_logits(eng, prompts, 2, 3)
    assert eng.decoder.launches_per_step > 4
    assert got[0].shape == (9, cfg.vocab_size)


def test_the_recorder_refuses_what_the_kernel_does_not_take():
    from zlm_b200.engine.stream import NotStreamable, StepRecorder
    k = kernels()
    r = StepRecorder(k, 148)
    x = torch.zeros(9, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(32, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NotStreamable):
        r.linear(torch.zeros(9, 32, device="cuda", dtype=torch.bfloat16), x, w)
    with pytest.raises(NotStreamable):
        r.swiglu(x, x)
    with pytest.raises(NotStreamable):
        r.linear(torch.zeros(2, 32, device="cuda"), torch.zeros(2, 64, device="cuda"), torch.zeros(32, 64, device="cuda"))
