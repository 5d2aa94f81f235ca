"""The engine at the layer sizes of Qwen3-8B (width 4096, 32 query heads over 8 kv
heads of size 128, feed-forward 12288), of Qwen3-0.6B (width 1024, 16 over 8 heads of
128, so that heads x size is not the width; feed-forward 3072, tied head) and of
Qwen3-32B (width 5120, 64 over 8 heads: groups of 8; feed-forward 25600), one or two
layers each and a reduced vocabulary so that the plain implementation finishes in seconds:
every kernel at the shapes the benchmark runs, in 32-bit and in bfloat16, whole prompt,
chunks and decode."""
import pytest
import torch

from helpers import assert_close, plain_logits, random_prompts, reference_tensors

pytestmark = pytest.mark.gpu

# Sums here run over 4096 to 12288 terms instead of the tiny models' 64 to 160, and the logits
# are an order of magnitude larger: the rounding of a 32-bit sum grows with the square root of
# its length, so the element-wise bound of the 32-bit comparison is ten times the tiny models'.
# In bfloat16 the rows keep the tiny models' bound (2% of a row's norm); the element-wise bound
# is there to catch single wild values, and among 2.4 million logits of standard deviation 1.3
# the largest rounding error is several times the typical one: 0.15.
TOL_8B = {"float32": dict(atol=2e-4, rtol=1e-4, row=1e-4), "bfloat16": dict(atol=0.15, rtol=2e-2, row=2e-2)}

SIZES_8B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 8192, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 4096, "hidden_act": "silu",
}


SIZES = {
    "8B": SIZES_8B,
    "0.6B": dict(SIZES_8B, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072,
                 tie_word_embeddings=True, vocab_size=8200),
    "32B": dict(SIZES_8B, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600,
                vocab_size=4104, num_hidden_layers=1),
}


@pytest.fixture(scope="module", params=["8B", "0.6B", "32B"])
def model(request):
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    from zlm_b200.weights import random_tensors
    cfg = config_from_dict(SIZES[request.param])
    tensors = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 5, "cpu", torch.float32)
    (prompt,) = random_prompts(cfg.vocab_size, [300], seed=9)
    want = {dt: plain_logits(reference_tensors(tensors, dt), cfg, prompt) for dt in ("float32", "bfloat16")}
    return cfg, tensors, prompt, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sizes_of_the_benchmark(model, dtype):
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.engine import parse_dtype
    from zlm_b200.sampling import SamplingParams
    from zlm_b200.weights.loader import target_dtype
    from zlm_b200.parts.model import DecoderModel
    cfg, tensors, prompt, want = model
    dt = parse_dtype(dtype)
    specs = DecoderModel(cfg.to_model_spec()).param_specs()
    dev = {n: t.to("cuda").to(target_dtype(specs[n], t.dtype, dt)) for n, t in tensors.items()}
    eng = Engine(cfg, dev, dt, "cuda:0", max_tokens=2048, max_batch=4)
    ref = want[dtype]
    # whole (tcgen05 products and tiled attention in bfloat16)
    s = eng.new_sequence()
    got = eng.step([StepEntry(s, prompt, list(range(300)))]).clone()
    assert_close(got, ref, dtype, f"layer sizes whole {dtype}", TOL_8B[dtype])
    eng.release(s)
    # a long chunk, a short chunk (the few-token kernels), then single tokens through the decode path
    s = eng.new_sequence()
    parts = [eng.step([StepEntry(s, prompt[:200], list(range(200)))]).clone(),
             eng.step([StepEntry(s, prompt[200:240], list(range(40)))]).clone(),
             eng.step([StepEntry(s, prompt[240:250], list(range(10)))]).clone()]
    assert_close(torch.cat(parts), ref[:250], dtype, f"layer sizes chunks {dtype}", TOL_8B[dtype])
    for t in range(250, 262):
        eng.decoder.step([s], [prompt[t]], SamplingParams())
        assert_close(eng.decoder.last_logits.clone(), ref[t:t + 1], dtype, f"layer sizes decode {t} {dtype}", TOL_8B[dtype])
    if dtype == "bfloat16":
        assert eng.rt.k.gemm_tc_status() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_sequences_chunks_and_reused_slots_at_head_size_128(dtype):
    """Three sequences of unequal lengths prefilled as one step, one of them continued by a
    chunk while the others decode... (the tcgen05 flash attention with a cached prefix and
    the split-KV decode attention at head size 128 inside one model), the shortest ending
    early; then a second batch in the slots and pages the first gave back."""
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.engine import parse_dtype
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    from zlm_b200.sampling import SamplingParams
    from zlm_b200.weights import random_tensors
    from zlm_b200.weights.loader import target_dtype
    cfg = config_from_dict(dict(SIZES_8B, num_hidden_layers=1, vocab_size=2048))
    tensors = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 6, "cpu", torch.float32)
    ref_t = reference_tensors(tensors, dtype)
    dt = parse_dtype(dtype)
    specs = DecoderModel(cfg.to_model_spec()).param_specs()
    dev = {n: t.to("cuda").to(target_dtype(specs[n], t.dtype, dt)) for n, t in tensors.items()}
    eng = Engine(cfg, dev, dt, "cuda:0", max_tokens=64 * 12, max_batch=3)
    tol = TOL_8B[dtype]
    for b, lens in enumerate(([200, 77, 129], [64, 260, 1])):
        full = random_prompts(cfg.vocab_size, [n + 8 for n in lens], seed=20 + b)
        want = [plain_logits(ref_t, cfg, p) for p in full]
        slots = [eng.new_sequence() for _ in full]
        assert sorted(slots) == [0, 1, 2]
        # unequal prompts as one step; the longest is cut: its first part now, the rest as a chunk
        cut = [min(n, 130) for n in lens]
        got = eng.step([StepEntry(s, p[:c], [c - 1]) for s, p, c in zip(slots, full, cut)]).clone()
        for j in range(3):
            assert_close(got[j], want[j][cut[j] - 1], dtype, f"batch {b} row {j} first part", tol)
        j_long = max(range(3), key=lambda j: lens[j])
        rest = list(range(cut[j_long], lens[j_long]))
        got = eng.step([StepEntry(slots[j_long], [full[j_long][t] for t in rest], list(range(len(rest))))]).clone()
        assert_close(got, want[j_long][rest[0]:rest[-1] + 1], dtype, f"batch {b} continued chunk", tol)
        # decode: all three, then without the shortest (it ends early and gives its slot back)
        j_short = min(range(3), key=lambda j: lens[j])
        for step in range(8):
            live = [j for j in range(3) if not (j == j_short and step >= 3)]
            if step == 3:
                eng.release(slots[j_short])
            eng.decoder.step([slots[j] for j in live], [full[j][lens[j] + step] for j in live], SamplingParams())
            got = eng.decoder.last_logits[:len(live)].clone()
            for r, j in enumerate(live):
                assert_close(got[r], want[j][lens[j] + step], dtype, f"batch {b} row {j} decode {step}", tol)
        for j in range(3):
            if j != j_short:
                eng.release(slots[j])
        eng.cache.check()
    assert eng.cache.slots.held == 0
    if dtype == "bfloat16":
        assert eng.rt.k.gemm_tc_status() == 0


@pytest.mark.parametrize("sizes", ["8B", "0.6B"])
def test_many_token_steps_through_the_fused_projection(sizes):
    """Steps of more than 384 tokens, where the q/k/v projection carries norm, rotation and
    cache write in its epilogue: a whole prompt, then two sequences of unequal lengths as
    one step on top of cached prefixes, then decode steps that read what those epilogues
    wrote into the cache."""
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    from zlm_b200.sampling import SamplingParams
    from zlm_b200.weights import random_tensors
    from zlm_b200.weights.loader import target_dtype
    dtype = "bfloat16"
    cfg = config_from_dict(dict(SIZES[sizes], num_hidden_layers=1, vocab_size=2048))
    tensors = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 8, "cpu", torch.float32)
    ref_t = reference_tensors(tensors, dtype)
    specs = DecoderModel(cfg.to_model_spec()).param_specs()
    dev = {n: t.to("cuda").to(target_dtype(specs[n], t.dtype, torch.bfloat16)) for n, t in tensors.items()}
    eng = Engine(cfg, dev, torch.bfloat16, "cuda:0", max_tokens=64 * 24, max_batch=3)
    fused = []
    real = eng.rt.k.linear_qkv_rope
    eng.rt.k.linear_qkv_rope = lambda *a, **kw: (fused.append(a[1].shape[0]), real(*a, **kw))[1]
    try:
        tol = TOL_8B[dtype]
        full = random_prompts(cfg.vocab_size, [460, 330, 270], seed=33)
        want = [plain_logits(ref_t, cfg, p) for p in full]
        s0 = eng.new_sequence()
        got = eng.step([StepEntry(s0, full[0][:450], [0, 200, 449])]).clone()
        assert_close(got, want[0][[0, 200, 449]], dtype, "whole prompt of 450 tokens", tol)
        s1, s2 = eng.new_sequence(), eng.new_sequence()
        eng.step([StepEntry(s1, full[1][:20], []), StepEntry(s2, full[2][:7], [])])
        got = eng.step([StepEntry(s1, full[1][20:320], [299]), StepEntry(s2, full[2][7:260], [0, 252])]).clone()
        assert_close(got[0], want[1][319], dtype, "second sequence, end of its chunk", tol)
        assert_close(got[1:], want[2][[7, 259]], dtype, "third sequence, first and last of its chunk", tol)
        assert fused == [450, 553], f"the fused projection ran for steps of {fused} tokens"
        for step in range(4):
            eng.decoder.step([s0, s1, s2], [full[0][450 + step], full[1][320 + step], full[2][260 + step]], SamplingParams())
            got = eng.decoder.last_logits[:3].clone()
            for r, (j, base) in enumerate(((0, 450), (1, 320), (2, 260))):
                assert_close(got[r], want[j][base + step], dtype, f"decode {step} of sequence {j}", tol)
        assert eng.rt.k.gemm_tc_status() == 0
    finally:
        eng.rt.k.linear_qkv_rope = real
