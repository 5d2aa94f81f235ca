"""The engine on the GPU against the plain implementation, in 32-bit and in
bfloat16: whole requests, the last 32 tokens one by one, batches of unequal
lengths one after another (slots and pages are used again), long decoding, and
the first tokens of a sequence."""
import pytest
import torch

from helpers import SHARP, assert_close, make_model, plain_logits, random_prompts, reference_tensors

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C"]


def build(tmp_path, name, dtype, max_tokens=2048, **kw):
    from zlm_b200 import Engine
    folder, cfg, tensors = make_model(tmp_path, name, seed=3, sharp=SHARP[dtype])
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=max_tokens, **kw)
    return eng, cfg, reference_tensors(tensors, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests_alone(tmp_path, name, dtype):
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    maxlen = min(cfg.max_position_embeddings, 200)
    for i, n in enumerate([1, 5, 64, 65, maxlen]):
        (p,) = random_prompts(cfg.vocab_size, [n], seed=10 + i)
        s = eng.new_sequence()
        got = eng.step([StepEntry(s, p, list(range(n)))]).clone()
        eng.release(s)
        assert_close(got, plain_logits(ref, cfg, p), dtype, f"{name} whole len {n}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_one_by_one(tmp_path, name, dtype):
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    n = min(cfg.max_position_embeddings, 150)
    (p,) = random_prompts(cfg.vocab_size, [n], seed=21)
    want = plain_logits(ref, cfg, p)
    s = eng.new_sequence()
    head = n - 32
    got = [eng.step([StepEntry(s, p[:head], [head - 1])]).clone()]
    for t in range(head, n):
        got.append(eng.step([StepEntry(s, [p[t]], [0])]).clone())
    got = torch.cat(got)
    assert_close(got, want[head - 1:], dtype, f"{name} last 32 one by one")
    eng.release(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_reuse_slots(tmp_path, name, dtype):
    """Batches of unequal prompts, each decoded for a different number of steps so
    that short requests end early; three batches in a cache that holds little more
    than one, so that slots and pages come back and are used again."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype, max_tokens=64 * 8, max_batch=4)
    cap = cfg.max_position_embeddings
    for b in range(3):
        lens = [min(cap - 12, l) for l in ([3, 70, 17, 1] if b % 2 == 0 else [65, 2, 100])]
        extra = [4, 9, 1, 12][:len(lens)]
        full = random_prompts(cfg.vocab_size, [l + e for l, e in zip(lens, extra)], seed=30 + b)
        want = [plain_logits(ref, cfg, p) for p in full]
        slots = [eng.new_sequence() for _ in full]
        got = eng.step([StepEntry(s, p[:l], [l - 1]) for s, p, l in zip(slots, full, lens)]).clone()
        for j in range(len(full)):
            assert_close(got[j], want[j][lens[j] - 1], dtype, f"{name} batch {b} row {j} prompt end")
        live = list(range(len(full)))
        for step in range(max(extra)):
            live = [j for j in live if step < extra[j]]
            ended = [j for j in range(len(full)) if step == extra[j]]
            for j in ended:
                eng.release(slots[j])
            got = eng.step([StepEntry(slots[j], [full[j][lens[j] + step]], [0]) for j in live]).clone()
            for r, j in enumerate(live):
                assert_close(got[r], want[j][lens[j] + step], dtype,
                             f"{name} batch {b} row {j} decode step {step}")
        for j in range(len(full)):
            if extra[j] >= max(extra):
                eng.release(slots[j])
        eng.cache.check()
    assert eng.cache.slots.held == 0 and all(g.pages.held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decode_far_keys(tmp_path, dtype):
    """600 tokens through configuration C (full and windowed layers): a short
    prompt, then one token at a time across many page and window edges."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, "C", dtype)
    n = 600
    (p,) = random_prompts(cfg.vocab_size, [n], seed=44)
    want = plain_logits(ref, cfg, p)
    s = eng.new_sequence()
    got = [eng.step([StepEntry(s, p[:7], list(range(7)))]).clone()]
    for t in range(7, n):
        got.append(eng.step([StepEntry(s, [p[t]], [0])]).clone())
    assert_close(torch.cat(got), want, dtype, "C long decode")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_chunks(tmp_path, dtype):
    """The first tokens one by one from an empty cache, then chunks of odd sizes."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, "B", dtype)
    (p,) = random_prompts(cfg.vocab_size, [90], seed=51)
    want = plain_logits(ref, cfg, p)
    s = eng.new_sequence()
    got, t = [], 0
    for n in [1, 1, 1, 2, 3, 9, 47, 1, 25]:
        got.append(eng.step([StepEntry(s, p[t:t + n], list(range(n)))]).clone())
        t += n
    assert t == 90
    assert_close(torch.cat(got), want, dtype, "B chunks")


def test_fp32_cuttings_are_bitwise_equal(tmp_path):
    """In 32-bit the order of every sum depends only on a token's own sequence, so
    whole, one by one and batched runs give the same bits."""
    from zlm_b200 import StepEntry
    eng, cfg, _ = build(tmp_path, "C", "float32")
    ps = random_prompts(cfg.vocab_size, [130, 40], seed=61)
    s = eng.new_sequence()
    whole = eng.step([StepEntry(s, ps[0], list(range(130)))]).clone()
    eng.release(s)
    a, b = eng.new_sequence(), eng.new_sequence()
    got = [eng.step([StepEntry(b, ps[1][:20], []), StepEntry(a, ps[0][:100], list(range(100)))]).clone()]
    for t in range(100, 130):
        ents = [StepEntry(a, [ps[0][t]], [0])]
        if t < 120:
            ents.insert(0, StepEntry(b, [ps[1][t - 80]], []))
        got.append(eng.step(ents).clone())
    assert torch.equal(torch.cat(got), whole)


@pytest.mark.parametrize("name", NAMES)
def test_decode_steps_leave_the_norms_to_the_products(tmp_path, name):
    """In a bfloat16 step of a few tokens every norm but the first and the last has a streaming
    product before it and streaming products after it, and launches nothing: two launches fewer a
    layer than with the norms' own kernels, the same logits within rounding (both are compared
    with the plain implementation by the other tests; here with each other, at steps of 1, 5 and
    16 tokens), and nothing of it in a step of 17 tokens, which the other products take."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, "bfloat16")
    k = eng.rt.k
    L = cfg.num_hidden_layers
    (p,) = random_prompts(cfg.vocab_size, [60], seed=33)
    want = plain_logits(ref, cfg, p)
    for chunk in (1, 5, 16, 17):
        got, launches = {}, {}
        for lazy in (True, False):
            k.lazy_norms = lazy
            s = eng.new_sequence()
            eng.step([StepEntry(s, p[:20], [])])
            before = k._launches
            got[lazy] = eng.step([StepEntry(s, p[20:20 + chunk], list(range(chunk)))]).clone()
            launches[lazy] = k._launches - before
            eng.release(s)
        k.lazy_norms = True
        assert launches[False] - launches[True] == (2 * L - 1 if chunk <= 16 else 0), (chunk, launches)
        assert_close(got[True], want[20:20 + chunk], "bfloat16", f"{name} norms left to the products, {chunk} tokens")
        assert_close(got[True], got[False], "bfloat16", f"{name} with and without the norms' kernels, {chunk} tokens")
    assert k._lazy is None and k._norm_halves is None and k._norm_hint is None
