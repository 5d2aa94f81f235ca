"""Generation through the Python entry point and the command line against the
plain implementation: greedy tokens, stop tokens, more requests than fit at
once, and temperature sampling that does not depend on the batch."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as P
from helpers import ROOT, make_model, random_prompts, reference_tensors
from tiny_configs import plain_sizes

pytestmark = pytest.mark.gpu


def safe_prefix(tensors, cfg, prompt, out, eps):
    """How many leading tokens of the plain greedy run were chosen with a margin over
    the runner-up larger than eps, so that rounding cannot have flipped them."""
    ids = list(prompt)
    for n, tok in enumerate(out):
        l = P.forward(tensors, plain_sizes(cfg), ids)[-1]
        top = torch.topk(l, 2).values
        if float(top[0] - top[1]) < eps:
            return n
        ids.append(tok)
    return len(out)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "float32"), ("B", "bfloat16")])
def test_greedy_generation_matches_plain(tmp_path, name, dtype):
    from zlm_b200 import Engine
    folder, cfg, tensors = make_model(tmp_path, name, seed=11)
    ref = reference_tensors(tensors, dtype)
    lens = [5, 9, 13, 70, 1, 30, 2]
    prompts = random_prompts(cfg.vocab_size, lens, seed=5)
    # a cache that holds three of the seven requests at a time: batches follow one another
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=64 * 4, max_batch=3)
    res = eng.generate(prompts, max_tokens=8)
    assert res.stats.batches >= 3 and eng.cache.slots.held == 0
    eng.cache.check()
    eps = 1e-4 if dtype == "float32" else 2e-2
    checked = 0
    for p, got in zip(prompts, res.tokens):
        assert len(got) == 8
        want = P.greedy_generate(ref, plain_sizes(cfg), p, 8)
        n = safe_prefix(ref, cfg, p, want, eps)
        assert got[:n] == want[:n]
        checked += n
    assert checked >= (40 if dtype == "float32" else 8)


def test_stop_tokens_end_a_row_early(tmp_path):
    from zlm_b200 import Engine
    folder, cfg, tensors = make_model(tmp_path, "A", seed=12)
    prompts = random_prompts(cfg.vocab_size, [6, 20, 3], seed=6)
    eng = Engine.from_pretrained(folder, dtype="float32", max_tokens=512)
    free = eng.generate(prompts, max_tokens=10).tokens
    stop = free[1][3]
    res = eng.generate(prompts, max_tokens=10, stop_token_ids=[stop])
    for f, t, why in zip(free, res.tokens, res.finish_reasons):
        if stop in f:
            assert t == f[:f.index(stop)] and why == "stop"
        else:
            assert t == f and why == "length"
    assert eng.cache.slots.held == 0


def test_queued_steps_generate_what_single_steps_generate(tmp_path):
    """The loop that queues decode steps one ahead against the loop that waits for every step,
    on the same engine: rows that meet a stop token at different steps, rows that reach their
    length, sampled and greedy.  In 32-bit a row's logits do not depend on the batch, so the
    tokens must be the same."""
    from zlm_b200 import Engine
    from zlm_b200.engine.generate import generate
    from zlm_b200.sampling import SamplingParams

    class OneAtATime:
        """The engine without its queued steps."""
        def __init__(self, eng):
            self._e = eng

        def __getattr__(self, name):
            if name in ("decode_launch", "decode_fetch"):
                raise AttributeError(name)
            return getattr(self._e, name)

    folder, cfg, _ = make_model(tmp_path, "C", seed=15)
    prompts = random_prompts(cfg.vocab_size, [4, 33, 9, 64, 2, 17], seed=8)
    eng = Engine.from_pretrained(folder, dtype="float32", max_tokens=2048, max_batch=4)
    for params in (SamplingParams(), SamplingParams(0.9, 20, 0.95, 3)):
        free = generate(OneAtATime(eng), prompts, 14, params, stop_token_ids=()).tokens
        stops = [free[0][2], free[3][9], free[5][0]]
        want = generate(OneAtATime(eng), prompts, 14, params, stop_token_ids=stops)
        got = generate(eng, prompts, 14, params, stop_token_ids=stops)
        assert got.tokens == want.tokens and got.finish_reasons == want.finish_reasons
        assert "stop" in got.finish_reasons and "length" in got.finish_reasons
        assert eng.cache.slots.held == 0
    eng.cache.check()


def _needs_graphs(request):
    if request.config.getoption("--zlm-bounds-check"):
        pytest.skip("the bounds-check build runs without CUDA graphs")


def test_an_engine_dropped_earlier_does_not_disturb_a_later_capture(tmp_path, request):
    """An engine that is no longer referenced is freed by Python's cycle collector at a moment
    of its choosing; when that moment fell inside another engine's graph capture, the capture
    was lost.  Here the dropped engine is kept from being collected until the second engine
    captures, and a collection is forced in the middle of that capture: it must find nothing
    left to free."""
    _needs_graphs(request)
    import gc
    from zlm_b200 import Engine
    folder, cfg, _ = make_model(tmp_path, "B", seed=4)
    prompts = random_prompts(cfg.vocab_size, [6, 3], seed=2)
    first = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=256, max_batch=2)
    want = first.generate(prompts, max_tokens=6)
    assert first.decoder.graphs
    first.myself = first                 # a cycle: only the collector can free this engine now
    gc.collect()
    gc.disable()
    try:
        del first
        second = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=256, max_batch=2)
        argmax = second.rt.k.argmax
        seen = []

        def collecting_argmax(*a, **kw):
            if torch.cuda.is_current_stream_capturing():
                seen.append(gc.collect())
            return argmax(*a, **kw)

        second.rt.k.argmax = collecting_argmax
        got = second.generate(prompts, max_tokens=6)
    finally:
        gc.enable()
    assert seen and got.tokens == want.tokens


def test_a_dropped_engine_is_freed_at_once(tmp_path, request):
    """Nothing in an engine refers back to it strongly: when the last reference goes, its
    weights, cache and graphs go with it, without waiting for the cycle collector."""
    _needs_graphs(request)
    import gc
    import weakref
    from zlm_b200 import Engine
    folder, cfg, _ = make_model(tmp_path, "B", seed=4)
    gc.collect()
    gc.disable()
    try:
        eng = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=256, max_batch=2)
        eng.generate(random_prompts(cfg.vocab_size, [6, 3], seed=2), max_tokens=4)
        assert eng.decoder.graphs
        gone = weakref.ref(eng)
        runner = eng.decoder
        del eng
        assert gone() is None
        with pytest.raises(RuntimeError, match="gone"):
            runner.step([0], [1], None)
    finally:
        gc.enable()


def test_temperature_sampling_is_reproducible_and_batch_independent(tmp_path):
    from zlm_b200 import Engine
    folder, cfg, _ = make_model(tmp_path, "B", seed=13)
    prompts = random_prompts(cfg.vocab_size, [1, 7, 16, 31], seed=7)
    eng = Engine.from_pretrained(folder, dtype="float32", max_tokens=1024)
    a = eng.generate(prompts, max_tokens=12, temperature=0.8, seed=42).tokens
    b = eng.generate(prompts, max_tokens=12, temperature=0.8, seed=42).tokens
    c = eng.generate(prompts, max_tokens=12, temperature=0.8, seed=43).tokens
    assert a == b and a != c
    assert all(len(t) == 12 for t in a)
    # request 2 alone must draw what it drew in the batch: same seed, request index and positions
    eng2 = Engine.from_pretrained(folder, dtype="float32", max_tokens=1024, max_batch=1)
    d = eng2.generate(prompts, max_tokens=12, temperature=0.8, seed=42).tokens
    assert d == a
    e = eng.generate(prompts, max_tokens=12, temperature=0.8, top_k=5, top_p=0.9, seed=42).tokens
    assert all(len(t) == 12 for t in e)


def test_command_line(tmp_path):
    folder, cfg, tensors = make_model(tmp_path, "A", seed=14)
    p = [3, 9, 27, 81]
    want = P.greedy_generate(tensors, plain_sizes(cfg), p, 5)
    out = subprocess.run([sys.executable, "-m", "zlm_b200", "run", folder, "-p", " ".join(map(str, p)),
                          "--max-tokens", "5", "--dtype", "float32", "--no-stream", "--metrics=full"],
                         cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    first = out.stdout.splitlines()[0]
    assert first == "0\t" + " ".join(map(str, want))
    assert "decode:" in out.stdout and "phases:" in out.stdout
