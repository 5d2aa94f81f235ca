"""bin/trace_run as a user drives it: requests whole, with the last 32 tokens
one by one, and in batches of unequal lengths one after another in a cache that
is only as large as the trace needs, in 32-bit and in bfloat16, against the
plain implementation."""
import os

import numpy as np
import pytest
import torch

from helpers import SHARP, TraceRun, assert_close, make_model, plain_logits, random_prompts, reference_tensors

pytestmark = pytest.mark.gpu


def up64(n):
    return (n + 63) // 64 * 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_replay_three_ways(tmp_path, name, dtype):
    folder, cfg, tensors = make_model(tmp_path, name, seed=21, sharp=SHARP[dtype])
    ref = reference_tensors(tensors, dtype)
    V = cfg.vocab_size
    cap = cfg.max_position_embeddings
    lens = [min(cap, n) for n in (100, 37, 128, 65)]
    prompts = random_prompts(V, lens, seed=8)
    want = [plain_logits(ref, cfg, p) for p in prompts]

    # 1. each request alone and whole; 2. with its last 32 tokens one by one
    tr = TraceRun(folder, dtype, str(tmp_path / f"out1_{dtype}"), max_tokens=up64(max(lens)))
    step = 0
    for i, p in enumerate(prompts):
        n = len(p)
        got = tr.step(step, [{"id": f"w{i}", "tokens": p, "want": list(range(n))}], end=[f"w{i}"])
        step += 1
        assert_close(torch.from_numpy(got.reshape(n, V)), want[i], dtype, f"{name} whole {i}")
        head = n - 32
        rows = [tr.step(step, [{"id": f"d{i}", "tokens": p[:head], "want": [head - 1]}])]
        step += 1
        for t in range(head, n):
            rows.append(tr.step(step, [{"id": f"d{i}", "tokens": [p[t]], "want": [0]}],
                                end=[f"d{i}"] if t == n - 1 else []))
            step += 1
        assert_close(torch.from_numpy(np.concatenate(rows).reshape(33, V)), want[i][head - 1:], dtype,
                     f"{name} last 32 of {i}")
    assert tr.close() == 0

    # 3. batches of unequal lengths; shorter requests end earlier; a second batch reuses what the first held
    batches = [[0, 1, 2], [3, 1]]
    need = max(sum(up64(lens[i]) for i in b) for b in batches)
    tr = TraceRun(folder, dtype, str(tmp_path / f"out3_{dtype}"), max_tokens=need)
    step = 0
    for b, members in enumerate(batches):
        cut = {i: max(1, lens[i] - 8 - 3 * k) for k, i in enumerate(members)}     # prompt part; the rest decodes
        ids = {i: f"b{b}r{i}" for i in members}
        got = tr.step(step, [{"id": ids[i], "tokens": prompts[i][:cut[i]], "want": [cut[i] - 1]} for i in members])
        step += 1
        got = got.reshape(len(members), V)
        for r, i in enumerate(members):
            assert_close(torch.from_numpy(got[r]), want[i][cut[i] - 1], dtype, f"{name} batch {b} prompt {i}")
        t = 0
        while True:
            live = [i for i in members if cut[i] + t < lens[i]]
            if not live:
                break
            ending = [ids[i] for i in live if cut[i] + t == lens[i] - 1]
            got = tr.step(step, [{"id": ids[i], "tokens": [prompts[i][cut[i] + t]], "want": [0]} for i in live],
                          end=ending).reshape(len(live), V)
            step += 1
            for r, i in enumerate(live):
                assert_close(torch.from_numpy(got[r]), want[i][cut[i] + t], dtype, f"{name} batch {b} row {i} step {t}")
            t += 1
    assert tr.close() == 0


def test_steps_without_wanted_logits_write_no_file(tmp_path):
    folder, cfg, tensors = make_model(tmp_path, "B", seed=22)
    tr = TraceRun(folder, "float32", str(tmp_path / "o"), max_tokens=128)
    assert tr.step(0, [{"id": "x", "tokens": [1, 2, 3], "want": []}]) is None
    got = tr.step(1, [{"id": "x", "tokens": [4], "want": [0]}], end=["x"])
    assert_close(torch.from_numpy(got.reshape(1, -1)), plain_logits(tensors, cfg, [1, 2, 3, 4])[3:], "float32")
    assert tr.close() == 0
    assert sorted(os.listdir(tmp_path / "o")) == ["1.f32"]
