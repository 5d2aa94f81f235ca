"""Shared helpers of the tests: tiny random model folders, the plain reference's
inputs, tolerances, and a driver for bin/trace_run."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_qwen3 as P
from tiny_configs import TINY, plain_sizes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# absolute + relative tolerance on logits.  fp32: reassociation only.  bf16:
# activations are rounded to 8 bits of mantissa between kernels; the plain
# reference runs in fp32 on the same bf16-rounded weights.
# rows are also compared as vectors: |got - want|_2 <= row * |want|_2.
TOL = {"float32": dict(atol=2e-5, rtol=1e-4, row=1e-4), "bfloat16": dict(atol=2e-2, rtol=2e-2, row=2e-2)}

# scale of the q/k norm weights in the tiny models: 2 makes attention peaked, so a
# wrong or missing far key shows in 32-bit; in bfloat16 a peaked softmax multiplies
# the rounding of q and k (measured: the plain implementation on fp32 weights and on
# bf16-rounded weights then differ by up to 8% of a row), so bfloat16 runs keep 1
SHARP = {"float32": 2.0, "bfloat16": 1.0}


def make_model(tmp_path, name: str, seed: int = 0, sharp: float = 1.0):
    """Writes tiny model ``name`` to a folder; returns (folder, typed config, fp32
    tensors by checkpoint name).  ``sharp`` scales the q/k norm weights so that
    attention is peaked and single far keys matter."""
    from zlm_b200.registry import config_from_dict
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.weights import random_tensors, write_safetensors
    cfg = config_from_dict(TINY[name])
    tensors = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), seed, "cpu", torch.float32)
    if sharp != 1.0:
        for n in tensors:
            if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
                tensors[n] = tensors[n] * sharp
    folder = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder, cfg, tensors


def reference_tensors(tensors: Dict[str, torch.Tensor], dtype: str) -> Dict[str, torch.Tensor]:
    """What the plain implementation computes on: fp32 as stored, or, for the
    bfloat16 engine, the matrices rounded to bf16 (norm vectors stay 32-bit, as the
    loader keeps them)."""
    if dtype == "float32":
        return tensors
    return {n: (t if t.dim() == 1 else t.to(torch.bfloat16).float()) for n, t in tensors.items()}


def plain_logits(tensors, cfg, ids: Sequence[int]) -> torch.Tensor:
    return P.forward(tensors, plain_sizes(cfg), ids)


def random_prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", tol=None):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    tol = tol or TOL[dtype]
    err = (got - want).abs()
    bound = tol["atol"] + tol["rtol"] * want.abs()
    if got.dim() > 1:
        rel = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-6)
        assert bool((rel <= tol["row"]).all()), (
            f"{what}: row {int(rel.argmax())} differs by {rel.max():.3e} of its norm; rows over the bound: "
            f"{(rel > tol['row']).nonzero().flatten().tolist()[:10]}")
    if not bool((err <= bound).all()):
        idx = int((err - bound).argmax())
        r, c = divmod(idx, got.shape[-1]) if got.dim() > 1 else (0, idx)
        raise AssertionError(f"{what}: first/worst mismatch at row {r} col {c}: got {got.flatten()[idx]:.6f} "
                             f"want {want.flatten()[idx]:.6f} (max err {err.max():.3e}); rows with errors: "
                             f"{sorted(set((err > bound).nonzero()[:, 0].tolist()))[:10] if got.dim() > 1 else ''}")


class TraceRun:
    """Drives bin/trace_run over a pipe, one step at a time."""

    def __init__(self, model: str, dtype: str, out: str, max_tokens: int):
        self.out = out
        env = dict(os.environ)
        self.proc = subprocess.Popen(
            [os.path.join(ROOT, "bin", "trace_run"), "--model", model, "--dtype", dtype, "--out", out,
             "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)

    def step(self, step: int, entries, end=()):
        rec = {"step": step, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {step}", f"trace_run answered {line!r} (exit {self.proc.poll()})"
        path = os.path.join(self.out, f"{step}.f32")
        if any(e.get("want") for e in entries):
            return np.fromfile(path, dtype="<f4")
        assert not os.path.exists(path)
        return None

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)
