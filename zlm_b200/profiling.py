"""Per-operation timing of a step, in the manner of the reference's ``run --profile``
(per-op nanoseconds, weight bytes per token and matvec GB/s:
src/cli/commands/run.zig:233-299, counters filled in src/runtime/executor.zig:104-128).

``ProfilingKernels`` stands in the kernel object's place (parts never launch anything
themselves, they call ``rt.k``): every call is bracketed by two CUDA events on the
launching stream and filed under the operation's name, with the bytes it has to move and
the floating-point operations it has to do, counted from its arguments.  Steps run
eagerly (no graph) while it is in place.  So that the times are the kernels' and not the
host's launch gaps, a profiled step begins with a short device-side wait that lets the
host queue the step's launches ahead.

Events around every launch are right for the long kernels of a prefill.  The kernels of a
decode step take a few microseconds each, as long as an event and the launch gap beside it;
for them ``mode="graph"`` only notes the calls of one step, and ``table`` then captures, for
each operation, all its calls of the step (one per layer, each with that layer's own
weights, which together are far larger than L2) as one CUDA graph, replays it, and divides
its time by the number of calls: the operation as it runs inside a captured step, weights
streaming from HBM.

``profile_engine`` runs one prefill and some decode steps this way and returns a table.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class OpRecord:
    calls: int = 0
    bytes: float = 0.0
    flops: float = 0.0
    events: List[Tuple[torch.cuda.Event, torch.cuda.Event]] = field(default_factory=list)
    noted: List = field(default_factory=list)       # graph mode: the calls, to be replayed
    ms: float = 0.0

    def settle(self) -> None:
        for a, b in self.events:
            self.ms += a.elapsed_time(b)
        self.events = []


def _nbytes(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.numel() * t.element_size()


class ProfilingKernels:
    """Wraps a kernel object; same methods, timed."""

    name = "profiling"

    def __init__(self, kernels, weight_names: Optional[Dict[int, str]] = None, mode: str = "events",
                 pdl: bool = False):
        self.k = kernels
        self.weight_names = weight_names or {}
        self.mode = mode
        self.pdl = pdl          # graph mode: capture with programmatic dependent launch, as the decode runner does
        self.phase = "step"
        self.records: "OrderedDict[Tuple[str, str], OpRecord]" = OrderedDict()

    def __getattr__(self, name):
        # whatever is not timed here (status, scratch, settings) goes to the real object
        return getattr(self.k, name)

    # ------------------------------------------------------------------ bookkeeping
    def _timed(self, op: str, nbytes: float, flops: float, fn, *args, **kw):
        rec = self.records.setdefault((self.phase, op), OpRecord())
        if self.mode == "graph":
            rec.calls += 1
            rec.bytes += nbytes
            rec.flops += flops
            rec.noted.append((fn, args, kw))
            return fn(*args, **kw)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*args, **kw)
        e1.record()
        rec.calls += 1
        rec.bytes += nbytes
        rec.flops += flops
        rec.events.append((e0, e1))
        return out

    def run_ahead(self, microseconds: int = 2000) -> None:
        """Keeps the device busy for a moment so that the host can queue launches ahead."""
        sleep = getattr(torch.cuda, "_sleep", None)
        if sleep is not None:
            sleep(int(microseconds * 1900))         # cycles at about 1.9 GHz

    def _replay_noted(self, rec: OpRecord, repeats: int = 5) -> None:
        """All noted calls of one operation as one graph; the best of a few replays."""
        import gc
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        gc.collect()
        if self.pdl:
            self.k.set_pdl(True)
        try:
            with torch.cuda.graph(g):
                for fn, args, kw in rec.noted:
                    fn(*args, **kw)
        finally:
            if self.pdl:
                self.k.set_pdl(False)
        best = None
        for _ in range(repeats + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1)
            best = t if best is None else min(best, t)
        rec.ms = best
        rec.noted = []

    def table(self) -> List[dict]:
        torch.cuda.synchronize()
        rows = []
        for (phase, op), r in self.records.items():
            if r.noted:
                self._replay_noted(r)
            r.settle()
            us = r.ms * 1e3 / max(1, r.calls)
            sec = r.ms * 1e-3
            rows.append({"phase": phase, "op": op, "calls": r.calls, "us_per_call": round(us, 2),
                         "total_ms": round(r.ms, 4), "mb_per_call": round(r.bytes / max(1, r.calls) / 1e6, 3),
                         "gb_s": round(r.bytes / sec / 1e9, 1) if sec > 0 else 0.0,
                         "tflop_s": round(r.flops / sec / 1e12, 2) if sec > 0 else 0.0})
        return rows

    # ------------------------------------------------------------------ the kernels
    def embed(self, out, table, ids):
        n = _nbytes(out) + out.shape[0] * out.shape[1] * table.element_size()
        return self._timed("embed", n, 0, self.k.embed, out, table, ids)

    def rmsnorm(self, out, x, w, eps, rows=None):
        R, H = out.shape
        return self._timed("rmsnorm", R * H * 4 + _nbytes(out) + _nbytes(w), 0, self.k.rmsnorm, out, x, w, eps, rows)

    def swiglu(self, out, gu):
        return self._timed("swiglu", _nbytes(out) + _nbytes(gu), 0, self.k.swiglu, out, gu)

    def _linear_name(self, w, kind: str) -> str:
        return f"{kind} {self.weight_names.get(w.data_ptr(), f'[{w.shape[0]}x{w.shape[1]}]')}"

    def linear(self, out, x, w, accumulate=False, impl=None, defer=False):
        T, K = x.shape
        N = w.shape[0]
        n = _nbytes(w) + T * K * x.element_size() + T * N * out.element_size() * (2 if accumulate else 1)
        # graph mode times every operation by itself, so a product is finished where it is issued
        return self._timed(self._linear_name(w, "linear"), n, 2.0 * T * N * K, self.k.linear, out, x, w,
                           accumulate=accumulate, impl=impl, defer=defer and self.mode != "graph")

    def linear_swiglu(self, out, x, w, impl=None):
        T, K = x.shape
        N = w.shape[0]
        n = _nbytes(w) + T * K * x.element_size() + _nbytes(out)
        return self._timed(self._linear_name(w, "linear+swiglu"), n, 2.0 * T * N * K, self.k.linear_swiglu, out, x, w,
                           impl=impl)

    def rope_table(self, out, inv_freq, n_rot, token_pos):
        return self._timed("rope_table", _nbytes(out), 0, self.k.rope_table, out, inv_freq, n_rot, token_pos)

    def linear_qkv_rope(self, q_out, x, w, *args, **kw):
        T, K = x.shape
        N = w.shape[0]
        n = _nbytes(w) + T * K * x.element_size() + T * N * q_out.element_size()
        return self._timed(self._linear_name(w, "linear+qk_norm+rope+cache_write"), n, 2.0 * T * N * K,
                           self.k.linear_qkv_rope, q_out, x, w, *args, **kw)

    def qk_norm_rope_write(self, qkv, q_w, k_w, eps, inv_freq, n_rot, token_pos, token_slot, block_table, pool,
                           nq, nkv, hd, write=True):
        T, el = qkv.shape[0], qkv.element_size()
        n = T * (nq + 2 * nkv) * hd * el + T * nq * hd * el + T * 2 * nkv * hd * el
        return self._timed("qk_norm+rope+cache_write", n, 0, self.k.qk_norm_rope_write, qkv, q_w, k_w, eps, inv_freq,
                           n_rot, token_pos, token_slot, block_table, pool, nq, nkv, hd, write)

    def attention(self, out, q, pool, block_table, token_pos, token_slot, nq, nkv, hd, scale, window, plan=None,
                  len_bucket=None):
        T, el = q.shape[0], q.element_size()
        keys_read, pairs = 0, 0
        if plan is not None and getattr(plan, "h_seq_start", None):
            for start, new in zip(plan.h_seq_start, plan.h_seq_new):
                end = start + new
                lo = max(0, start + 1 - window) if window else 0
                keys_read += end - lo
                for p in range(start, end):                 # visible keys of each new token
                    pairs += (p + 1) - (max(0, p + 1 - window) if window else 0)
        n = 2 * T * nq * hd * el + keys_read * 2 * nkv * hd * pool.element_size()
        kind = "attention decode" if (plan is not None and plan.is_decode) else "attention prefill"
        return self._timed(kind, n, 4.0 * nq * hd * pairs, self.k.attention, out, q, pool, block_table, token_pos,
                           token_slot, nq, nkv, hd, scale, window, plan, len_bucket=len_bucket)

    def argmax(self, out, logits, fresh=False):
        return self._timed("argmax", _nbytes(logits), 0, self.k.argmax, out, logits, fresh=fresh)

    def sample(self, out, logits, *args, **kw):
        return self._timed("sample", _nbytes(logits), 0, self.k.sample, out, logits, *args, **kw)


def weight_names(model) -> Dict[int, str]:
    """Device address of every matrix a part holds -> "Part.attribute" (the same for all layers)."""
    names: Dict[int, str] = {}
    parts = [model.embedding, model.final_norm, model.head]
    for b in model.blocks:
        parts.append(b)
        children = getattr(b, "children", None)
        if children:
            parts += list(children().values())
    for p in parts:
        for attr, val in vars(p).items():
            if isinstance(val, torch.Tensor) and val.dim() == 2 and val.is_cuda:
                names.setdefault(val.data_ptr(), f"{type(p).__name__}.{attr}")
    return names


def profile_engine(engine, prompts: Sequence[Sequence[int]], decode_steps: int = 8, sampling=None,
                   decode_mode: str = "graph") -> List[dict]:
    """One prefill step with every prompt whole and ``decode_steps`` decode steps of all
    rows, each operation timed by CUDA events; returns ``ProfilingKernels.table()``.  The
    sequences are released again."""
    from .sampling import SamplingParams
    sampling = sampling or SamplingParams()
    real = engine.rt.k
    prof = ProfilingKernels(real, weight_names(engine.model))
    if decode_mode == "graph":
        decode_steps = min(decode_steps, 1)        # one step's calls are noted and replayed per operation
    graphs = engine.decoder.use_graphs
    slots = [engine.new_sequence() for _ in prompts]
    # as many prompts per prefill step as the engine's step takes
    per = max(1, engine.max_step_tokens // max(len(p) for p in prompts))

    def prefill():
        toks = []
        for i in range(0, len(prompts), per):
            prof.run_ahead()
            toks += engine.prefill_sample(slots[i:i + per], prompts[i:i + per], sampling,
                                          list(range(i, i + len(prompts[i:i + per]))))
        return toks

    try:
        # once unprofiled, so that no first-call set-up (scratch buffers, attributes) is timed
        toks = prefill()
        for s in slots:
            engine.release(s)
        slots = [engine.new_sequence() for _ in prompts]
        engine.rt.k = prof
        engine.decoder.use_graphs = False
        prof.phase = "prefill"
        toks = prefill()
        prof.phase = "decode"
        if decode_steps:
            toks = engine.decode_sample(slots, toks, sampling, list(range(len(prompts))))     # first-call set-up, untimed
            prof.records = OrderedDict((k, v) for k, v in prof.records.items() if k[0] != "decode")
            prof.mode = decode_mode
            prof.pdl = len(prompts) <= 16 and hasattr(real, "set_pdl")
        for _ in range(decode_steps):
            if any(engine.length(s) + 1 > engine.max_seq_len for s in slots):
                break
            prof.run_ahead()
            toks = engine.decode_sample(slots, toks, sampling, list(range(len(prompts))))
        rows = prof.table()          # graph mode replays the noted calls: the sequences must still be held
    finally:
        engine.rt.k = real
        engine.decoder.use_graphs = graphs
        for s in slots:
            engine.release(s)
    return rows


def format_table(rows: List[dict]) -> str:
    out = []
    for phase in OrderedDict((r["phase"], None) for r in rows):
        sel = [r for r in rows if r["phase"] == phase]
        total = sum(r["total_ms"] for r in sel) or 1.0
        out.append(f"{phase}: {total:.3f} ms in timed operations")
        out.append(f"  {'operation':<44}{'calls':>6}{'us/call':>10}{'ms':>9}{'share':>7}{'MB/call':>10}{'GB/s':>9}{'TFLOP/s':>9}")
        for r in sorted(sel, key=lambda r: -r["total_ms"]):
            out.append(f"  {r['op']:<44}{r['calls']:>6}{r['us_per_call']:>10.2f}{r['total_ms']:>9.3f}"
                       f"{100 * r['total_ms'] / total:>6.1f}%{r['mb_per_call']:>10.3f}{r['gb_s']:>9.1f}{r['tflop_s']:>9.2f}")
    return "\n".join(out)
