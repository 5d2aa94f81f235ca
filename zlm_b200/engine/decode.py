"""Decode steps as replayed CUDA graphs.

A decode step (one token for each of R live sequences, logits at every row, one
sampled token per row) is a chain of a few hundred small operations; launched one
by one the GPU finishes them faster than the host can launch them.  All inputs of
a step live at fixed device addresses (the per-step integer arrays in the engine's
staging buffer, the block tables, the scratch buffers) and only their content
changes from step to step, so the step's device work is captured once per (rows,
what the parts say changes their launches, sampling parameters) as a CUDA graph and
replayed.

Sampled tokens stay on the device and can be fed to the next step from there, so
a run of steps needs no host round trip unless the caller wants the tokens.

A persistent kernel that walked a recorded step in one cooperative launch was built
and measured against the graph; it lost at every size (Qwen3-8B sizes, batch 8: 6.7
against 3.9 ms a step; Qwen3-0.6B sizes, batch 1 / 8: 580 / 2,580 against 1,010 /
6,160 tokens a second) and was taken out.
"""
from __future__ import annotations

import gc
import weakref
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..sampling import SamplingParams
from .batch import StepError, make_context

MAX_GRAPHS = 64      # captured steps kept; the one unused for longest goes first


class DecodeRunner:
    def __init__(self, engine, use_graphs: Optional[bool] = None):
        # the engine owns this runner: a weak reference back, so that dropping the engine frees
        # its weights and cache at once instead of when the cycle collector next runs
        self._engine = weakref.ref(engine)
        cuda = engine.device.type == "cuda"
        # (the bounds-check build reads its findings back after every call, which a capture does not allow)
        checked = bool(getattr(engine.rt.k, "bounds_check", False))
        self.use_graphs = (cuda and engine.model.graph_safe and not checked) if use_graphs is None else use_graphs
        # Programmatic dependent launch between the step's kernels (a kernel's blocks may be
        # scheduled while the kernel before it drains; each waits before it reads what that one
        # wrote): None = on, unless a part of the model asks for plain stream order at this
        # number of rows (``Part.prefers_plain_launches``).  Measured against plain stream order:
        # Qwen3-8B sizes, batch 8: 2,074 -> 2,097 tokens/s, batch 1: 296 -> 299; 0.6B sizes,
        # batch 8: 5,940 -> 6,100, batch 1: 964 -> 1,028.  Above 16 rows it used to gain nothing
        # (batch 64: 8,446 -> 8,475 and 16,450 -> 16,120); since the decode attention loads its
        # first pages, and the few-token products their first weights, before their wait it does:
        # a step at batch 17 / 24 / 40 / 64 is 2 to 6 / 1 to 3 / 5 / 3 % shorter at 8B sizes and
        # 7 / 6 / 5 to 7 / 2 to 5 % at 0.6B sizes.
        self.use_pdl: Optional[bool] = None
        self.graphs: "OrderedDict[Tuple, torch.cuda.CUDAGraph]" = OrderedDict()
        self.graph_generation = -1
        self.replays = 0
        self.out = torch.zeros(engine.max_batch, dtype=torch.int32, device=engine.device)
        # where queued steps leave their tokens for the host: two buffers, so that a step can be
        # queued while the one before it is still being read
        self._landing = [torch.zeros(engine.max_batch, dtype=torch.int32, pin_memory=cuda) for _ in range(2)]
        self._flip = 0
        self.last_logits: Optional[torch.Tensor] = None
        self.launches_per_step = 0

    @property
    def e(self):
        engine = self._engine()
        if engine is None:
            raise RuntimeError("the engine of this decode runner is gone")
        return engine

    # ------------------------------------------------------------------ one step
    def step(self, slots: Sequence[int], tokens: Optional[Sequence[int]], params: SamplingParams,
             requests: Optional[Sequence[int]] = None) -> torch.Tensor:
        """One token for every slot.  ``tokens`` are the host's token ids, or None to
        feed the tokens that the previous step of the same rows sampled (they are still
        on the device).  Returns the sampled ids, int32 [R], on the device."""
        e = self.e
        R = len(slots)
        if R == 0:
            raise StepError("a step needs at least one sequence")
        if R > e.layout.max_seqs:
            raise StepError(f"the step brings {R} sequences; the engine was built for {e.layout.max_seqs}")
        if len(set(slots)) != R:
            raise StepError("a slot appears twice in one step")
        lengths = e.cache.lengths
        try:
            start = np.fromiter((lengths[s] for s in slots), np.int32, R)
        except KeyError as k:
            raise StepError(f"slot {k.args[0]} is not held by any sequence") from None
        growth = [(s, 1) for s in slots]
        e.cache.reserve(growth)
        slot_a = np.asarray(slots, np.int32)
        ar = np.arange(R, dtype=np.int32)
        arrays = {"token_pos": start, "token_slot": slot_a, "token_seq": ar, "seq_slot": slot_a,
                  "seq_start": start, "seq_new": np.ones(R, np.int32),
                  "cu_seqlens": np.arange(R + 1, dtype=np.int32), "want_rows": ar}
        if tokens is not None:
            tok = np.asarray(tokens, np.int64)
            if tok.shape != (R,):
                raise StepError("one token per slot is needed")
            if tok.min() < 0 or tok.max() >= e.spec.vocab_size:
                raise StepError(f"a token id is outside the vocabulary [0, {e.spec.vocab_size})")
            arrays["token_ids"] = tok.astype(np.int32)
        if not params.greedy:
            # they travel with the step's other integers: nothing here waits for the device
            arrays["sample_request"] = np.asarray(requests if requests is not None else range(R), np.int32)
            arrays["sample_position"] = start + 1
        e.stager.upload(arrays, R, R)
        if tokens is None:
            e.stager.view("token_ids", R).copy_(self.out[:R])
        arrays.setdefault("token_ids", ar)   # make_context only needs the shapes
        ctx = make_context(e.stager, arrays, R, R, e.rt.ws)
        if self.use_graphs:
            self._replay(ctx, R, params)
        else:
            self._device_work(ctx, R, params)
        e.cache.commit(growth)
        e.steps_run += 1
        return self.out[:R]

    # ------------------------------------------------------------------ queued steps
    def launch(self, slots: Sequence[int], tokens: Optional[Sequence[int]], params: SamplingParams,
               requests: Optional[Sequence[int]] = None):
        """``step`` without waiting: the sampled ids are copied to pinned host memory in stream
        order (before a later step can overwrite them on the device).  At most two steps may
        be unfetched at a time."""
        R = len(slots)
        out = self.step(slots, tokens, params, requests)
        buf = self._landing[self._flip]
        self._flip ^= 1
        buf[:R].copy_(out, non_blocking=True)
        done = None
        if self.e.device.type == "cuda":
            done = torch.cuda.Event()
            done.record()
        return done, buf, R

    def fetch(self, handle) -> List[int]:
        done, buf, R = handle
        if done is not None:
            done.synchronize()
        # the host has just waited for the step: what its kernels reported is there to be read
        check = getattr(self.e.rt.k, "check_status", None)
        if check is not None:
            check()
        return buf[:R].tolist()

    # ------------------------------------------------------------------ device work
    def _pdl(self, R: int) -> bool:
        if not hasattr(self.e.rt.k, "set_pdl"):
            return False
        if self.use_pdl is not None:
            return self.use_pdl
        return not self.e.model.prefers_plain_launches(R)

    def _device_work(self, ctx, R: int, params: SamplingParams) -> None:
        if self._pdl(R):
            self.e.rt.k.set_pdl(True)
            try:
                self._device_work_inner(ctx, R, params)
            finally:
                self.e.rt.k.set_pdl(False)
        else:
            self._device_work_inner(ctx, R, params)

    def _device_work_inner(self, ctx, R: int, params: SamplingParams) -> None:
        logits = self.e.run_model(ctx, R)
        self.last_logits = logits
        self._choose(logits, R, params)

    def _choose(self, logits: torch.Tensor, R: int, params: SamplingParams) -> None:
        e = self.e
        if params.greedy:
            e.rt.k.argmax(self.out[:R], logits, fresh=True)      # straight from the model's head
        else:
            e.rt.k.sample(self.out[:R], logits, params.temperature, params.top_k, params.top_p, params.seed,
                          e.stager.view("sample_request", R), e.stager.view("sample_position", R))

    def _generation(self):
        """Changes whenever a scratch buffer that a captured graph may point at has moved."""
        return (self.e.rt.ws.generation, getattr(self.e.rt.k, "scratch_generation", 0))

    def _replay(self, ctx, R: int, params: SamplingParams) -> None:
        e = self.e
        key = (R, e.model.step_key(ctx), params, self._pdl(R))
        if self.graph_generation != self._generation():
            self.graphs.clear()
        entry = self.graphs.get(key)
        if entry is not None:
            self.graphs.move_to_end(key)
        if entry is None:
            # a first eager run creates every scratch buffer the step needs; it also is
            # this step's result, so nothing is computed twice on replayed steps
            self._device_work(ctx, R, params)
            gen = self._generation()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            counter = getattr(e.rt.k, "launches", None)
            before = counter() if counter else 0
            # Python's cycle collector must not run inside the capture: what it frees there (an
            # engine that was dropped earlier, with its graphs and their memory pools) makes
            # CUDA calls that are not allowed while a stream captures, and the capture is lost.
            # So garbage is collected now, and the collector rests until the capture has ended.
            gc.collect()
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g):
                    self._device_work(ctx, R, params)
            finally:
                if collecting:
                    gc.enable()
            if counter:
                self.launches_per_step = counter() - before
            if gen != self._generation():
                raise RuntimeError("scratch buffers moved during graph capture")
            self.graph_generation = gen
            self.graphs[key] = (g, self.last_logits)
            while len(self.graphs) > MAX_GRAPHS:
                self.graphs.popitem(last=False)
            # the capture did not run the kernels; the eager run above already did
            return
        g, self.last_logits = entry          # the logits of these rows, where this graph leaves them
        g.replay()
        self.replays += 1
