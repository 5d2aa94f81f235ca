"""Decode steps as replayed CUDA graphs.

A decode step (one token for each of R live sequences, logits at every row, one
sampled token per row) launches a few hundred small kernels; at small batches the
GPU finishes them faster than the host can launch them.  The step's device work
is therefore captured once per (R, sampling parameters) and replayed.  All its
inputs live at fixed device addresses: the per-step integer arrays in the
engine's staging buffer, the block tables, the scratch buffers; what changes
from step to step is their content, which is uploaded before the replay.

Sampled tokens stay on the device and can be fed to the next step from there, so
a run of steps needs no host round trip unless the caller wants the tokens.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..sampling import SamplingParams
from .batch import StepError, make_context


class DecodeRunner:
    def __init__(self, engine, use_graphs: Optional[bool] = None):
        self.e = engine
        cuda = engine.device.type == "cuda"
        self.use_graphs = (cuda and engine.model.graph_safe) if use_graphs is None else use_graphs
        # programmatic dependent launch between the step's kernels: off.  Measured at batch 8,
        # Qwen3-8B sizes: 5.32 ms a step with early triggers and weight prefetch before the
        # wait, 4.46 ms with late triggers, 4.49 ms in plain stream order.
        self.use_pdl = False
        self.graphs: Dict[Tuple, torch.cuda.CUDAGraph] = {}
        self.graph_generation = -1
        self.out = torch.zeros(engine.max_batch, dtype=torch.int32, device=engine.device)
        self.last_logits: Optional[torch.Tensor] = None
        self.launches_per_step = 0

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
        e.stager.upload(arrays, R, R)
        if tokens is None:
            e.stager.view("token_ids", R).copy_(self.out[:R])
        if not params.greedy:
            req = np.asarray(requests if requests is not None else range(R), np.int32)
            meta = torch.from_numpy(np.stack([req, start + 1]))
            e._sample_meta[:, :R].copy_(meta)
        arrays.setdefault("token_ids", ar)   # make_context only needs the shapes
        ctx = make_context(e.stager, arrays, R, R, e.rt.ws)
        if self.use_graphs:
            self._replay(ctx, R, params)
        else:
            self._device_work(ctx, R, params)
        e.cache.commit(growth)
        e.steps_run += 1
        return self.out[:R]

    # ------------------------------------------------------------------ device work
    def _device_work(self, ctx, R: int, params: SamplingParams) -> None:
        if self.use_pdl:
            self.e.rt.k.set_pdl(True)
            try:
                self._device_work_inner(ctx, R, params)
            finally:
                self.e.rt.k.set_pdl(False)
        else:
            self._device_work_inner(ctx, R, params)

    def _device_work_inner(self, ctx, R: int, params: SamplingParams) -> None:
        e = self.e
        logits = e.run_model(ctx, R)
        self.last_logits = logits
        meta = e._sample_meta[:, :R]
        if params.greedy:
            e.rt.k.argmax(self.out[:R], logits)
        else:
            e.rt.k.sample(self.out[:R], logits, params.temperature, params.top_k, params.top_p, params.seed,
                          meta[0], meta[1])

    def _generation(self):
        """Changes whenever a scratch buffer that a captured graph may point at has moved."""
        return (self.e.rt.ws.generation, getattr(self.e.rt.k, "scratch_generation", 0))

    def _replay(self, ctx, R: int, params: SamplingParams) -> None:
        e = self.e
        key = (R, ctx.len_bucket, params)
        if self.graph_generation != self._generation():
            self.graphs.clear()
        g = self.graphs.get(key)
        if g is None:
            # a first eager run creates every scratch buffer the step needs; it also is
            # this step's result, so nothing is computed twice on replayed steps
            self._device_work(ctx, R, params)
            gen = self._generation()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            counter = getattr(e.rt.k, "launches", None)
            before = counter() if counter else 0
            with torch.cuda.graph(g):
                self._device_work(ctx, R, params)
            if counter:
                self.launches_per_step = counter() - before
            if gen != self._generation():
                raise RuntimeError("scratch buffers moved during graph capture")
            self.graph_generation = gen
            self.graphs[key] = g
            # the capture did not run the kernels; the eager run above already did
            return
        g.replay()
