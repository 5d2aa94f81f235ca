"""The engine: a model, its weights, its cache, and the one step function.

``step`` takes a batch of sequences with the next tokens of each (a whole prompt,
a chunk, or one token), runs exactly these tokens as one batch against the cache
and returns fp32 logits at the wanted places.  The reference has two entry
points for one sequence, one token (src/runtime/executor.zig:45-86) and a block
of up to 16 prompt tokens (:360-380); here one function serves every cutting.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache import KVCache
from ..config.spec import ConfigError
from ..kernels import PAGE_TOKENS
from ..parts.base import Runtime
from ..parts.model import DecoderModel
from ..registry import config_from_dict, config_from_folder
from ..weights import load_weights, random_tensors
from ..weights.loader import target_dtype
from .batch import MetaLayout, MetaStager, StepEntry, StepError, make_context, plan_step

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


class Engine:
    """Build with ``from_pretrained`` (a folder with config.json and
    model.safetensors) or ``from_random`` (a typed configuration and a seed)."""

    def __init__(self, config, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device,
                 max_tokens: int, max_batch: Optional[int] = None, max_seq_len: Optional[int] = None,
                 max_step_tokens: Optional[int] = None, kernels=None):
        self.config = config
        self.dtype = dtype
        self.device = torch.device(device)
        if kernels is None:
            from ..kernels import get_kernels
            kernels = get_kernels()
        self.spec = config.to_model_spec()
        self.model = DecoderModel(self.spec)
        self.rt = Runtime(self.device, dtype, kernels)
        self.model.attach(self.rt)
        self.model.bind(tensors)
        pages = (int(max_tokens) + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.max_tokens = pages * PAGE_TOKENS
        self.max_seq_len = int(min(max_seq_len or self.spec.max_position, self.spec.max_position, self.max_tokens))
        self.max_batch = int(max_batch or min(pages, 256))
        self.cache = KVCache(self.spec.schedule, self.model.cache_requests(), self.model.state_requests(),
                             self.max_tokens, self.max_batch, self.max_seq_len, dtype, self.device)
        self.max_step_tokens = int(max_step_tokens or self.max_tokens)
        self.layout = MetaLayout(self.max_step_tokens, self.max_batch)
        self.stager = MetaStager(self.layout, self.device)
        self.steps_run = 0
        # dependent launches for the kernels of ``step`` (prefill and chunks; the decode runner has
        # a switch of its own).  Measured, a step of 2,048 / 512 tokens: Qwen3-8B sizes 23.8 -> 23.4 /
        # 9.35 -> 8.75 ms, 0.6B sizes 5.37 -> 4.93 / 3.98 -> 3.85 ms.
        self.use_pdl = True
        self.last_logits: Optional[torch.Tensor] = None      # of the last prefill_sample / decode_sample
        from ..sampling import Sampler
        self.sampler = Sampler(self.rt)
        self._sample_meta = torch.zeros((2, self.max_batch), dtype=torch.int32, device=self.device)
        from .decode import DecodeRunner
        self.decoder = DecodeRunner(self)

    # ---- construction -------------------------------------------------------
    @classmethod
    def from_pretrained(cls, folder: str, dtype="bfloat16", device="cuda:0", max_tokens: int = 4096,
                        **kw) -> "Engine":
        dt = parse_dtype(dtype)
        config = config_from_folder(folder)
        expected = DecoderModel(config.to_model_spec()).param_specs()
        tensors = load_weights(folder, expected, dt, device)
        return cls(config, tensors, dt, device, max_tokens, **kw)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", max_tokens: int = 4096,
                    **kw) -> "Engine":
        """Random weights made on the device (same distributions as the random model
        folder, other values: the device's generator is not the CPU's)."""
        dt = parse_dtype(dtype)
        if isinstance(config, dict):
            config = config_from_dict(config)
        expected = DecoderModel(config.to_model_spec()).param_specs()
        tensors = {}
        for name, p in expected.items():
            if p.ignorable:
                continue
            from ..weights.random_init import random_tensor
            tensors[name] = random_tensor(name, p, seed, device, target_dtype(p, torch.float32, dt))
        return cls(config, tensors, dt, device, max_tokens, **kw)

    def tensor(self, name: str) -> torch.Tensor:
        """Read-back of a weight by its checkpoint name (``model.layers.0.self_attn.q_proj.weight``
        ...), as the engine holds it: on the device, in the compute dtype.  The reference's
        counterpart is its session's tensor view (src/runtime/session.zig:696-724)."""
        return self.model.tensor(name)

    # ---- sequences ------------------------------------------------------------
    def new_sequence(self) -> int:
        """Takes a slot for a new sequence and returns it."""
        return self.cache.alloc_slot()

    def release(self, slot: int) -> None:
        """Gives back the slot and every page the sequence holds."""
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def check(self, sync: bool = False) -> None:
        """Raises ``KernelError`` if a bounded wait inside a kernel has given up since the
        last check (its results, and all after it, are then not valid).  The kernels report
        into pinned host memory, so this reads a word and waits for nothing; it knows of
        the steps the device has finished.  ``sync`` waits for the device first: call it so
        before trusting logits that ``step`` returned."""
        check = getattr(self.rt.k, "check_status", None)
        if check is not None:
            check(sync)

    # ---- the step ---------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the tokens of ``entries`` as one batch.  Returns fp32 logits
        [wanted, vocab] in the order of the entries and of their ``want`` (None if
        nothing is wanted).  The tensor is scratch: it is overwritten by the next step."""
        self.check()              # what earlier steps reported, if they are done by now
        arrays, T, R, W = plan_step(entries, self.cache.lengths, self.spec.vocab_size, self.layout)
        growth = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.reserve(growth)            # raises before anything is launched
        self.stager.upload(arrays, T, R)
        ctx = make_context(self.stager, arrays, T, R, self.rt.ws)
        # dependent launches: a kernel is set up, and has its first weights on the way, while the
        # kernel before it drains (every kernel that is launched so waits before it touches what
        # another one wrote)
        pdl = getattr(self.rt.k, "set_pdl", None) if self.use_pdl else None
        if pdl is not None:
            pdl(True)
        try:
            logits = self.run_model(ctx, W)
        finally:
            if pdl is not None:
                pdl(False)
        self.cache.commit(growth)
        self.steps_run += 1
        return logits

    def run_model(self, ctx, wanted: int) -> Optional[torch.Tensor]:
        """The device work of one step: every schedule entry over the step's tokens,
        then logits at the ``wanted`` first rows of the uploaded ``want_rows``."""
        forget = getattr(self.rt.k, "forget_pending", None)
        if forget is not None:
            forget()            # (only a step that raised half-way leaves anything)
        hidden = self.model.forward(ctx, self.cache.ios)
        logits = self.model.logits(hidden, self.stager.view("want_rows", wanted), wanted) if wanted else None
        flush = getattr(self.rt.k, "flush_shares", None)
        if flush is not None:
            flush()             # a product that a part left for a kernel which then never came
        return logits

    # ---- sampling and generation -------------------------------------------------
    def prefill_sample(self, slots: Sequence[int], prompts: Sequence[Sequence[int]], params,
                       requests: Sequence[int]) -> List[int]:
        """One step with every prompt whole; one token chosen per row at its prompt's
        end, back on the host."""
        logits = self.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        self.last_logits = logits
        R = len(slots)
        meta = self._sample_meta[:, :R]
        if not params.greedy:
            # the token being chosen sits at position len(prompt)
            meta.copy_(torch.tensor([list(requests), [len(p) for p in prompts]], dtype=torch.int32))
        chosen = self.sampler.sample(logits, params, meta[0], meta[1]).tolist()
        self.check()          # the host has just waited for the step
        return chosen

    def decode_sample(self, slots: Sequence[int], tokens: Sequence[int], params,
                      requests: Sequence[int]) -> List[int]:
        """One decode step: feeds one token per row, returns the next ones on the host."""
        chosen = self.decoder.step(slots, tokens, params, requests).tolist()
        self.last_logits = self.decoder.last_logits
        self.check()
        return chosen

    def decode_launch(self, slots: Sequence[int], tokens: Optional[Sequence[int]], params,
                      requests: Sequence[int]):
        """Queues one decode step and returns at once with a handle for ``decode_fetch``.
        ``tokens`` None feeds, for the same rows in the same order, the tokens that the
        step queued before this one samples; they never leave the device."""
        return self.decoder.launch(slots, tokens, params, requests)

    def decode_fetch(self, handle) -> List[int]:
        """Waits for a queued step and returns its sampled token ids."""
        return self.decoder.fetch(handle)

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 256, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 0,
                 stop_token_ids: Optional[Sequence[int]] = None, include_stop: bool = False, on_token=None,
                 on_logits=None):
        """Token-id prompts in, generated token ids out (see ``generate.generate``).
        Option names and defaults are the reference's ``run`` command's
        (src/cli/commands/run.zig:116-120): max_tokens 256, temperature 0 (greedy),
        top_k 0 (off), top_p 1 (off)."""
        from ..sampling import SamplingParams
        from .generate import generate
        return generate(self, prompts, max_tokens, SamplingParams(temperature, top_k, top_p, seed),
                        stop_token_ids, include_stop, on_token, on_logits)
