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

    # ---- sequences ------------------------------------------------------------
    def new_sequence(self) -> int:
        """Takes a slot for a new sequence and returns it."""
        return self.cache.alloc_slot()

    def release(self, slot: int) -> None:
        """Gives back the slot and every page the sequence holds."""
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step ---------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the tokens of ``entries`` as one batch.  Returns fp32 logits
        [wanted, vocab] in the order of the entries and of their ``want`` (None if
        nothing is wanted).  The tensor is scratch: it is overwritten by the next step."""
        arrays, T, R, W = plan_step(entries, self.cache.lengths, self.spec.vocab_size, self.layout)
        growth = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.reserve(growth)            # raises before anything is launched
        self.stager.upload(arrays)
        ctx = make_context(self.stager, arrays, T, R)
        hidden = self.model.forward(ctx, self.cache.ios)
        logits = None
        if W:
            logits = self.model.logits(hidden, self.stager.view("want_rows", W), W)
        self.cache.commit(growth)
        self.steps_run += 1
        return logits
