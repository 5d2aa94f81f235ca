"""Choosing the next token from fp32 logits, on the GPU.

temperature 0 is greedy argmax with ties to the lowest index; otherwise the
logits are weighed by exp((l - max) / temperature) over the top_k best
(0: all) and the nucleus of mass top_p (1: all), and one uniform number picks
the token (src/runtime/sampler.zig:6-67).  The uniform of a row is a hash of
(seed, request index, position of the token being chosen), so that what a
request draws does not depend on which other requests share its batch; the
reference seeds one generator per request from its prompt and parameters
(src/runtime/session.zig:167-174).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0 (0 disables it), got {self.top_k}")
        if self.top_p < 0 or self.top_p != self.top_p:
            raise ValueError(f"top_p must be >= 0 (1 or more disables it, 0 keeps the best token only), got {self.top_p}")
        if self.top_p > 1.0:
            object.__setattr__(self, "top_p", 1.0)       # "top_p >= 1 disables nucleus filtering"

    @property
    def greedy(self) -> bool:
        """Whether the choice is the argmax: temperature 0, and also a nucleus of mass 0 or the
        best one of top_k = 1, which keep the highest logit (the lowest index among equals) whatever
        the temperature (src/runtime/sampler.zig:85-110)."""
        return self.temperature <= 0 or self.top_p <= 0 or self.top_k == 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_for(seed: int, request: int, position: int) -> float:
    """The uniform in [0, 1) that the sampling kernel uses for this draw."""
    h = _splitmix64((seed & _MASK) ^ _splitmix64(((request & 0xFFFFFFFF) << 32) | (position & 0xFFFFFFFF)))
    return (h >> 40) / 16777216.0


class Sampler:
    """Runs the sampling kernels of the engine's runtime."""

    def __init__(self, rt):
        self.rt = rt

    def sample(self, logits: torch.Tensor, params: SamplingParams, request: torch.Tensor,
               position: torch.Tensor) -> torch.Tensor:
        """int32 [rows] on the device.  ``request`` and ``position`` are int32 [rows]."""
        R = logits.shape[0]
        out = self.rt.ws.get("sampler.out", (R,), torch.int32)
        if params.greedy:
            self.rt.k.argmax(out, logits, fresh=True)      # straight from the model's head
        else:
            self.rt.k.sample(out, logits, params.temperature, params.top_k, params.top_p, params.seed,
                             request, position)
        return out
