"""RMSNorm over rows of the fp32 residual stream.

y = (x * 1/sqrt(mean(x^2) + eps)) * w, weight used as it is
(src/kernels/transformer/norm.zig:4-37).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_norm
from .base import Norm, ParamSpec


@register_norm("rms_norm")
class RMSNorm(Norm):
    reads_stream_by_kernel = True

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), kind="vector", init="one_plus_normal")}

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        self.weight = params["weight"]

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        self.rt.k.rmsnorm(out, x, self.weight, self.eps, rows)
