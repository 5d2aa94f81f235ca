"""Dense SwiGLU feed-forward: down(silu(gate x) * up x), silu(g) = g / (1 + e^-g)
(src/architectures/impl/qwen3/block.zig:36-39,
src/kernels/transformer/activation.zig:8-13).  Gate and up are one fused
projection [gate | up], as the reference fuses them for decode
(src/kernels/linear/matvec/form/fused.zig:27-86).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_feed_forward
from .base import FeedForward, ParamSpec, StepContext


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    reads_input_by_products = True       # x goes into the gate/up product and nowhere else

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden = int(hidden_size)
        self.inter = int(intermediate_size)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate_proj.weight": ParamSpec((self.inter, self.hidden)),
                "up_proj.weight": ParamSpec((self.inter, self.hidden)),
                "down_proj.weight": ParamSpec((self.hidden, self.inter))}

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        gate, up = params.pop("gate_proj.weight"), params.pop("up_proj.weight")
        # bf16: gate and up rows interleaved in eights, so that the product's epilogue holds
        # a channel's gate and up together and writes silu(gate) * up directly
        self.fused = (gate.dtype == torch.bfloat16 and self.inter % 8 == 0
                      and hasattr(self.rt.k, "linear_swiglu"))
        if self.fused:
            from ..kernels import interleave_gate_up
            self.w_gu = interleave_gate_up(gate, up)
        else:
            self.w_gu = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = params.pop("down_proj.weight")
        self.check_products(gate_up_proj=self.w_gu, down_proj=self.w_down)

    def tensors(self) -> Dict[str, torch.Tensor]:
        I, K = self.inter, self.hidden
        if self.fused:
            gu = self.w_gu.view(I // 8, 2, 8, K)
            gate, up = gu[:, 0].reshape(I, K), gu[:, 1].reshape(I, K)
        else:
            gate, up = self.w_gu[:I], self.w_gu[I:]
        return {"gate_proj.weight": gate, "up_proj.weight": up, "down_proj.weight": self.w_down}

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        act = rt.ws.get("ffn.act", (T, self.inter), rt.dtype)
        if self.fused:
            k.linear_swiglu(act, x, self.w_gu)
        else:
            gu = rt.ws.get("ffn.gu", (T, 2 * self.inter), rt.dtype)
            k.linear(gu, x, self.w_gu)
            k.swiglu(act, gu)
        k.linear(residual, act, self.w_down, accumulate=True, defer=True)      # a norm reads the stream next
