"""Token embedding and the output head.

hidden = E[token, :], no scale (src/architectures/impl/qwen3/block.zig:16-18);
logits = W_out y in fp32, where W_out is the embedding table when the model is
tied (src/architectures/impl/qwen3/block.zig:43-46, src/tuner/compile.zig:170-174).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_embedding, register_head
from .base import ParamSpec, Part


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        self.weight = params["weight"]

    def forward(self, out: torch.Tensor, ids: torch.Tensor) -> None:
        self.rt.k.embed(out, self.weight, ids)


@register_head("lm_head")
class LMHead(Part):
    def __init__(self, vocab_size: int, hidden_size: int, tied: bool):
        self.vocab, self.hidden, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        # a tied checkpoint may still carry a copy of the table under the head's name
        return {"weight": ParamSpec((self.vocab, self.hidden), ignorable=self.tied)}

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = params["weight"]
            self.check_products(weight=self.weight)

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table
        self.check_products(weight=self.weight)

    def forward(self, logits: torch.Tensor, x: torch.Tensor) -> None:
        """logits [R, vocab] fp32 = x [R, hidden] . W^T"""
        self.rt.k.linear(logits, x, self.weight)
