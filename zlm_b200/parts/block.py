"""Block arrangements: how a mixer and a feed-forward sit on the residual stream.

``pre_norm``: h = h + mixer(norm(h)); h = h + ffn(norm(h)), plain adds in fp32
(src/architectures/impl/qwen3/block.zig:21-41).  The parts add their output
into the stream themselves, so the last projection of each can carry the add.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_arrangement
from .base import FeedForward, LayerIO, Mixer, Norm, Part, StepContext


@register_arrangement("pre_norm")
class PreNormBlock(Part):
    def __init__(self, hidden_size: int, mixer: Mixer, feed_forward: FeedForward,
                 mixer_norm: Norm, feed_forward_norm: Norm):
        self.hidden = int(hidden_size)
        self.mixer, self.ffn = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, feed_forward_norm

    def children(self) -> Dict[str, Part]:
        return {"mixer": self.mixer, "feed_forward": self.ffn,
                "mixer_norm": self.mixer_norm, "feed_forward_norm": self.ffn_norm}

    @property
    def graph_safe(self) -> bool:      # type: ignore[override]
        return all(c.graph_safe for c in self.children().values())

    def prefers_plain_launches(self, rows: int) -> bool:
        return any(c.prefers_plain_launches(rows) for c in self.children().values())

    def step_key(self, ctx: StepContext):
        keys = tuple(k for k in (c.step_key(ctx) for c in self.children().values()) if k is not None)
        return keys or None

    def first_norm_weight(self):
        """The weight of the norm that reads the stream first in this block, if that norm is the kernel
        object's ``rmsnorm`` and nothing else (what the block before may tell its last product)."""
        n = self.mixer_norm
        return getattr(n, "weight", None) if n.reads_stream_by_kernel else None

    def forward(self, hidden: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt = self.rt
        x = rt.ws.get("block.normed", hidden.shape, rt.dtype)
        # What the kernel object may make of knowing who follows whom (``CudaKernels.expect_norm``): the
        # norm after a part, so that the part's last product can prepare it, and whether a norm's
        # output goes to products alone.  A kernel object without these words is told nothing.
        expect = getattr(rt.k, "expect_norm", None)
        by_products = getattr(rt.k, "norm_output_read_by_products", None)
        if not self.mixer_norm.reads_stream_by_kernel:
            self.finish_products()
        if by_products is not None:
            by_products(self.mixer.reads_input_by_products)
        self.mixer_norm.forward(x, hidden)
        if expect is not None:
            expect(getattr(self.ffn_norm, "weight", None) if self.ffn_norm.reads_stream_by_kernel else None)
        self.mixer.forward(x, hidden, ctx, io)
        if not self.ffn_norm.reads_stream_by_kernel:
            self.finish_products()
        if by_products is not None:
            by_products(self.ffn.reads_input_by_products)
        self.ffn_norm.forward(x, hidden)
        if expect is not None:
            expect(ctx.extras.get("norm_after_block"))       # the model's word: the next block's first norm
        self.ffn.forward(x, hidden, ctx)
        if expect is not None:
            expect(None)
