"""A decoder put together from a ``ModelSpec``: embedding, the layers in the
order of the schedule, final norm, head.  This class is the same for every
architecture; what differs is the specification it is built from.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.spec import ConfigError, LayerSpec, ModelSpec, PartSpec
from ..registry import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, lookup)
from .base import (CacheRequest, LayerIO, ParamSpec, Part, Runtime, StateRequest, StepContext)


def _build(table, what: str, spec: PartSpec, **sizes) -> Part:
    cls = lookup(table, what, spec.kind)
    try:
        return cls(**sizes, **dict(spec.params))
    except TypeError as e:
        raise ConfigError(f"{what} '{spec.kind}': {e}") from None


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        H, V = spec.hidden_size, spec.vocab_size
        self.embedding = _build(EMBEDDINGS, "embedding", spec.embedding, vocab_size=V, hidden_size=H)
        self.final_norm = _build(NORMS, "norm", spec.final_norm, size=H)
        self.head = _build(HEADS, "head", spec.head, vocab_size=V, hidden_size=H)
        self.blocks: List[Part] = []
        # (part, its PartSpec) for every part that owns tensors
        self._owners: List[Tuple[Part, PartSpec]] = [
            (self.embedding, spec.embedding), (self.final_norm, spec.final_norm), (self.head, spec.head)]
        for ls in spec.layers:
            mixer = _build(MIXERS, "mixer", ls.mixer, hidden_size=H)
            ffn = _build(FEED_FORWARDS, "feed-forward", ls.feed_forward, hidden_size=H)
            n1 = _build(NORMS, "norm", ls.mixer_norm, size=H)
            n2 = _build(NORMS, "norm", ls.feed_forward_norm, size=H)
            block = lookup(ARRANGEMENTS, "block arrangement", ls.arrangement)(
                hidden_size=H, mixer=mixer, feed_forward=ffn, mixer_norm=n1, feed_forward_norm=n2)
            self.blocks.append(block)
            self._owners += [(mixer, ls.mixer), (ffn, ls.feed_forward), (n1, ls.mixer_norm),
                             (n2, ls.feed_forward_norm)]
        self.rt: Optional[Runtime] = None

    # ---- weights ------------------------------------------------------------
    def param_specs(self) -> Dict[str, ParamSpec]:
        """Checkpoint tensor name -> what is expected there."""
        out: Dict[str, ParamSpec] = {}
        for part, ps in self._owners:
            for local, p in part.param_specs().items():
                name = ps.tensor_name(local)
                if name in out and out[name] != p:
                    raise ConfigError(f"tensor '{name}' is wanted twice with different shapes")
                out[name] = p
        return out

    def attach(self, rt: Runtime) -> None:
        self.rt = rt
        for part, _ in self._owners:
            part.attach(rt)
        for b in self.blocks:
            b.attach(rt)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part, ps in self._owners:
            local = {l: tensors[ps.tensor_name(l)] for l in part.param_specs()
                     if ps.tensor_name(l) in tensors}
            part.bind(local)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.weight)

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor that the checkpoint calls ``name``, as the model holds it now (the
        compute dtype; fused projections are cut apart again)."""
        for part, ps in self._owners:
            for local in part.param_specs():
                if ps.tensor_name(local) == name:
                    got = part.tensors().get(local)
                    if got is None and local == "weight" and getattr(part, "tied", False):
                        got = getattr(part, "weight", None)
                    if got is not None:
                        return got
        raise KeyError(f"the model has no tensor '{name}'")

    def tensor_names(self) -> List[str]:
        return sorted(self.param_specs())

    # ---- what the cache has to provide -----------------------------------
    def cache_requests(self) -> List[Optional[CacheRequest]]:
        """Per schedule entry."""
        return [self.blocks[e.layer].mixer.cache_request() for e in self.spec.schedule]

    def state_requests(self) -> List[Optional[StateRequest]]:
        return [self.blocks[e.layer].mixer.state_request() for e in self.spec.schedule]

    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks)

    def prefers_plain_launches(self, rows: int) -> bool:
        asks = (getattr(b, "prefers_plain_launches", None) for b in self.blocks)
        return any(ask(rows) for ask in asks if ask is not None)

    def step_key(self, ctx: StepContext) -> Tuple:
        """The parts' say on which steps make the same launches (``Part.step_key``): the
        distinct keys of all parts, in the order of their first appearance."""
        seen: List = []
        leaves: List[Part] = [self.embedding, self.final_norm, self.head]
        for b in self.blocks:
            children = getattr(b, "children", None)
            leaves += list(children().values()) if children else [b]
        for p in leaves:
            k = p.step_key(ctx)
            if k is not None and k not in seen:
                seen.append(k)
        return tuple(seen)

    # ---- the step -------------------------------------------------------------
    def forward(self, ctx: StepContext, ios: List[LayerIO]) -> torch.Tensor:
        """Runs the step's tokens through every schedule entry; returns the fp32
        residual stream [T, hidden]."""
        rt = self.rt
        hidden = rt.ws.get("model.hidden", (ctx.T, self.spec.hidden_size), torch.float32)
        self.embedding.forward(hidden, ctx.token_ids)
        sched = self.spec.schedule
        for i, (e, io) in enumerate(zip(sched, ios)):
            # who reads the stream after this block: the next block's first norm (the final norm reads
            # chosen rows only and is told of nothing)
            nxt = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else None
            first = getattr(nxt, "first_norm_weight", None)
            ctx.extras["norm_after_block"] = first() if first is not None else None
            self.blocks[e.layer].forward(hidden, ctx, io)
        ctx.extras["norm_after_block"] = None
        return hidden

    def logits(self, hidden: torch.Tensor, rows: torch.Tensor, n_rows: int,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits [n_rows, vocab] at the token rows ``rows`` of ``hidden``."""
        rt = self.rt
        x = rt.ws.get("model.head_in", (n_rows, self.spec.hidden_size), rt.dtype)
        if not self.final_norm.reads_stream_by_kernel:
            self.final_norm.finish_products()
        self.final_norm.forward(x, hidden, rows)
        if out is None:
            out = rt.ws.get("model.logits", (n_rows, self.spec.vocab_size), torch.float32)
        self.head.forward(out, x)
        return out
