"""Grouped-query attention over the paged cache, with optional per-head RMSNorm
of q and k and a position encoding.

q = Wq x, k = Wk x, v = Wv x from the same normed input; per-head norm of q and
k (one weight of head_dim for all heads) before the rotation; k and v go to the
cache; each query head h reads kv head h // (heads / kv_heads); scores are
scaled by 1/sqrt(head_dim) after the dot; the window, if any, keeps the last
``window`` keys (src/architectures/impl/qwen3/block.zig:23-33,
src/architectures/impl/qwen3/arch.zig:98-116, src/runtime/executor.zig:93-98).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Mapping, Optional

import torch

from ..registry import POSITION_ENCODINGS, lookup, register_mixer
from .base import CacheRequest, LayerIO, Mixer, ParamSpec, StepContext


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    reads_input_by_products = True       # x goes into the q/k/v projection and nowhere else

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm: bool = False, qk_norm_eps: float = 1e-6, window: int = 0,
                 position: Optional[Mapping[str, Any]] = None, kv_proj: bool = True):
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} heads over {num_kv_heads} kv heads")
        self.hidden = int(hidden_size)
        self.nq, self.nkv, self.hd = int(num_heads), int(num_kv_heads), int(head_dim)
        self.qk_norm, self.eps = bool(qk_norm), float(qk_norm_eps)
        self.window = int(window)
        self.kv_proj = bool(kv_proj)
        self.scale = 1.0 / math.sqrt(self.hd)
        position = dict(position or {"kind": "none"})
        kind = position.pop("kind")
        self.position = lookup(POSITION_ENCODINGS, "position encoding", kind)(**position)
        self.Q, self.KV = self.nq * self.hd, self.nkv * self.hd

    # ---- declarations -----------------------------------------------------
    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {"q_proj.weight": ParamSpec((self.Q, self.hidden)),
             "o_proj.weight": ParamSpec((self.hidden, self.Q))}
        if self.kv_proj:
            s["k_proj.weight"] = ParamSpec((self.KV, self.hidden))
            s["v_proj.weight"] = ParamSpec((self.KV, self.hidden))
        if self.qk_norm:
            s["q_norm.weight"] = ParamSpec((self.hd,), kind="vector", init="one_plus_normal")
            if self.kv_proj:
                s["k_norm.weight"] = ParamSpec((self.hd,), kind="vector", init="one_plus_normal")
        return s

    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(self.nkv, self.hd, self.window)

    def attach(self, rt) -> None:
        super().attach(rt)
        self.position.attach(rt)

    def prefers_plain_launches(self, rows: int) -> bool:
        # Measured at 8 kv heads of 128, Qwen3-8B and 0.6B sizes, contexts 2,048 to 4,095: dependent
        # launches shorten a decode step by 1 to 6 % at every batch size from 1 to 64 but 28 to 33,
        # where the decode attention runs one part per (token, kv head) pair on 224 to 264 blocks, half
        # to six tenths of what the device holds at a time, and a step is 2 to 6 % longer with them.
        sm = getattr(self.rt.k, "sm_count", 0)
        if not sm:
            return False
        from ..kernels import DECODE_BLOCKS_PER_SM
        blocks = sm * DECODE_BLOCKS_PER_SM
        return blocks // 2 <= rows * self.nkv <= blocks * 3 // 5

    def step_key(self, ctx: StepContext):
        # the decode kernel cuts the longest sequence's pages into parts: its grid, and with
        # it a captured step, holds for one rounded length
        if not ctx.is_decode:
            return None
        from ..kernels import attention_len_bucket
        return ("gqa_attention", attention_len_bucket(ctx.max_len))

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        if self.kv_proj:
            # one fused projection: rows [q | k | v]
            self.w_qkv = torch.cat([params.pop("q_proj.weight"), params.pop("k_proj.weight"),
                                    params.pop("v_proj.weight")], dim=0).contiguous()
            self.w_q = self.w_qkv[: self.Q]
        else:
            self.w_qkv = None
            self.w_q = params.pop("q_proj.weight")
        self.w_o = params.pop("o_proj.weight")
        self.q_norm = params.pop("q_norm.weight", None)
        self.k_norm = params.pop("k_norm.weight", None)
        self.check_products(q_proj=self.w_q, o_proj=self.w_o)
        if self.q_norm is not None and self.k_norm is not None and self.q_norm.dtype != self.k_norm.dtype:
            self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    def tensors(self) -> Dict[str, torch.Tensor]:
        out = {"q_proj.weight": self.w_q, "o_proj.weight": self.w_o}
        if self.kv_proj:
            out["k_proj.weight"] = self.w_qkv[self.Q: self.Q + self.KV]
            out["v_proj.weight"] = self.w_qkv[self.Q + self.KV:]
        if self.q_norm is not None:
            out["q_norm.weight"] = self.q_norm
        if self.k_norm is not None:
            out["k_norm.weight"] = self.k_norm
        return out

    # ---- the step -----------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        cache = io.cache
        writes = cache.writes and self.kv_proj
        fused_pos = getattr(self.position, "fused", False)
        tbl = cache.block_table if writes else None
        pool = cache.pool if writes else None
        # many tokens: norm, rotation and cache write ride in the projection's epilogue
        w_in = self.w_qkv if writes else self.w_q
        n_rot = getattr(self.position, "n_rot", 0) if fused_pos else -1
        if (fused_pos and hasattr(k, "qkv_rope_supported") and (n_rot == 0 or hasattr(self.position, "table"))
                and k.qkv_rope_supported(x, w_in, self.nq, self.nkv if writes else 0, self.hd, n_rot)):
            q = rt.ws.get("attn.q", (T, self.Q), rt.dtype)
            k.linear_qkv_rope(q, x, w_in, self.q_norm, self.k_norm if writes else None, self.eps,
                              self.position.table(ctx) if n_rot else None, ctx.token_pos, ctx.token_slot, tbl, pool,
                              self.nq, self.nkv if writes else 0, self.hd)
            self._attend(q, residual, ctx, cache)
            return
        if writes:
            qkv = rt.ws.get("attn.qkv", (T, self.Q + 2 * self.KV), rt.dtype)
            # (the norm / rotation / cache write kernel reads the projection next, where there is one)
            k.linear(qkv, x, self.w_qkv, defer=fused_pos or self.qk_norm)
            nkv = self.nkv
        else:
            qkv = rt.ws.get("attn.qkv", (T, self.Q), rt.dtype)
            k.linear(qkv, x, self.w_q, defer=fused_pos or self.qk_norm)
            nkv = 0
        q = qkv[:, : self.Q]
        if fused_pos:
            k.qk_norm_rope_write(qkv, self.q_norm, self.k_norm, self.eps, self.position.inv_freq,
                                 self.position.n_rot, ctx.token_pos, ctx.token_slot, tbl, pool,
                                 self.nq, nkv, self.hd)
        else:
            # norm in place, then the part's own position encoding, then the cache write
            if self.qk_norm:
                k.qk_norm_rope_write(qkv, self.q_norm, self.k_norm, self.eps, None, 0, ctx.token_pos,
                                     ctx.token_slot, None, None, self.nq, nkv, self.hd, write=False)
            kk = qkv[:, self.Q: self.Q + self.KV] if writes else None
            self.position.apply(q, kk, ctx)
            if writes:
                k.qk_norm_rope_write(qkv, None, None, self.eps, None, 0, ctx.token_pos, ctx.token_slot,
                                     tbl, pool, self.nq, nkv, self.hd)
        self._attend(q, residual, ctx, cache)

    def _attend(self, q: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache) -> None:
        rt, k = self.rt, self.rt.k
        out = rt.ws.get("attn.out", (q.shape[0], self.Q), rt.dtype)
        key = self.step_key(ctx)
        k.attention(out, q, cache.pool, cache.block_table, ctx.token_pos, ctx.token_slot,
                    self.nq, self.nkv, self.hd, self.scale, self.window, ctx,
                    len_bucket=key[1] if key else None)
        k.linear(residual, out, self.w_o, accumulate=True, defer=True)       # a norm reads the stream next
