"""Plain torch stand-ins for the CUDA kernel library, one function per kernel.

Two uses, both in tests only: (1) the plain reference that each CUDA kernel is
compared with on the GPU; (2) a stand-in that lets the engine's host logic
(cache paging, step planning, generation loop) run on a machine without a GPU.
The product never imports this file and has no CPU path of its own.

Formulas as in tests/plain_qwen3.py (same reference citations); this file adds
only what the kernels add: the paged cache layout and packed tokens.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

PAGE = 64


class PlainKernels:
    name = "plain"

    def embed(self, out, table, ids):
        out.copy_(table[ids.long()].float())

    def rmsnorm(self, out, x, w, eps, rows=None):
        R = out.shape[0]
        src = x[rows[:R].long()] if rows is not None else x[:R]
        ms = (src * src).sum(-1, keepdim=True) / src.shape[-1]
        out.copy_(((src * (1.0 / torch.sqrt(ms + eps))) * w.float()).to(out.dtype))

    def swiglu(self, out, gu):
        I = out.shape[1]
        g, u = gu[:, :I].float(), gu[:, I:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    def linear(self, out, x, w, accumulate=False, defer=False):
        y = x.float() @ w.float().t()
        if accumulate:
            out += y
        else:
            out.copy_(y.to(out.dtype))

    def qk_norm_rope_write(self, qkv, q_w, k_w, eps, inv_freq, n_rot, token_pos, token_slot,
                           block_table, pool, nq, nkv, hd, write=True):
        T = qkv.shape[0]
        write = bool(write and nkv)
        x = qkv.float().view(T, nq + 2 * nkv, hd).clone()

        def norm(h, w):
            ms = (h * h).sum(-1, keepdim=True) / hd
            return (h * (1.0 / torch.sqrt(ms + eps))) * w.float()

        if q_w is not None:
            x[:, :nq] = norm(x[:, :nq], q_w)
            if nkv:
                x[:, nq:nq + nkv] = norm(x[:, nq:nq + nkv], k_w)
        if inv_freq is not None and n_rot > 0:
            half, ang = hd // 2, n_rot // 2
            a = token_pos.float()[:, None] * inv_freq.float()[None, :]
            c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
            qk = x[:, :nq + nkv]
            x0, x1 = qk[..., :ang].clone(), qk[..., half:half + ang].clone()
            qk[..., :ang] = x0 * c - x1 * s
            qk[..., half:half + ang] = x0 * s + x1 * c
        upto = nq + (0 if write else nkv)
        qkv.view(T, nq + 2 * nkv, hd)[:, :upto] = x[:, :upto].to(qkv.dtype)
        if write:
            for t in range(T):
                p, sl = int(token_pos[t]), int(token_slot[t])
                page = int(block_table[sl, p // PAGE])
                pool[page, 0, :, p % PAGE, :] = x[t, nq:nq + nkv].to(pool.dtype)
                pool[page, 1, :, p % PAGE, :] = x[t, nq + nkv:].to(pool.dtype)

    def attention(self, out, q, pool, block_table, token_pos, token_slot, nq, nkv, hd, scale, window,
                  plan=None, len_bucket=None):
        T = q.shape[0]
        group = nq // nkv
        for t in range(T):
            p, sl = int(token_pos[t]), int(token_slot[t])
            seq = p + 1
            t0 = seq - window if (window and seq > window) else 0
            keys = torch.arange(t0, seq)
            pages = block_table[sl, (keys // PAGE)].long()
            K = pool[pages, 0, :, keys % PAGE, :].float()     # [n, nkv, hd]
            V = pool[pages, 1, :, keys % PAGE, :].float()
            qt = q[t].float().view(nq, hd)
            for h in range(nq):
                s = (K[:, h // group, :] @ qt[h]) * scale
                w = torch.softmax(s, 0)
                out[t, h * hd:(h + 1) * hd] = (w @ V[:, h // group, :]).to(out.dtype)

    def argmax(self, out, logits, fresh=False):
        R, V = logits.shape
        for r in range(R):
            row = logits[r]
            m = row.max()
            out[r] = int((row == m).nonzero()[0])
