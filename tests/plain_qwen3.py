"""Plain, slow Qwen3-dense forward: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the
``zlm_b200`` package: it takes a dict of tensors keyed by the checkpoint's own
tensor names plus a plain dict of sizes, and recomputes every position of a
sequence from scratch each time it is called.

It rests on the formulas of the reference (Lucas-Palomo/zlm); the reference is
written in Zig and can be neither imported nor compiled where these tests run,
so nothing here was compared with the reference's own binaries.  Each function
cites the reference file and lines whose arithmetic it restates.

Every function works in the dtype of the tensors it is given (float32 in the
tests, float64 for the self-check of the oracle).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def embed(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """hidden = E[token, :], no scale (src/architectures/impl/qwen3/block.zig:16-18,
    src/architectures/impl/qwen3/arch.zig:121)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ms = sum(x^2)/n; inv = 1/sqrt(ms+eps); y = (x*inv)*w over the last axis
    (src/kernels/transformer/norm.zig:4-37)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(ms + eps)
    return (x * inv) * weight


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out_i = sum_j W[i,j] x_j, W row-major [out][in], no bias
    (src/kernels/linear/matvec/kernels/float.zig:69-80)."""
    return x @ w.t()


def head_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head RMSNorm over head_dim with one weight shared by all heads;
    x is [T, heads, head_dim] (src/kernels/transformer/norm.zig:116-126)."""
    return rms_norm(x, weight, eps)


def rope_inv_freq(theta: float, head_dim: int, n_rot: int, dtype) -> torch.Tensor:
    """inv[i] = theta^(-2 i / head_dim), i < n_rot/2 (src/image/zcom.zig:95-109)."""
    i = torch.arange(n_rot // 2, dtype=torch.float64)
    return (float(theta) ** (-2.0 * i / head_dim)).to(dtype)


def rope_half_split(x: torch.Tensor, positions: torch.Tensor, theta: float,
                    n_rot: Optional[int] = None) -> torch.Tensor:
    """Rotate pairs (i, i + head_dim/2), i < n_rot/2, by angle pos * inv[i]
    (src/kernels/transformer/rope.zig:161-206).  x is [T, heads, head_dim]."""
    hd = x.shape[-1]
    n_rot = hd if n_rot is None else n_rot
    half, ang = hd // 2, n_rot // 2
    inv = rope_inv_freq(theta, hd, n_rot, x.dtype)
    a = positions.to(x.dtype)[:, None] * inv[None, :]            # [T, ang]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    x0, x1 = x[..., :ang], x[..., half:half + ang]
    out[..., :ang] = x0 * c - x1 * s
    out[..., half:half + ang] = x0 * s + x1 * c
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: int = 0) -> torch.Tensor:
    """Per query head h (kv head h // group): s_t = (q . k_t) * 1/sqrt(hd) for
    t in [t_start, pos], softmax, o = sum p_t v_t
    (src/kernels/transformer/attention.zig:184-241, scale after the dot :288-301;
    window start: seq = pos+1, t_start = seq - w if w != 0 and seq > w else 0,
    src/runtime/executor.zig:93-98).  q [T, nq, hd]; k, v [T, nkv, hd]."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    for h in range(nq):
        kh = h // group
        for p in range(T):
            seq = p + 1
            t0 = seq - window if (window != 0 and seq > window) else 0
            s = (k[t0:seq, kh, :] @ q[p, h, :]) * scale
            w = torch.softmax(s, dim=0)
            out[p, h, :] = w @ v[t0:seq, kh, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """m = silu(g) * u, silu(g) = g / (1 + e^-g)
    (src/kernels/transformer/activation.zig:8-13)."""
    return (gate / (1.0 + torch.exp(-gate))) * up


# ----------------------------------------------------------------------------
# arrangement
# ----------------------------------------------------------------------------

def layer_window(sizes: Dict, layer: int) -> int:
    """Window of one layer: ``sizes['windows'][layer]`` if present, else 0 (full
    attention, src/architectures/impl/qwen3/arch.zig:43-59)."""
    w = sizes.get("windows")
    return int(w[layer]) if w else 0


def attention_block(x, tensors, sizes, layer, positions):
    """q/k/v -> per-head norm -> rope -> attention -> output projection
    (src/architectures/impl/qwen3/block.zig:23-32)."""
    p = f"model.layers.{layer}.self_attn."
    nq, nkv, hd, eps = sizes["num_heads"], sizes["num_kv_heads"], sizes["head_dim"], sizes["eps"]
    T = x.shape[0]
    q = linear(x, tensors[p + "q_proj.weight"]).reshape(T, nq, hd)
    k = linear(x, tensors[p + "k_proj.weight"]).reshape(T, nkv, hd)
    v = linear(x, tensors[p + "v_proj.weight"]).reshape(T, nkv, hd)
    q = head_rms_norm(q, tensors[p + "q_norm.weight"], eps)
    k = head_rms_norm(k, tensors[p + "k_norm.weight"], eps)
    q = rope_half_split(q, positions, sizes["rope_theta"])
    k = rope_half_split(k, positions, sizes["rope_theta"])
    o = causal_attention(q, k, v, layer_window(sizes, layer)).reshape(T, nq * hd)
    return linear(o, tensors[p + "o_proj.weight"])


def feed_forward(x, tensors, layer):
    """down(silu(gate x) * up x) (src/architectures/impl/qwen3/block.zig:36-39)."""
    p = f"model.layers.{layer}.mlp."
    g = linear(x, tensors[p + "gate_proj.weight"])
    u = linear(x, tensors[p + "up_proj.weight"])
    return linear(swiglu(g, u), tensors[p + "down_proj.weight"])


def decoder_layer(h, tensors, sizes, layer, positions):
    """Pre-norm residual block, plain adds
    (src/architectures/impl/qwen3/block.zig:21-41)."""
    p = f"model.layers.{layer}."
    eps = sizes["eps"]
    h = h + attention_block(rms_norm(h, tensors[p + "input_layernorm.weight"], eps),
                            tensors, sizes, layer, positions)
    h = h + feed_forward(rms_norm(h, tensors[p + "post_attention_layernorm.weight"], eps),
                         tensors, layer)
    return h


def forward(tensors: Dict[str, torch.Tensor], sizes: Dict, ids: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of every position of one whole sequence.  The head is
    ``lm_head.weight`` if the model is untied, else the embedding table
    (src/architectures/impl/qwen3/block.zig:43-46, src/tuner/compile.zig:170-174)."""
    h = embed(tensors["model.embed_tokens.weight"], ids)
    positions = torch.arange(len(ids))
    for layer in range(sizes["num_layers"]):
        h = decoder_layer(h, tensors, sizes, layer, positions)
    h = rms_norm(h, tensors["model.norm.weight"], sizes["eps"])
    head = tensors["model.embed_tokens.weight"] if sizes["tied"] else tensors["lm_head.weight"]
    return linear(h, head)


# ----------------------------------------------------------------------------
# sampling and generation
# ----------------------------------------------------------------------------

def argmax(logits: torch.Tensor) -> int:
    """Highest logit, ties to the lowest index (src/runtime/sampler.zig:14-21)."""
    best = 0
    vals = logits.tolist()
    for i, v in enumerate(vals):
        if v > vals[best]:
            best = i
    return best


def kept_set(logits: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """Indices (sorted by logit, descending) and float64 weights that survive
    top-k and the nucleus cut (src/runtime/sampler.zig:30-58)."""
    l = logits.double()
    order = sorted(range(l.numel()), key=lambda i: (-float(l[i]), i))
    k = min(top_k, len(order)) if top_k > 0 else len(order)
    order = order[:k]
    mx = float(l[order[0]])
    w = [math.exp((float(l[i]) - mx) / temperature) for i in order]
    total = sum(w)
    n = k
    if top_p < 1.0:
        cum = 0.0
        for j, wj in enumerate(w):
            cum += wj / total
            if cum >= top_p:
                n = j + 1
                break
    return order[:n], w[:n]


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """Draw with one uniform u in [0,1): r = u * kept; the first kept index whose
    running sum exceeds r (src/runtime/sampler.zig:59-67)."""
    if temperature <= 0:
        return argmax(logits)
    idx, w = kept_set(logits, temperature, top_k, top_p)
    r = u * sum(w)
    cum = 0.0
    for i, wi in zip(idx, w):
        cum += wi
        if r < cum:
            return i
    return idx[-1]


def greedy_generate(tensors, sizes, prompt: Sequence[int], max_tokens: int,
                    stop_ids: Sequence[int] = ()) -> List[int]:
    """next = argmax(logits at the last position); a stop token ends the
    sequence and is not emitted (src/runtime/session.zig:1524-1566)."""
    ids, out = list(prompt), []
    while len(out) < max_tokens:
        nxt = argmax(forward(tensors, sizes, ids)[-1])
        if nxt in stop_ids:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
