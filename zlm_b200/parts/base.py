"""Interfaces of the parts a model is put together from, and the two objects they
are handed: ``Runtime`` (device, compute dtype, kernels, scratch buffers; lives
as long as the engine) and ``StepContext`` (which tokens this step runs, where
they sit in their sequences and in the cache; lives for one step).

No part knows which model it is in: it gets its sizes and constants as
constructor parameters, names its tensors by local names, and sees the rest of
the world only through these two objects.

Interfaces
----------
Norm              forward(out[R, H], x_f32[T, H], rows=None)
PositionEncoding  either fused into the mixer (``RotaryHalfSplit`` exposes
                  ``inv_freq`` / ``n_rot``) or ``apply(q, k, ctx)`` in place
Mixer             forward(x[T, H], residual_f32[T, H], ctx, io): residual += mix(x)
FeedForward       forward(x[T, H], residual_f32[T, H], ctx): residual += ffn(x)
Block             forward(hidden_f32[T, H], ctx, io)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part wants from the checkpoint.

    kind:  "matrix"  cast to the compute dtype;
           "vector"  kept in 32-bit if the file stores it so, else compute dtype;
           "int"     integer table, kept as int32.
    init:  how the random-weights mode fills it ("normal": N(0, 0.02);
           "one_plus_normal": 1 + N(0, 0.02); "zeros").
    ignorable: may be present in the file although the part does not use it.
    """
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"
    ignorable: bool = False


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer wants to keep per token: keys and values for ``num_kv_heads``
    heads of ``head_dim``, either all of them (window == 0) or the last
    ``window``.  The pool is then [pages, 2, kv_heads, PAGE_TOKENS, head_dim] in the
    compute dtype, the layout the library's attention kernels read.

    A mixer that keeps something else per token (a compressed latent, keys and values of
    different widths, another element type) names the shape of one token's record in
    ``token_shape`` and, if it is not the compute dtype, its ``dtype``: the pool is then
    [pages, PAGE_TOKENS, *token_shape], paged, sized, trimmed by the window and given back
    like any other, and read by the mixer's own code (``num_kv_heads`` and ``head_dim``
    are then only part of what tells one group of layers from another)."""
    num_kv_heads: int
    head_dim: int
    window: int = 0
    token_shape: Optional[Tuple[int, ...]] = None
    dtype: Optional[torch.dtype] = None


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size state a mixer wants per sequence (zeroed when a slot is taken)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Workspace:
    """Scratch buffers by name.  A buffer grows when asked for more and keeps its
    address otherwise, so steady-state steps allocate nothing and captured
    graphs stay valid; ``generation`` counts the reallocations."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self.generation = 0

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = f"{name}:{dtype}"
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.generation += 1
        return buf[:n].view(*shape)


class Runtime:
    def __init__(self, device, dtype: torch.dtype, kernels):
        self.device = device
        self.dtype = dtype
        self.k = kernels
        self.ws = Workspace(device)


@dataclass
class CacheView:
    """One schedule entry's share of a cache group: ``pool`` is
    [pages, 2, kv_heads, PAGE_TOKENS, head_dim] (or [pages, PAGE_TOKENS, *token_shape] for a
    request with a record of its own); ``block_table`` [slots, max_pages]
    maps a slot's logical page to a pool page; ``writes`` is False for an entry
    that reads another entry's cache."""
    pool: torch.Tensor
    block_table: torch.Tensor
    writes: bool
    group: Any = None


@dataclass
class LayerIO:
    """What one schedule entry owns beside its weights."""
    cache: Optional[CacheView] = None
    state: Optional[torch.Tensor] = None     # [slots, *StateRequest.shape]


@dataclass
class StepContext:
    """The tokens of one step.  Device tensors are int32.  Sequence r contributes
    tokens cu_seqlens[r] .. cu_seqlens[r+1]-1, which sit at positions
    seq_start[r] .. seq_start[r] + seq_new[r] - 1 of slot seq_slot[r]."""
    T: int
    R: int
    token_ids: torch.Tensor
    token_pos: torch.Tensor
    token_slot: torch.Tensor
    token_seq: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_new: torch.Tensor
    cu_seqlens: torch.Tensor
    # host copies of the per-sequence arrays
    h_seq_slot: List[int] = field(default_factory=list)
    h_seq_start: List[int] = field(default_factory=list)
    h_seq_new: List[int] = field(default_factory=list)
    is_decode: bool = False
    max_new: int = 0
    max_len: int = 0          # longest sequence after this step
    workspace: Any = None     # the runtime's Workspace
    extras: Dict[str, Any] = field(default_factory=dict)

    def scratch(self, name: str, shape, dtype) -> torch.Tensor:
        """A scratch buffer that lives until the next kernel asks for the same name."""
        return self.workspace.get(name, shape, dtype)


class Part:
    """Base of every part.  ``rt`` is set by ``attach`` before ``bind``."""
    rt: Runtime

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def attach(self, rt: Runtime) -> None:
        self.rt = rt

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        """Takes the loaded tensors (by local name).  May fuse or re-lay them."""

    def check_products(self, **weights: torch.Tensor) -> None:
        """For ``bind``: refuses, when the model is built and not at its first step, a
        weight whose sizes no product kernel takes."""
        check = getattr(self.rt.k, "check_linear", None)
        if check is not None:
            for name, w in weights.items():
                if w is not None:
                    check(f"{type(self).__name__}.{name}", w)

    def tensors(self) -> Dict[str, torch.Tensor]:
        """The part's tensors by the local names of ``param_specs``, as they are used now:
        the inverse of ``bind`` (a part that fused or re-laid tensors undoes it here).  The
        default serves a part that keeps each tensor under an attribute of the name's
        first component (``weight``, ``q_proj`` ...)."""
        out = {}
        for name in self.param_specs():
            t = getattr(self, name.split(".")[0], None)
            if isinstance(t, torch.Tensor):
                out[name] = t
        return out

    def finish_products(self) -> None:
        """Has a product finished that a part left in shares of K for the kernel it expected next
        (``kernels.linear(..., defer=True)``).  Kernels called through the runtime's kernel object
        see to this themselves; code that reads such a product's output in any other way (torch
        operations on the stream, a kernel library of its own) calls this first."""
        finish = getattr(self.rt.k, "flush_shares", None)
        if finish is not None:
            finish()

    # a part whose forward launches only kernels (no host-side branching on
    # device data, no allocation) may be captured in a CUDA graph
    graph_safe = True

    def prefers_plain_launches(self, rows: int) -> bool:
        """Whether a decode step of ``rows`` sequences should launch its kernels in plain stream
        order instead of as dependent launches (a kernel's blocks scheduled while the kernel
        before it drains).  One part that says yes decides for the step."""
        return False

    def step_key(self, ctx: "StepContext"):
        """What about a step, beyond its numbers of tokens and sequences, changes the
        launches this part makes (grid sizes, kernel choices): any hashable value, or
        None if nothing does.  A captured decode step is replayed only for steps whose
        keys are equal, so a part whose launches depend on, say, the longest sequence
        returns that quantity here, rounded the way its launches round it."""
        return None


class Norm(Part):
    # Whether this norm reads the stream through ``kernels.rmsnorm`` alone (with the tensor it keeps as
    # ``weight``, if the product before it is to prepare it: ``CudaKernels.expect_norm``).  A part before it may have
    # left its last product into the stream in shares of K for that kernel to add up
    # (``linear(..., defer=True)``); before a norm that reads the stream in any other way the
    # arrangement has that product finished (``finish_products``).
    reads_stream_by_kernel = False

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], ctx: StepContext) -> None:
        raise NotImplementedError


class Mixer(Part):
    # Whether the part reads its input x only through the kernel object's products (``linear`` and
    # its fused forms), all of them before it first writes into the stream, and not afterwards.  The
    # arrangement passes this on for the norm before the part (``norm_output_read_by_products``), whose
    # rows may then never be written out: the products take them from the product before the norm.
    reads_input_by_products = False

    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        raise NotImplementedError


class FeedForward(Part):
    reads_input_by_products = False      # as Mixer.reads_input_by_products

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        raise NotImplementedError
