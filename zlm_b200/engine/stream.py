"""A decode step as one persistent kernel.

The model's parts do not launch kernels themselves: they call methods of the
kernel object they are handed (``rt.k``).  Handing them a ``StepRecorder`` instead
turns one walk over the model into a list of operation records, the program of
``csrc/decode_stream.cu``: one cooperative launch that carries out the whole step
with the weights streaming through shared memory without a pause between
operations.  A program holds device addresses and sizes only, so it is recorded
once per (rows, length bucket) and run every step; what changes from step to step
(token ids, positions, block tables) is the content of buffers at fixed addresses.

The recorder takes what the stand-alone kernels take in a bf16 decode step of up
to 8 rows; anything else raises ``NotStreamable`` and the caller keeps launching
kernels one by one.  The kernel computes what they compute, in the same order of
sums.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int32, c_void_p
from typing import List, Optional

import numpy as np
import torch

from ..kernels import ACCUM, BF16, F32, PAGE_TOKENS, STORE, STORE_F32, SWIGLU, KernelError, decode_splits

END, EMBED, RMSNORM, GEMV, ROPE, ATTN, COMBINE = range(7)
MAX_TOKENS = 8


class NotStreamable(AttributeError):
    """The step uses something the persistent kernel does not take (an AttributeError, so that
    asking the recorder for a kernel it does not have reads as 'not there')."""


class StreamOp(ctypes.Structure):
    # mirrors ZlmStreamOp (csrc/zlm_stream.h)
    _fields_ = [("type", c_int32), ("barrier", c_int32), ("i", c_int32 * 14), ("f", c_float * 4),
                ("p", c_void_p * 10)]


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _vec_dtype(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise NotStreamable(f"vector weight of dtype {t.dtype}")


class StepRecorder:
    """Stands in for ``CudaKernels`` during one walk over the model and records the
    operations instead of launching them."""

    name = "stream-recorder"

    def __init__(self, kernels, blocks: int):
        self.k = kernels
        self.blocks = blocks
        self.ops: List[StreamOp] = []
        self.keep: List[torch.Tensor] = []        # what the records point at

    # ---- plumbing ----------------------------------------------------------
    def _add(self, kind: int, ints, floats=(), ptrs=()) -> None:
        op = StreamOp()
        op.type = kind
        op.barrier = 1 if self.ops else 0         # every operation reads what the one before wrote
        for n, v in enumerate(ints):
            op.i[n] = int(v)
        for n, v in enumerate(floats):
            op.f[n] = float(v)
        for n, t in enumerate(ptrs):
            if isinstance(t, torch.Tensor):
                self.keep.append(t)
                op.p[n] = t.data_ptr()
            else:
                op.p[n] = t or None
        self.ops.append(op)

    def scratch(self, name, n, dtype, device):
        return self.k.scratch(name, n, dtype, device)

    @property
    def scratch_generation(self):
        return self.k.scratch_generation

    def launches(self) -> int:
        return self.k.launches()

    def __getattr__(self, name):
        # any kernel that is not listed below cannot be part of a program
        raise NotStreamable(f"kernel '{name}' is not part of the persistent decode kernel")

    # ---- the operations ----------------------------------------------------------
    def embed(self, out, table, ids) -> None:
        T, H = out.shape
        if table.dtype != torch.bfloat16 or T > MAX_TOKENS:
            raise NotStreamable("embedding table is not bf16")
        assert out.dtype == torch.float32 and ids.dtype == torch.int32 and out.is_contiguous() and table.is_contiguous()
        self._add(EMBED, (T, H, table.shape[0]), (), (out, table, ids))

    def rmsnorm(self, out, x, w, eps, rows=None) -> None:
        R, H = out.shape
        if out.dtype != torch.bfloat16 or R > MAX_TOKENS:
            raise NotStreamable("rmsnorm output is not bf16")
        assert x.dtype == torch.float32 and x.shape[1] == H and w.shape == (H,)
        assert out.is_contiguous() and x.is_contiguous() and w.is_contiguous()
        vthreads = self.k.lib.zlm_rmsnorm_threads(BF16, R, H)
        self._add(RMSNORM, (R, H, _vec_dtype(w), vthreads), (eps,), (out, x, w, rows))

    def _product(self, out, x, w, mode) -> None:
        T, K = x.shape
        N = w.shape[0]
        if x.dtype != torch.bfloat16 or T > MAX_TOKENS:
            raise NotStreamable(f"product of {T} tokens in {x.dtype}")
        assert w.shape[1] == K and w.dtype == x.dtype and x.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
        unit_rows = self.k.lib.zlm_stream_unit_rows(N, mode, self.blocks)
        self._add(GEMV, (T, N, K, x.stride(0), out.stride(0), mode, unit_rows), (), (out, x, w))

    def linear(self, out, x, w, accumulate=False, impl=None) -> None:
        if impl is not None:
            raise NotStreamable("a forced product kernel")
        if accumulate:
            assert out.dtype == torch.float32
        mode = ACCUM if accumulate else (STORE_F32 if out.dtype == torch.float32 else STORE)
        assert out.shape == (x.shape[0], w.shape[0])
        self._product(out, x, w, mode)

    def linear_swiglu(self, out, x, w, impl=None) -> None:
        if impl is not None:
            raise NotStreamable("a forced product kernel")
        assert w.shape[0] % 16 == 0 and out.shape == (x.shape[0], w.shape[0] // 2) and out.dtype == torch.bfloat16
        self._product(out, x, w, SWIGLU)

    def qk_norm_rope_write(self, qkv, q_w, k_w, eps, inv_freq, n_rot, token_pos, token_slot, block_table, pool,
                           nq, nkv, hd, write=True) -> None:
        T = qkv.shape[0]
        if qkv.dtype != torch.bfloat16 or T > MAX_TOKENS or hd > 128:
            raise NotStreamable("q/k norm and rotation outside bf16, 8 tokens, head size 128")
        assert qkv.shape[1] == (nq + 2 * nkv) * hd and qkv.stride(1) == 1
        has_norm = q_w is not None
        if inv_freq is None:
            n_rot = 0
        write = bool(write and nkv)
        if write:
            assert pool.dtype == qkv.dtype and pool.is_contiguous() and tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hd)
        self._add(ROPE, (T, qkv.stride(0), int(has_norm), n_rot, block_table.stride(0) if block_table is not None else 0,
                         nq, nkv, hd, int(write), _vec_dtype(q_w) if has_norm else F32,
                         self.k.lib.zlm_rope_vector_form(hd, 2, qkv.stride(0), c_void_p(qkv.data_ptr()),
                                                         c_void_p(pool.data_ptr() if write else 0))),
                  (eps,), (qkv, q_w, k_w, inv_freq, token_pos, token_slot, block_table if write else None,
                           pool if write else None))

    def attention(self, out, q, pool, block_table, token_pos, token_slot, nq, nkv, hd, scale, window, plan=None) -> None:
        T = q.shape[0]
        if (plan is None or not plan.is_decode or q.dtype != torch.bfloat16 or T > MAX_TOKENS
                or not self.k.lib.zlm_attention_decode_supported(nq, nkv, hd)):
            raise NotStreamable("attention outside the bf16 decode kernel's shapes")
        assert out.shape == (T, nq * hd) and q.stride(1) == 1 and out.stride(1) == 1 and pool.is_contiguous()
        assert tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hd)
        splits, per = decode_splits(T, nkv, plan.len_bucket, getattr(plan, "attention_blocks", None) or self.blocks)
        part_o = part_ml = None
        if splits > 1:
            part_o = plan.scratch("attn.part_o", (T * nq * splits * hd,), torch.float32)
            part_ml = plan.scratch("attn.part_ml", (T * nq * splits * 2,), torch.float32)
        self._add(ATTN, (T, out.stride(0), q.stride(0), block_table.stride(0), nq, nkv, hd, window, splits, per),
                  (float(np.float32(scale) * np.float32(1.4426950408889634)),), (out, q, pool, block_table, token_pos, token_slot, part_o, part_ml))
        if splits > 1:
            self._add(COMBINE, (T, out.stride(0), nq, hd, splits, per, window), (), (out, part_o, part_ml, token_pos))


class StreamProgram:
    """A recorded step on the device, ready to run."""

    def __init__(self, kernels, rec: StepRecorder, device):
        self.k = kernels
        n = len(rec.ops)
        if ctypes.sizeof(StreamOp) != kernels.lib.zlm_stream_op_bytes():
            raise KernelError("kernel library and Python disagree on the decode program's record size")
        # one tensor map (128 bytes) per product, in device memory beside the program
        products = [op for op in rec.ops if op.type == GEMV]
        host_maps = (ctypes.c_ubyte * (128 * max(1, len(products))))()
        for j, op in enumerate(products):
            rc = kernels.lib.zlm_stream_make_map(ctypes.byref(host_maps, 128 * j), c_void_p(op.p[2]), c_int(op.i[1]),
                                                 c_int(op.i[2]), c_int(op.i[6]))
            if rc != 0:
                raise KernelError(kernels.lib.zlm_last_error().decode())
        self.maps = torch.frombuffer(bytearray(bytes(host_maps)), dtype=torch.uint8).to(device)
        assert self.maps.data_ptr() % 64 == 0
        for j, op in enumerate(products):
            op.p[3] = self.maps.data_ptr() + 128 * j
        arr = (StreamOp * n)(*rec.ops)
        if kernels.lib.zlm_stream_validate(ctypes.byref(arr), c_int(n)) != 0:
            raise KernelError(kernels.lib.zlm_last_error().decode())
        raw = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
        self.ops = raw.to(device)
        self.n_ops = n
        self.counter = torch.zeros(4, dtype=torch.int32, device=device)
        self.keep = rec.keep
        self.kinds = [op.type for op in rec.ops]

    def run(self) -> None:
        self.k._call("zlm_stream_run", c_void_p(self.ops.data_ptr()), c_int(self.n_ops),
                     c_void_p(self.counter.data_ptr()), self.k._stream())


def stream_blocks(kernels) -> int:
    """Blocks of the persistent kernel on the current device; 0 if it cannot run there."""
    lib = getattr(kernels, "lib", None)
    if lib is None or not hasattr(lib, "zlm_stream_blocks"):
        return 0
    return int(lib.zlm_stream_blocks())
