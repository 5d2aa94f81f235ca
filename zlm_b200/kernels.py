"""Python face of the CUDA kernel library (``csrc/*.cu`` -> ``libzlm_b200.so``).

Every method takes torch tensors that already live on the GPU, checks what the
kernel cannot check itself (dtype, contiguity, shapes), and launches on torch's
current stream.  There is no CPU path: constructing ``CudaKernels`` without the
library or without a GPU raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

F32, BF16 = 0, 1
PAGE_TOKENS = 64

_DT = {torch.float32: F32, torch.bfloat16: BF16}

STORE, ACCUM, STORE_F32, SWIGLU = 0, 1, 2, 3


class KernelError(RuntimeError):
    pass


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2I, K] with rows 8 gate, 8 up, 8 gate, ...: the layout ``linear_swiglu`` wants."""
    I, K = gate.shape
    assert up.shape == (I, K) and I % 8 == 0
    return torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


def attention_len_bucket(max_len: int) -> int:
    """The longest sequence of a step in pages, rounded up: powers of two up to 8, then
    multiples of 8.  The decode attention sizes its grid by it, so a captured decode step
    holds for every step with the same bucket."""
    pages = (max_len + PAGE_TOKENS - 1) // PAGE_TOKENS
    bucket = 1
    while bucket < pages and bucket < 8:
        bucket *= 2
    if bucket < pages:
        bucket = (pages + 7) // 8 * 8
    return bucket


DECODE_BLOCKS_PER_SM = 3      # blocks of the decode attention that an SM holds at a time


def decode_splits(rows: int, nkv: int, len_bucket: int, blocks: int = 148 * DECODE_BLOCKS_PER_SM):
    """How the decode attention cuts a sequence's pages: (splits, pages per split).
    ``len_bucket`` is the longest sequence of the step in pages, rounded up, so that the
    choice (and a captured graph) holds for many steps; ``blocks`` is what the device holds
    at a time (its SMs x 3).

    A block's start (the query, its first pages) and end (merging its warps, writing its
    partial result) cost about as much as several pages, and one block streams a page in
    about 0.8 us however idle the memory is (two pages in flight).  Timed inside whole decode
    steps (Qwen3-8B and 0.6B sizes, contexts 2,048 and 4,095; timed alone, kernel after
    kernel, fewer and longer parts look better than they are in a step, where every block's
    first two pages are loaded while the kernels before still run):
    - more (token, kv head) pairs than the device holds blocks (batch 64 at 8 kv heads): parts
      for two waves of blocks (at 2,100 tokens 5.7 TB/s with two waves against 5.5 with four and
      4.6 with sixteen; one part a pair 113 us against 95), one wave for short sequences;
    - otherwise one part for every block the device holds, parts of at least two pages, and no
      second wave of blocks (a few blocks over, 448 on 444 places at batch 8, cost nothing in a
      step while the parts are of up to 12 pages; 224 pairs cut in two parts of 25 pages cost
      a step 5 %): so from 223 pairs on there is one part and no combine (batch 32: a step 5 to 7 %
      shorter than with two waves; batch 16 at 4,095 tokens 2 to 3 % shorter with three parts
      than with seven);
    - up to 32 pairs (batch 1 to 4 at 8 kv heads) the parts' own chains of pages bound the kernel
      and the combine reads every part: as many parts as give half of what the device holds, of
      at least 4 pages (2 for sequences of up to 16 pages, 8 at 32 pairs): batch 1 at 4,095
      tokens 16 parts of 4 pages instead of 32 of 2, a step 3 % (8B sizes) to 7 % (0.6B) shorter."""
    pairs = max(1, rows * nkv)
    if pairs > blocks:
        work = len_bucket * pairs
        waves = 2 if work >= 16 * blocks else 1
        per = max(2, -(-work // (blocks * waves)))
    elif pairs <= 32:
        wanted = -(-(blocks // 2) // pairs)
        least = 8 if pairs == 32 else (2 if len_bucket <= 16 else 4)
        per = max(least, -(-len_bucket // wanted))
    else:
        per = max(2, -(-len_bucket * pairs // blocks))
        # (a few blocks over, 64 pairs x 7 on 444 places, are let be where the parts are short; four
        # blocks of 25 pages that start when the first places come free cost a step 5 %)
        while per < len_bucket and -(-len_bucket // per) * pairs * 10 > blocks * (11 if per <= 12 else 10):
            per += 1
    per = min(per, max(1, len_bucket))
    splits = -(-len_bucket // per)
    while splits > 1024:
        per *= 2
        splits = -(-len_bucket // per)
    return splits, per


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}") from None


def _span_bytes(t: torch.Tensor) -> int:
    """Bytes from the tensor's first element to the end of its last one."""
    if t.numel() == 0:
        return 0
    last = sum((n - 1) * st for n, st in zip(t.shape, t.stride()))
    return (last + 1) * t.element_size()


# what a status code's family byte stands for (tc_common.cuh: TC_FAMILY)
_STATUS_FAMILY = {1: "tcgen05 product", 2: "tcgen05 prefill attention"}


class CudaKernels:
    """Loads (building first if needed) the kernel library and exposes its entry
    points.  One instance per process is enough; see ``get_kernels``."""

    name = "cuda"

    def __init__(self, verbose_build: bool = True, variant: str = ""):
        from .csrc.build import library_path
        self.variant = variant
        self.lib_path = library_path(verbose=verbose_build, variant=variant)
        self.lib = ctypes.CDLL(self.lib_path)
        self.lib.zlm_last_error.restype = ctypes.c_char_p
        self.lib.zlm_launch_count.restype = ctypes.c_longlong
        if self.lib.zlm_page_tokens() != PAGE_TOKENS:
            raise KernelError("kernel library and Python disagree on the cache page size")
        if not torch.cuda.is_available():
            raise KernelError("zlm_b200 needs a CUDA GPU (sm_100a); none is visible and there is no CPU path")
        # binds the status block (pinned host memory the kernels report to) for every part of
        # the library; it copies to device symbols, so it happens here, outside any capture
        if self.lib.zlm_runtime_init() != 0:
            raise KernelError(self.lib.zlm_last_error().decode())
        self.lib.zlm_bounds_first_address.restype = ctypes.c_ulonglong
        self.bounds_check = bool(self.lib.zlm_bounds_check_build())
        self._ranges = []
        # blocks the decode attention cuts its work for; None: what the device holds at a time
        self.decode_blocks: Optional[int] = None
        self.sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
        self._fn = {}
        self._shares = None            # (output, scratch, shares, accumulate) of a product left in shares of K (see linear)
        self.defer_shares = True       # whether linear(defer=True) may leave a product so
        self._candidates = None        # (address of the last logits a few-token product wrote, rows, width, blocks, values, indices)
        # An RMSNorm between two streaming products without a kernel of its own (see ``expect_norm``):
        self.lazy_norms = True         # whether that may happen at all
        self._norm_hint = None         # the weight of the norm that is to follow the next product into the stream
        self._norm_halves = None       # (stream, rows times weight, sums of squares, blocks, weight): a product left them
        self._lazy_ok = False          # the next norm's output is read by products only (the arrangement's word)
        self._lazy = None              # (out, stream, weight, eps, rows times weight, sums of squares, blocks): a norm not run
        self._scratch = {}
        self.scratch_generation = 0
        self._launches = 0

    def scratch(self, name: str, n: int, dtype: torch.dtype, device) -> torch.Tensor:
        """Scratch memory that a kernel needs beyond its operands.  It grows when asked for
        more and keeps its address otherwise; ``scratch_generation`` counts the moves, so
        that a captured graph that holds an old address is not replayed."""
        buf = self._scratch.get(name)
        if buf is None or buf.numel() < n or buf.dtype != dtype or buf.device != device:
            self._scratch[name] = buf = torch.empty(max(n, 1 << 16), dtype=dtype, device=device)
            self.scratch_generation += 1
        return buf

    def launches(self) -> int:
        """Kernels that the library has launched so far (those captured into a graph are counted
        once, when they are captured)."""
        return int(self.lib.zlm_launch_count())

    # -- plumbing ---------------------------------------------------------
    def _call(self, name: str, *args):
        fn = self._fn.get(name)
        if fn is None:
            fn = getattr(self.lib, name)
            fn.restype = c_int
            self._fn[name] = fn
        if self.bounds_check:
            self._register_ranges()
        rc = fn(*args)
        self._launches += 1
        if rc != 0:
            raise KernelError(self.lib.zlm_last_error().decode())
        if self.bounds_check:
            self.check_bounds(name)

    def _p(self, t: Optional[torch.Tensor]) -> c_void_p:
        """The tensor's address as a kernel argument.  In the bounds-check build the bytes it
        spans are also noted as memory the next call may touch."""
        if t is None:
            return c_void_p(0)
        if self._shares is not None:
            # a product whose shares of K are not added up yet: whoever touches its output gets it finished first
            lo, n = self._shares[0].data_ptr(), _span_bytes(self._shares[0])
            if t.data_ptr() < lo + n and lo < t.data_ptr() + _span_bytes(t):
                noted, self._ranges = self._ranges, []      # (this happens while a call's arguments are gathered)
                self.flush_shares()
                self._ranges = noted
        if self._lazy is not None or self._norm_halves is not None:
            self._touch_norms(t)
        if self.bounds_check:
            self._ranges.append((t.data_ptr(), _span_bytes(t)))
        return c_void_p(t.data_ptr())

    @staticmethod
    def _overlap(a: torch.Tensor, b: torch.Tensor) -> bool:
        return a.data_ptr() < b.data_ptr() + _span_bytes(b) and b.data_ptr() < a.data_ptr() + _span_bytes(a)

    def _touch_norms(self, t: torch.Tensor) -> None:
        """A kernel is about to be given ``t``.  Halves of a norm that a product left are void once anything
        else touches the stream they belong to.  A norm that was not run is run now if ``t`` is its output;
        if ``t`` is its stream, the part that was to read the output has gone on to write (the arrangement
        said that it reads before it writes and nobody reads afterwards), and the norm is forgotten."""
        if self._norm_halves is not None and self._overlap(t, self._norm_halves[0]):
            self._norm_halves = None
        if self._lazy is not None:
            if self._overlap(t, self._lazy[0]):
                noted, self._ranges = self._ranges, []      # (this happens while a call's arguments are gathered)
                self.finish_norm()
                self._ranges = noted
            elif self._overlap(t, self._lazy[1]):
                self._lazy = None

    def expect_norm(self, weight: Optional[torch.Tensor]) -> None:
        """An arrangement's word that ``rmsnorm`` with this weight is the next reader of the stream after
        the next product into it (``linear(..., accumulate=True, defer=True)``); None takes it back.  A
        streaming product (up to 16 tokens) then also leaves the normed rows but for their scale, and
        the rows' sums of squares block by block; ``rmsnorm`` launches nothing, and the streaming
        products that read its output take the scale from those sums and apply it to their own sums.
        Two launches fewer a layer in a decode step.  Whatever else is given the norm's output through this
        class has the norm run first (``finish_norm``), so the word is never wrong, only sometimes
        useless; code that reads it by other means says so beforehand (``norm_output_read_by_products``)."""
        self._norm_hint = weight if self.lazy_norms else None

    def norm_output_read_by_products(self, yes: bool) -> None:
        """An arrangement's word on the next ``rmsnorm``: its output is read only through this class,
        before the reading part writes into the stream, and by nobody after that.  Holds for one call."""
        self._lazy_ok = bool(yes) and self.lazy_norms

    def forget_pending(self) -> None:
        """Drops what one call left for a later one (shares of K, a norm's halves, a norm not run, the
        arrangement's words) without finishing any of it: for the start of a step, where anything still
        pending belongs to a step that was given up."""
        self._shares = self._norm_hint = self._norm_halves = self._lazy = None
        self._lazy_ok = False

    def finish_norm(self) -> None:
        """Runs a norm that ``rmsnorm`` left to the products after it."""
        if self._lazy is None:
            return
        out, x, w, eps = self._lazy[:4]
        self._lazy = None
        R, H = out.shape
        self._call("zlm_rmsnorm", self._p(out), c_int(_dt(out)), self._p(x), self._p(w), c_int(_dt(w)),
                   self._p(None), c_int(R), c_int(H), c_float(eps), self._stream())

    def _register_ranges(self) -> None:
        lib = self.lib
        if lib.zlm_bounds_clear_ranges() != 0:
            raise KernelError(lib.zlm_last_error().decode())
        for base, n in self._ranges:
            if n and lib.zlm_bounds_add_range(c_void_p(base), ctypes.c_ulonglong(n)) != 0:
                raise KernelError(lib.zlm_last_error().decode())
        self._ranges = []

    def check_bounds(self, what: str = "") -> None:
        """Bounds-check build: waits for the device and raises if a kernel asked for memory
        outside the tensors it was given (the access itself was skipped)."""
        torch.cuda.synchronize()
        n = int(self.lib.zlm_bounds_violations())
        if n:
            site = int(self.lib.zlm_bounds_first_site())
            addr = int(self.lib.zlm_bounds_first_address())
            self.lib.zlm_bounds_reset()
            raise KernelError(f"{what}: {n} accesses outside the tensors passed; the first at address "
                              f"{addr:#x}, source file id {site >> 16} line {site & 0xffff}")

    # -- the status word ----------------------------------------------------
    def status(self, sync: bool = False) -> int:
        """0, or the mark of the first bounded wait inside a kernel that gave up:
        (kernel family << 8) | place of the wait.  The word lives in pinned host memory
        that the GPU writes directly, so reading it costs nothing and waits for nothing;
        it tells of the kernels that have finished (``sync`` waits for all of them first)."""
        if sync:
            torch.cuda.synchronize()
        return int(self.lib.zlm_status())

    def clear_status(self) -> None:
        self.lib.zlm_status_clear()

    def check_status(self, sync: bool = False) -> None:
        """Raises if a kernel's bounded wait gave up: what that kernel computed, and
        everything after it, is not to be trusted.  The word is cleared, so that the
        caller may go on (the GPU and the library remain usable)."""
        code = self.status(sync)
        if code:
            self.clear_status()
            family = _STATUS_FAMILY.get(code >> 8, f"kernel family {code >> 8}")
            raise KernelError(f"a bounded wait inside a {family} kernel gave up (place {code & 0xff}, "
                              f"status {code:#x}): results since the last check are not valid")

    @staticmethod
    def _stream() -> c_void_p:
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    def check_linear(self, what: str, w: torch.Tensor) -> None:
        """Raises at once, with the weight's name, if no kernel takes a product with this
        weight [N, K]: the bf16 kernels read 16 bytes (8 elements) of a row at a time."""
        if w.dtype == torch.bfloat16 and w.shape[1] % 8 != 0:
            raise KernelError(f"{what} [{w.shape[0]}, {w.shape[1]}]: the bfloat16 kernels need an inner size "
                              f"that is a multiple of 8 (run this model with dtype float32)")

    # -- kernels ----------------------------------------------------------
    def embed(self, out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
        """out[t, :] = table[ids[t], :] widened to fp32."""
        T, H = out.shape
        assert out.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == H
        assert out.is_contiguous() and table.is_contiguous()
        self._call("zlm_embed", self._p(out), self._p(table), c_int(_dt(table)),
                   self._p(ids), c_int(T), c_int(H), c_int(table.shape[0]), self._stream())

    def rmsnorm(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float,
                rows: Optional[torch.Tensor] = None) -> None:
        """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * w; x is the fp32 stream."""
        R, H = out.shape
        assert x.dtype == torch.float32 and x.shape[1] == H and w.shape == (H,)
        assert out.is_contiguous() and x.is_contiguous() and w.is_contiguous()
        assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= R)
        halves, self._norm_halves = self._norm_halves, None
        ok, self._lazy_ok = self._lazy_ok, False
        if (halves is not None and ok and rows is None and out.dtype == torch.bfloat16
                and halves[0].data_ptr() == x.data_ptr() and tuple(halves[0].shape) == (R, H)
                and halves[4].data_ptr() == w.data_ptr()):
            # the product before left this norm's halves and only streaming products read ``out``: nothing to launch
            self._lazy = (out, x, w, float(eps)) + tuple(halves[1:4])
            return
        self._lazy = None
        taken = self._takes_shares(x, ACCUM) if (rows is None and x.shape[0] == R) else None
        if taken is not None:
            self._call("zlm_rmsnorm_shares", self._p(out), c_int(_dt(out)), self._p(x), self._p(w), c_int(_dt(w)),
                       c_int(R), c_int(H), c_float(eps), self._p(taken[0]), c_int(taken[1]), self._stream())
            return
        self._call("zlm_rmsnorm", self._p(out), c_int(_dt(out)), self._p(x),
                   self._p(w), c_int(_dt(w)), self._p(rows), c_int(R), c_int(H),
                   c_float(eps), self._stream())

    def swiglu(self, out: torch.Tensor, gu: torch.Tensor) -> None:
        """out[t, i] = silu(gu[t, i]) * gu[t, I + i]."""
        T, I = out.shape
        assert gu.shape == (T, 2 * I) and gu.dtype == out.dtype
        assert out.is_contiguous() and gu.is_contiguous()
        self._call("zlm_swiglu", self._p(out), self._p(gu), c_int(_dt(out)),
                   c_int(T), c_int(I), self._stream())

    def linear(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, accumulate: bool = False,
               impl: Optional[str] = None, defer: bool = False) -> None:
        """out = x @ w.T (out in x's dtype, or fp32), or out += x @ w.T into the fp32
        residual stream when ``accumulate``.  w is [N, K] row-major and is not written by any kernel
        of the same step (in a decode step the products' first loads of w do not wait for the kernels
        before them).  bf16 products pick
        their kernel by the number of tokens: "gemv" (register-fragment streaming, up to
        8), "tc" (TMA + tcgen05, from 9 on), "mma" (mma.sync, what the others do not take);
        ``impl`` forces one (tests).

        ``defer``: the caller expects ``rmsnorm`` (for a product into the stream) or
        ``qk_norm_rope_write`` (for a q/k/v projection) to read ``out`` next.  A few-token product
        that cuts K into shares may then leave them to that kernel, which adds them up on its way
        (two launches fewer per layer at 17 to 64 tokens); any other use of ``out`` through this
        class finishes the product first, so the hint is never wrong, only sometimes useless."""
        T, K = x.shape
        N = w.shape[0]
        if self._candidates is not None and self._candidates[0] == out.data_ptr():
            self._candidates = None         # whatever writes this tensor now, the old candidates are not its
        assert w.shape[1] == K and out.shape == (T, N) and w.dtype == x.dtype
        assert x.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
        ldx, ldy = x.stride(0), out.stride(0)
        if accumulate:
            assert out.dtype == torch.float32
        if x.dtype == torch.float32:
            assert out.dtype == torch.float32 and ldx == K
            self._call("zlm_gemm_f32", self._p(out), self._p(x),
                       self._p(w), c_int(T), c_int(N), c_int(K), c_int(ldy),
                       c_int(1 if accumulate else 0), self._stream())
            return
        if x.dtype != torch.bfloat16:
            raise KernelError(f"linear: unsupported dtype {x.dtype}")
        mode = ACCUM if accumulate else (STORE_F32 if out.dtype == torch.float32 else STORE)
        if mode == STORE:
            assert out.dtype == torch.bfloat16
        if accumulate and defer:
            hint, self._norm_hint = self._norm_hint, None
            if (hint is not None and impl is None and self.streams_weights(T, N) and out.is_contiguous()
                    and hint.is_contiguous() and tuple(hint.shape) == (N,)):
                self._gemv(out, x, w, T, N, K, ldx, ldy, ACCUM, norm_weight=hint)
                return
        if (defer and self.defer_shares and impl is None and mode in (ACCUM, STORE) and T > 16 and out.is_contiguous()
                and not self.streams_weights(T, N)):
            ks = int(self.lib.zlm_gemm_tc_shares_plan(c_int(T), c_int(N), c_int(K), c_int(ldx)))
            if ks > 1:
                self.flush_shares()
                scratch = self.scratch("gemm_tc.partials", ks * T * N, torch.float32, out.device)
                self._call("zlm_gemm_tc_shares", self._p(x), self._p(w), c_int(T), c_int(N), c_int(K), c_int(ldx),
                           self._p(scratch), self._stream())
                self._shares = (out, scratch, ks, mode)
                return
        self._bf16_product(out, x, w, T, N, K, ldx, ldy, mode, impl)

    def flush_shares(self) -> None:
        """Finishes a product that ``linear(defer=True)`` left in shares of K (its second kernel), and a
        norm that was left to the products after it."""
        self.finish_norm()
        self._norm_halves = None
        if self._shares is None:
            return
        out, scratch, ks, mode = self._shares
        self._shares = None
        T, N = out.shape
        self._call("zlm_gemm_tc_add_shares", self._p(out), self._p(scratch), c_int(T), c_int(N), c_int(out.stride(0)),
                   c_int(mode), c_int(ks), self._stream())

    def _takes_shares(self, t: torch.Tensor, mode: int):
        """The pending shares if they are those of ``t`` (whole, in this mode), else None after finishing them."""
        if self._shares is None:
            return None
        out, scratch, ks, m = self._shares
        if out.data_ptr() == t.data_ptr() and tuple(out.shape) == tuple(t.shape) and out.stride() == t.stride() and m == mode:
            self._shares = None
            return scratch, ks
        return None

    # outputs from which a product counts as "as wide as a vocabulary" (see streams_weights)
    WIDE_PRODUCT = 65536

    def streams_weights(self, tokens: int, N: int) -> bool:
        """Whether a bf16 product of this many tokens and N outputs runs as the register-fragment
        streaming product (else a tcgen05 form).  Measured at Qwen3-8B sizes: it wins up to 16
        tokens (a layer's four products at 9 / 16 tokens: 78 / 84 us against 88 / 90 us), except
        for products as wide as a vocabulary, whose thousand tiles the persistent tcgen05 form
        streams faster from 9 tokens on (191 against 197 to 216 us)."""
        return tokens <= 8 or (tokens <= 16 and N < self.WIDE_PRODUCT)

    def _bf16_product(self, out, x, w, T, N, K, ldx, ldy, mode, impl) -> None:
        if impl is None:
            # few tokens: the streaming product; from 17 tokens on the tcgen05 forms
            tc_ok = self.lib.zlm_gemm_tc_supported(T, N, K, ldx)
            small = self.streams_weights(T, N)
            impl = "gemv" if (small or (T <= 16 and not tc_ok)) else ("tc" if tc_ok else "mma")
        if impl == "tc":
            self.flush_shares()             # the shares' scratch is about to be written again
            ks = self.lib.zlm_gemm_tc_ksplit(T, N, K)
            scratch = self.scratch("gemm_tc.partials", ks * T * N, torch.float32, out.device) if ks > 1 else None
            self._call("zlm_gemm_tc", self._p(out), self._p(x), self._p(w),
                       c_int(T), c_int(N), c_int(K), c_int(ldx), c_int(ldy), c_int(mode), self._p(scratch),
                       self._stream())
            return
        if impl == "gemv":
            self._gemv(out, x, w, T, N, K, ldx, ldy, mode)
            return
        self._call("zlm_gemm_bf16_mma", self._p(out), self._p(x), self._p(w),
                   c_int(T), c_int(N), c_int(K), c_int(ldx), c_int(ldy), c_int(mode), self._stream())

    def _gemv(self, out, x, w, T, N, K, ldx, ldy, mode, norm_weight: Optional[torch.Tensor] = None) -> None:
        """The streaming product, with what it may carry beside its sums: candidates for the argmax of
        logits, the scale of a norm that was not run (``x`` is that norm's output), the halves of the
        norm that follows (``norm_weight``)."""
        lazy = self._lazy
        if not (lazy is not None and lazy[0].data_ptr() == x.data_ptr() and tuple(lazy[0].shape) == (T, K) and ldx == K):
            lazy = None
        nb = int(self.lib.zlm_gemv_blocks(c_int(N)))
        cv = ci = nxt = sq = None
        if mode == STORE_F32 and out.is_contiguous():
            # fp32 outputs of a few-token product are logits: the product also leaves, for every
            # token, the best of each block's 16 outputs, and ``argmax`` of the same tensor picks
            # among those candidates instead of reading the logits again
            cv = self.scratch("gemv.best_values", T * nb, torch.float32, out.device)
            ci = self.scratch("gemv.best_indices", T * nb, torch.int32, out.device)
        if norm_weight is not None:
            nxt = self.scratch("gemv.norm_rows", T * N, torch.bfloat16, out.device)
            sq = self.scratch("gemv.norm_squares", T * nb, torch.float32, out.device)
        # a norm not run: its rows times weight stand in for x, the scale comes from the sums of squares
        px = self._p(lazy[4]) if lazy is not None else self._p(x)
        self._call("zlm_gemv_bf16_norms", self._p(out), px, self._p(w), c_int(T), c_int(N), c_int(K),
                   c_int(ldx), c_int(ldy), c_int(mode), self._p(cv), self._p(ci),
                   self._p(lazy[5]) if lazy is not None else c_void_p(0), c_int(lazy[6] if lazy is not None else 0),
                   c_float(lazy[3] if lazy is not None else 0.0), self._p(norm_weight),
                   c_int(_dt(norm_weight) if norm_weight is not None else 0), self._p(nxt), self._p(sq), self._stream())
        if cv is not None:
            self._candidates = (out.data_ptr(), T, N, nb, cv, ci)
        if norm_weight is not None:
            self._norm_halves = (out, nxt, sq, nb, norm_weight)

    def set_gemm_form(self, form: Optional[str] = None, width: int = 0) -> None:
        """Forces the many-token tcgen05 product's form ("single": one block per tile,
        "pair": two blocks per tile with cta_group::2) and tile width (256, 240, 224; pairs also 128);
        None / 0 give the choice back to the dispatcher.  For tests and measurements."""
        code = {None: 0, "single": 1, "pair": 2}[form]
        if self.lib.zlm_gemm_tc_set_form(c_int(code), c_int(width)) != 0:
            raise KernelError(self.lib.zlm_last_error().decode())

    def set_prefill_attention_heads(self, heads: int = 0) -> None:
        """Forces how many heads of a kv group share a block of the tcgen05 prefill attention
        (1 or 2; 0 gives the choice back to the dispatcher).  For tests and measurements."""
        if self.lib.zlm_attention_prefill_tc_set_heads(c_int(heads)) != 0:
            raise KernelError(self.lib.zlm_last_error().decode())

    def linear_swiglu(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, impl: Optional[str] = None) -> None:
        """out[t, c] = silu(x[t] . gate_c) * (x[t] . up_c) in one pass over w (bf16).  w is
        [2I, K] with the rows in groups of 16: 8 gate channels, then the 8 matching up
        channels (``interleave_gate_up``); out is [T, I]."""
        T, K = x.shape
        N = w.shape[0]
        assert x.dtype == w.dtype == out.dtype == torch.bfloat16 and w.shape[1] == K and N % 16 == 0
        assert out.shape == (T, N // 2) and x.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
        self._bf16_product(out, x, w, T, N, K, x.stride(0), out.stride(0), SWIGLU, impl)

    def rope_table(self, out: torch.Tensor, inv_freq: torch.Tensor, n_rot: int, token_pos: torch.Tensor) -> None:
        """out [2, n_rot/2, T] fp32: cos and sin of token_pos[t] * inv_freq[i], the step's rotation
        table (the same for every layer with the same frequencies); tokens innermost, so that the
        32 token rows of a warp in the projection's epilogue read neighbouring floats."""
        T = token_pos.shape[0]
        assert out.dtype == torch.float32 and out.is_contiguous() and out.numel() == T * n_rot
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == n_rot and token_pos.dtype == torch.int32
        self._call("zlm_rope_table", self._p(out), self._p(inv_freq), c_int(n_rot), self._p(token_pos), c_int(T),
                   self._stream())

    def qkv_rope_supported(self, x: torch.Tensor, w: torch.Tensor, nq: int, nkv: int, hd: int, n_rot: int) -> bool:
        """Whether ``linear_qkv_rope`` takes this step: bf16, many tokens, heads that divide a tile."""
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            return False
        return bool(self.lib.zlm_gemm_tc_qkv_supported(c_int(x.shape[0]), c_int(w.shape[0]), c_int(w.shape[1]),
                                                       c_int(x.stride(0)), c_int(nq), c_int(nkv), c_int(hd), c_int(n_rot)))

    def linear_qkv_rope(self, q_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, q_w: Optional[torch.Tensor],
                        k_w: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                        token_pos: torch.Tensor, token_slot: torch.Tensor, block_table: Optional[torch.Tensor],
                        pool: Optional[torch.Tensor], nq: int, nkv: int, hd: int) -> None:
        """The fused q/k/v projection x @ w.T (w rows [q | k | v]) with its epilogue doing what
        ``qk_norm_rope_write`` does: per-head RMSNorm of q and k, rotation by ``cos_sin`` (from
        ``rope_table``), k and v into the paged pool; q_out [T, nq*hd] receives q.  With nkv == 0
        w holds q rows only."""
        T, K = x.shape
        N = w.shape[0]
        assert q_out.shape == (T, nq * hd) and q_out.dtype == torch.bfloat16 and q_out.stride(1) == 1
        assert w.shape == ((nq + 2 * nkv) * hd, K) and w.is_contiguous() and x.stride(1) == 1
        if nkv:
            assert pool is not None and pool.dtype == torch.bfloat16 and pool.is_contiguous()
            assert tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hd) and block_table.dtype == torch.int32
        if q_w is not None:
            assert q_w.shape == (hd,) and (nkv == 0 or (k_w is not None and k_w.dtype == q_w.dtype))
        if cos_sin is not None:
            assert cos_sin.dtype == torch.float32 and cos_sin.numel() == T * hd and cos_sin.is_contiguous()
        self._call("zlm_gemm_tc_qkv", self._p(q_out), self._p(x), self._p(w), c_int(T), c_int(N), c_int(K),
                   c_int(x.stride(0)), c_int(q_out.stride(0)), self._p(q_w), self._p(k_w),
                   c_int(_dt(q_w) if q_w is not None else F32), c_float(eps), self._p(cos_sin),
                   self._p(token_pos), self._p(token_slot), self._p(block_table),
                   c_int(block_table.stride(0) if block_table is not None else 0), self._p(pool), c_int(nq), c_int(nkv),
                   c_int(hd), self._stream())

    def qk_norm_rope_write(self, qkv: torch.Tensor, q_w: Optional[torch.Tensor],
                           k_w: Optional[torch.Tensor], eps: float,
                           inv_freq: Optional[torch.Tensor], n_rot: int, token_pos: torch.Tensor,
                           token_slot: torch.Tensor, block_table: Optional[torch.Tensor],
                           pool: Optional[torch.Tensor], nq: int, nkv: int, hd: int,
                           write: bool = True) -> None:
        """On qkv [T, (nq + 2 nkv) hd]: per-head RMSNorm of q and k (if weights are
        given), rotation of q and k by the token's position (if inv_freq is given); q is
        updated in place; with ``write`` k and v go to the token's place in the paged
        pool, without it k is updated in place and v is left alone.  With nkv == 0 only
        q is touched (a layer that reads another layer's cache)."""
        T = qkv.shape[0]
        assert qkv.shape[1] == (nq + 2 * nkv) * hd and qkv.stride(1) == 1
        has_norm = q_w is not None
        if has_norm:
            assert q_w.shape == (hd,) and (nkv == 0 or (k_w is not None and k_w.shape == (hd,) and k_w.dtype == q_w.dtype))
        if inv_freq is not None:
            assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == n_rot
        else:
            n_rot = 0
        write = bool(write and nkv)
        if write:
            assert pool is not None and pool.dtype == qkv.dtype and pool.is_contiguous()
            assert tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hd)
            assert block_table is not None and block_table.dtype == torch.int32
        taken = self._takes_shares(qkv, STORE) if T < 512 else None
        args = (self._p(qkv), c_int(_dt(qkv)), c_int(qkv.stride(0)),
                self._p(q_w), self._p(k_w), c_int(_dt(q_w) if has_norm else F32),
                c_int(1 if has_norm else 0), c_float(eps), self._p(inv_freq), c_int(n_rot),
                self._p(token_pos), self._p(token_slot),
                self._p(block_table), c_int(block_table.stride(0) if block_table is not None else 0),
                self._p(pool), c_int(nq), c_int(nkv), c_int(hd), c_int(1 if write else 0), c_int(T))
        if taken is not None:
            self._call("zlm_qk_norm_rope_write_shares", *args, self._p(taken[0]), c_int(taken[1]), self._stream())
        else:
            self._call("zlm_qk_norm_rope_write", *args, self._stream())

    def attention(self, out: torch.Tensor, q: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                  token_pos: torch.Tensor, token_slot: torch.Tensor, nq: int, nkv: int, hd: int,
                  scale: float, window: int, plan=None, len_bucket: Optional[int] = None) -> None:
        """out[t, h] = softmax(q[t, h] . K * scale) V over the keys [start, pos[t]] of the
        token's slot; q may be a column view of the fused qkv buffer.  ``plan`` is the
        step's context (one token per sequence: the split-KV kernel; whole prompts or
        chunks: the flash kernels; none: the generic kernel); ``len_bucket`` is the longest
        sequence in pages as ``attention_len_bucket`` rounds it (computed if absent)."""
        T = q.shape[0]
        assert out.shape == (T, nq * hd) and q.shape[1] == nq * hd and q.dtype == out.dtype == pool.dtype
        assert q.stride(1) == 1 and out.stride(1) == 1 and pool.is_contiguous()
        assert tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hd)
        if (plan is not None and plan.is_decode and q.dtype == torch.bfloat16
                and self.lib.zlm_attention_decode_supported(nq, nkv, hd)):
            if len_bucket is None:
                len_bucket = attention_len_bucket(plan.max_len)
            splits, per = decode_splits(T, nkv, len_bucket, self.decode_blocks or self.sm_count * DECODE_BLOCKS_PER_SM)
            part_o = part_ml = None
            if splits > 1:
                part_o = plan.scratch("attn.part_o", (T * nq * splits * hd,), torch.float32)
                part_ml = plan.scratch("attn.part_ml", (T * nq * splits * 2,), torch.float32)
            # (a decode step writes one position per sequence: every page below that one is from earlier
            # steps, and its load need not wait for the kernel that wrote this step's keys and values)
            self._call("zlm_attention_decode_fresh", self._p(out), c_int(out.stride(0)),
                       self._p(q), c_int(q.stride(0)), self._p(pool),
                       self._p(block_table), c_int(block_table.stride(0)),
                       self._p(token_pos), self._p(token_slot), c_int(T), c_int(nq),
                       c_int(nkv), c_int(hd), c_float(scale), c_int(window), c_int(splits), c_int(per),
                       self._p(part_o), self._p(part_ml), c_int(max(1, int(getattr(plan, "max_new", 1) or 1))),
                       self._stream())
            return
        if (plan is not None and not plan.is_decode and q.dtype == torch.bfloat16
                and getattr(plan, "cu_seqlens", None) is not None
                and self.lib.zlm_attention_prefill_supported(nq, nkv, hd)):
            impl = getattr(plan, "attention_impl", None)
            if impl != "mma" and self.lib.zlm_attention_prefill_tc_supported(nq, nkv, hd, q.stride(0), out.stride(0)):
                self._call("zlm_attention_prefill_tc", self._p(out), c_int(out.stride(0)),
                           self._p(q), c_int(q.stride(0)), c_int(T), self._p(pool),
                           ctypes.c_longlong(pool.shape[0]), self._p(block_table),
                           c_int(block_table.stride(0)), self._p(plan.cu_seqlens),
                           self._p(plan.seq_slot), self._p(plan.seq_start), c_int(plan.R),
                           c_int(plan.max_new), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_int(window),
                           self._stream())
                return
            self._call("zlm_attention_prefill", self._p(out), c_int(out.stride(0)),
                       self._p(q), c_int(q.stride(0)), self._p(pool),
                       self._p(block_table), c_int(block_table.stride(0)),
                       self._p(plan.cu_seqlens), self._p(plan.seq_slot),
                       self._p(plan.seq_start), c_int(plan.R), c_int(plan.max_new), c_int(nq),
                       c_int(nkv), c_int(hd), c_float(scale), c_int(window), self._stream())
            return
        self._call("zlm_attention_generic", self._p(out), c_int(out.stride(0)),
                   self._p(q), c_int(q.stride(0)), c_int(_dt(q)), self._p(pool),
                   self._p(block_table), c_int(block_table.stride(0)),
                   self._p(token_pos), self._p(token_slot), c_int(T), c_int(nq),
                   c_int(nkv), c_int(hd), c_float(scale), c_int(window), self._stream())

    def argmax(self, out: torch.Tensor, logits: torch.Tensor, fresh: bool = False) -> None:
        """out[r] = index of the highest logit of row r, ties to the lowest index.  ``fresh``: the
        caller vouches that ``logits`` is what ``linear`` wrote last into this tensor and nothing
        has written it since (the engine's logits on their way to the sampler); the few-token
        product then has left every block's best candidates, and the logits are not read again."""
        R, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
        cand = self._candidates if fresh else None
        if cand is not None and cand[0] == logits.data_ptr() and cand[1] >= R and cand[2] == V and logits.is_contiguous():
            # these logits came from the few-token product just before: it left the candidates
            _, _, _, nb, cv, ci = cand
            self._call("zlm_argmax_candidates", self._p(out), self._p(cv), self._p(ci), c_int(R), c_int(nb), self._stream())
            return
        sv = self.scratch("argmax.values", R * 64, torch.float32, logits.device)
        si = self.scratch("argmax.indices", R * 64, torch.int32, logits.device)
        self._call("zlm_argmax", self._p(out), self._p(logits), c_int(R), c_int(V),
                   c_int(logits.stride(0)), self._p(sv), self._p(si), self._stream())

    def set_pdl(self, on: bool) -> None:
        """Launch the decode-path kernels with programmatic dependent launch (a kernel's
        blocks are scheduled, and its weights start streaming, while the kernel before it
        drains) or in plain stream order."""
        self.lib.zlm_set_pdl(c_int(1 if on else 0))

    def gemm_tc_status(self) -> int:
        """0 unless a bounded wait inside a tcgen05 kernel (product or attention) gave up
        since the status was last cleared (synchronises)."""
        return self.status(sync=True)

    def test_bounded_wait(self, limit_ns: int):
        """Runs the tcgen05 kernels' give-up path on purpose, once, in a one-block kernel
        made of the same helpers (a wait with the limit ``limit_ns`` on a barrier at which
        nobody arrives), and returns (code it reported, other waits released by the abort
        flag, nanoseconds the kernel took, its TMA copy had landed)."""
        src = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
        out = torch.zeros(4, dtype=torch.int32, device="cuda")
        self._call("zlm_test_bounded_wait", self._p(src), self._p(out), ctypes.c_ulonglong(int(limit_ns)),
                   self._stream())
        torch.cuda.synchronize()
        code, released, ns, landed = out.tolist()
        return code, bool(released), ns, bool(landed)

    def sample(self, out: torch.Tensor, logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
               seed: int, request: torch.Tensor, position: torch.Tensor, form: Optional[str] = None) -> None:
        """out[r] = a draw from softmax(logits[r] / temperature) restricted to the top_k
        best and to the nucleus of mass top_p; the uniform of row r is a hash of
        (seed, request[r], position[r]).  ``form`` forces one of the kernel's two forms
        (tests): "cluster" (8 blocks per row, the row in distributed shared memory) or
        "block" (one block per row; rows too long for the cluster form)."""
        R, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
        assert request.dtype == torch.int32 and position.dtype == torch.int32
        self._call("zlm_sample", self._p(out), self._p(logits), c_int(R), c_int(V),
                   c_int(logits.stride(0)), c_float(temperature), c_int(top_k), c_float(top_p),
                   ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), self._p(request),
                   self._p(position), c_int({None: 0, "block": 1, "cluster": 2}[form]), self._stream())


_KERNELS: Optional[CudaKernels] = None
_VARIANT = ""


def set_build_variant(variant: str) -> None:
    """Which build of the library ``get_kernels`` loads: "" (the ordinary one) or "check"
    (the bounds-check build).  To be called before the first ``get_kernels``."""
    global _VARIANT, _KERNELS
    if _KERNELS is not None and _KERNELS.variant != variant:
        raise KernelError("the kernel library is loaded already; choose the build variant before first use")
    _VARIANT = variant


def get_kernels() -> CudaKernels:
    global _KERNELS
    if _KERNELS is None:
        _KERNELS = CudaKernels(variant=_VARIANT)
    return _KERNELS
