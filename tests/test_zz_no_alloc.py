"""The allocation-free decode attention (zlm_attention_decode_static), called
through its exported C symbol as a caller outside this library would, against
the existing entry point (zlm_attention_decode) with scratch that the test
allocates.  It is for callers that cannot call cudaMalloc when they need
attention: inside another program's memory plan, or where the device-wide
synchronisation of an allocation is not acceptable.

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.  It passes alone in a fresh process and after the
other tests (the built-in scratch keeps what earlier calls left in it; the test
makes two calls in a row with different inputs to show that this does no harm).
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

PAGE = 64
SCRATCH_FLOATS = 4 * 1024 * 1024


def _lib():
    from zlm_b200.csrc.build import library_path
    lib = ctypes.CDLL(library_path())
    lib.zlm_last_error.restype = ctypes.c_char_p
    for name in ("zlm_attention_decode", "zlm_attention_decode_static"):
        getattr(lib, name).restype = c_int
    return lib


def _case(seed, lens, nq, nkv, hd):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + PAGE - 1) // PAGE for n in lens) + 3
    pool = torch.randn((n_pages, 2, nkv, PAGE, hd), generator=g).to(torch.bfloat16).cuda()
    table = torch.zeros((len(lens), 16), dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).tolist()
    for s, n in enumerate(lens):
        for lp in range((n + PAGE - 1) // PAGE):
            table[s, lp] = perm.pop()
    q = torch.randn((len(lens), nq * hd), generator=g).to(torch.bfloat16).cuda()
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    slot = torch.arange(len(lens), dtype=torch.int32).cuda()
    return q, pool, table.cuda(), pos, slot


def _run(lib, static, q, pool, table, pos, slot, nq, nkv, hd, splits, window=0):
    T = q.shape[0]
    per = -(-(int(pos.max()) // PAGE + 1) // splits)          # pages per split, so that the splits cover the longest
    out = torch.zeros((T, nq * hd), dtype=torch.bfloat16, device="cuda")
    st = c_void_p(torch.cuda.current_stream().cuda_stream)
    common = (c_void_p(out.data_ptr()), c_int(out.stride(0)), c_void_p(q.data_ptr()), c_int(q.stride(0)),
              c_void_p(pool.data_ptr()), c_void_p(table.data_ptr()), c_int(table.stride(0)),
              c_void_p(pos.data_ptr()), c_void_p(slot.data_ptr()), c_int(T), c_int(nq), c_int(nkv), c_int(hd),
              c_float(1.0 / math.sqrt(hd)), c_int(window), c_int(splits), c_int(per))
    free = None
    if static:
        torch.cuda.synchronize()
        free = torch.cuda.mem_get_info()[0]          # the device's free memory: any allocation shows, whoever makes it
        rc = lib.zlm_attention_decode_static(*common, st)
        torch.cuda.synchronize()
        free -= torch.cuda.mem_get_info()[0]
    else:
        part_o = torch.empty(T * nq * splits * hd, dtype=torch.float32, device="cuda")
        part_ml = torch.empty(T * nq * splits * 2, dtype=torch.float32, device="cuda")
        rc = lib.zlm_attention_decode(*common, c_void_p(part_o.data_ptr()), c_void_p(part_ml.data_ptr()), st)
    torch.cuda.synchronize()
    return rc, out, free


def _plain(q, pool, table, pos, slot, nq, nkv, hd, window):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from cpu_kernels import PlainKernels
    want = torch.empty(q.shape, dtype=torch.bfloat16)
    PlainKernels().attention(want, q.cpu(), pool.cpu(), table.cpu(), pos.cpu(), slot.cpu(), nq, nkv, hd,
                             1.0 / math.sqrt(hd), window)
    return want


def test_no_alloc_decode_attention_matches_twice():
    """Same kernels in the same order as the entry point with the caller's scratch, so the
    results must be the same bits; both must agree with the plain attention.  The first
    call warms the entry up (its look-up of the array's address); from then on the
    device's free memory must not move across a call.  The second and third case use
    fewer partials than the first, so that what the first left lies beyond them; one case
    has a window, one a single split (no scratch at all)."""
    lib = _lib()
    nq, nkv, hd = 8, 2, 128
    cases = ((1, [300, 64, 5, 700], 4, 0), (2, [129, 513], 3, 0), (3, [700, 64, 333], 2, 100),
             (4, [200, 90], 1, 0), (1, [300, 64, 5, 700], 4, 0))
    for i, (seed, lens, splits, window) in enumerate(cases):
        args = _case(seed, lens, nq, nkv, hd)
        rc0, want, _ = _run(lib, False, *args, nq, nkv, hd, splits, window)
        assert rc0 == 0, lib.zlm_last_error().decode()
        rc1, got, grew = _run(lib, True, *args, nq, nkv, hd, splits, window)
        assert rc1 == 0, lib.zlm_last_error().decode()
        assert torch.equal(got, want), f"case {i}: the two entry points differ"
        if i > 0:
            assert grew == 0, f"case {i}: the device's free memory fell by {grew} bytes during the call"
        plain = _plain(*args, nq, nkv, hd, window)
        torch.testing.assert_close(got.float().cpu(), plain.float(), atol=3e-2, rtol=3e-2)
        assert want.float().abs().sum() > 0


def test_no_alloc_decode_attention_refuses_what_does_not_fit():
    lib = _lib()
    nq, nkv, hd, splits = 32, 8, 128, 16
    T = SCRATCH_FLOATS // (nq * splits * (hd + 2)) + 1
    args = _case(3, [65] * T, nq, nkv, hd)
    rc, _, _ = _run(lib, True, *args, nq, nkv, hd, splits)
    assert rc != 0
    msg = lib.zlm_last_error().decode()
    assert "built-in scratch" in msg and str(SCRATCH_FLOATS) in msg
