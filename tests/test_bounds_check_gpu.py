"""The bounds-check build of the kernel library (``-DZLM_BOUNDS_CHECK``), which stands
where a memory checker would: the kernel tests and a tiny engine run again, in a process
of their own, against a library in which every global-memory access of the hand-written
kernels is first compared with the tensors the call was given.  An access outside them is
counted and skipped (nothing traps), and the call raises.  One test shows that the check
itself sees a stray access: a kernel told to write more rows than the tensor it was given
holds (inside a larger buffer that the test owns, so nothing can fault either way)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=900):
    r = subprocess.run([sys.executable, *args], cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    return r.returncode, r.stdout[-4000:] + r.stderr[-4000:]


def test_kernels_and_a_tiny_engine_stay_inside_their_tensors():
    rc, out = _run(["-m", "pytest", "-x", "-q", "--zlm-bounds-check", "-m", "gpu", "-p", "no:cacheprovider",
                    "tests/test_kernels_gpu.py", "tests/test_sampler_gpu.py",
                    "tests/test_engine_gpu.py::test_unequal_batches_reuse_slots",
                    "tests/test_engine_gpu.py::test_first_tokens_and_chunks"])
    assert rc == 0, out
    assert " passed" in out and "failed" not in out, out


STRAY = r"""
import ctypes, sys, torch
sys.path.insert(0, "tests")
from zlm_b200.kernels import CudaKernels, KernelError
K = CudaKernels(variant="check")
assert K.bounds_check
H, V, T = 64, 32, 8
table = torch.randn(V, H, device="cuda")
ids = torch.arange(T, dtype=torch.int32, device="cuda")
big = torch.zeros(T, H, device="cuda")
out = big[: T // 2]                       # the tensor the call is given: half of the rows it will write
try:
    K._call("zlm_embed", K._p(out), K._p(table), ctypes.c_int(0), K._p(ids), ctypes.c_int(T), ctypes.c_int(H),
            ctypes.c_int(V), K._stream())
except KernelError as e:
    assert "outside the tensors passed" in str(e), e
    torch.cuda.synchronize()
    assert torch.equal(big[: T // 2], table[: T // 2]), "rows inside the tensor must be written"
    assert float(big[T // 2:].abs().sum()) == 0.0, "rows outside the tensor must have been skipped"
    K.embed(big, table, ids)              # the library goes on
    assert torch.equal(big, table[:T])
    print("stray access seen and skipped")
    sys.exit(0)
print("the stray access went unseen")
sys.exit(1)
"""


def test_a_stray_access_is_seen_and_skipped():
    rc, out = _run(["-c", STRAY], timeout=300)
    assert rc == 0 and "stray access seen and skipped" in out, out
