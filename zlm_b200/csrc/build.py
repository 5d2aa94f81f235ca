"""Builds the CUDA kernel library in-tree with nvcc for sm_100a.

The library is plain CUDA behind ``extern "C"`` entry points (no torch headers),
so a cold build is a handful of nvcc calls run in parallel.  It is rebuilt when
a source changed (content hash), and a line is printed for every file so that a
first call that has to compile shows progress.

Two variants: the ordinary library, and ``variant="check"``, the bounds-check build
(``-DZLM_BOUNDS_CHECK``, ``libzlm_b200_check.so``), in which every global-memory
access of the hand-written kernels is first compared with the tensors the caller
passed; an access outside them is counted, recorded and skipped (nothing traps).
It stands where a memory checker would: ``python -m zlm_b200.csrc.build check``
builds it, ``CudaKernels(variant="check")`` loads it.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libzlm_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
# variant -> (library name, object folder, extra nvcc flags)
VARIANTS = {
    "": (LIB_NAME, "_build", []),
    "check": ("libzlm_b200_check.so", "_build_check", ["-DZLM_BOUNDS_CHECK"]),
}


def _variant(variant: str):
    try:
        return VARIANTS[variant or ""]
    except KeyError:
        raise ValueError(f"unknown build variant {variant!r}; known: {sorted(VARIANTS)}") from None


def _say(msg: str) -> None:
    print(f"[zlm_b200 build] {msg}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def source_hash(variant: str = "") -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(HERE)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(HERE, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + _variant(variant)[2]).encode())
    return h.hexdigest()


def find_nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and os.path.isfile(os.path.join(cand, "bin", "nvcc")):
            return os.path.join(cand, "bin", "nvcc")
    n = shutil.which("nvcc")
    if n:
        return n
    raise RuntimeError("nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); "
                       "the zlm_b200 kernels cannot be built")


def _writable(d: str) -> bool:
    try:
        os.makedirs(d, exist_ok=True)
        with tempfile.NamedTemporaryFile(dir=d):
            pass
        return True
    except OSError:
        return False


def library_path(build_if_needed: bool = True, verbose: bool = True, variant: str = "") -> str:
    """Path of an up-to-date kernel library, building it first if needed."""
    lib_name, obj_name, extra = _variant(variant)
    want = source_hash(variant)
    lib = os.path.join(HERE, lib_name)
    stamp = lib + ".hash"
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return lib
    if not build_if_needed:
        raise RuntimeError(f"{lib} is missing or stale")
    out_dir = HERE
    if not _writable(os.path.join(HERE, obj_name)):
        out_dir = os.path.join(tempfile.gettempdir(), f"zlm_b200_{os.getuid()}_{want[:16]}")
        lib = os.path.join(out_dir, lib_name)
        stamp = lib + ".hash"
        if os.path.isfile(lib) and os.path.isfile(stamp):
            return lib
    build(out_dir, lib, verbose, obj_name, extra)
    with open(stamp, "w") as f:
        f.write(want)
    return lib


def build(out_dir: str, lib: str, verbose: bool = True, obj_name: str = "_build", extra_flags=()) -> None:
    nvcc = find_nvcc()
    obj_dir = os.path.join(out_dir, obj_name)
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} (first call only)")

    def compile_one(src: str) -> str:
        obj = os.path.join(obj_dir, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    objs = []
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        futs = {ex.submit(compile_one, s): s for s in srcs}
        for i, fut in enumerate(as_completed(futs), 1):
            objs.append(fut.result())
            if verbose:
                _say(f"  [{i}/{len(srcs)}] {futs[fut]} done ({time.time() - t0:.0f}s)")
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp, *sorted(objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking {lib} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f}s")


if __name__ == "__main__":
    print(library_path(variant=sys.argv[1] if len(sys.argv) > 1 else ""))
