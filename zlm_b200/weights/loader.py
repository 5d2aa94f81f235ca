"""Binding checkpoint tensors to the tensors a model expects, by name.

The loader compares the set of names and shapes in the file with what the
model's parts declare and reports every problem in one error: missing tensors,
unexpected tensors, wrong shapes.  (The reference resolves each role to a
tensor by formatted name and fails with a shape error at first use:
src/tuner/compile.zig:295-311, src/kernels/linear/matvec/form/single.zig:172-175;
failing at load with the whole list is kinder.)

Dtype policy: matrices go to the compute dtype (bfloat16 or float32); vectors
(norm weights) stay 32-bit if the file stores them so; integer tables become
int32.  In float32 mode every float tensor is widened to float32.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import SafetensorsError, open_model_files


class WeightError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the names."""

    def __init__(self, folder: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: List[Tuple[str, str]] = ()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"{folder}: the weights do not fit the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unsupported dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {dt}" for n, dt in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def target_dtype(spec: ParamSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.kind == "int":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if spec.kind == "vector" and stored in (torch.float32, torch.float16):
        return torch.float32
    return compute


def check_names(folder: str, expected: Mapping[str, ParamSpec], shapes: Mapping[str, Tuple[int, ...]],
                dtypes: Mapping[str, torch.dtype]) -> None:
    missing = [n for n, p in expected.items() if n not in shapes and not p.ignorable]
    unexpected = [n for n in shapes if n not in expected]
    wrong = [(n, tuple(shapes[n]), tuple(p.shape)) for n, p in expected.items()
             if n in shapes and tuple(shapes[n]) != tuple(p.shape) and not p.ignorable]
    bad_dt = []
    for n, p in expected.items():
        if n in dtypes and not p.ignorable:
            ok = dtypes[n] in (_INTS if p.kind == "int" else _FLOATS)
            if not ok:
                bad_dt.append((n, str(dtypes[n])))
    if missing or unexpected or wrong or bad_dt:
        raise WeightError(folder, sorted(missing), sorted(unexpected), sorted(wrong), sorted(bad_dt))


def load_weights(folder: str, expected: Mapping[str, ParamSpec], compute: torch.dtype,
                 device) -> Dict[str, torch.Tensor]:
    """name -> tensor on ``device`` for every expected tensor of the checkpoint in
    ``folder``."""
    try:
        where = open_model_files(folder)
    except SafetensorsError as e:
        raise WeightError(str(e), [], [], []) from None
    shapes = {n: f.shape(n) for n, f in where.items()}
    dtypes = {n: f.dtype(n) for n, f in where.items()}
    check_names(folder, expected, shapes, dtypes)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if name not in where or (spec.ignorable and tuple(shapes[name]) != tuple(spec.shape)):
            continue
        if spec.ignorable:
            continue
        src = where[name].tensor(name)
        dt = target_dtype(spec, src.dtype, compute)
        # to(device) first when it narrows nothing: the cast then runs on the GPU
        out[name] = src.to(device=device).to(dt).contiguous()
    return out
