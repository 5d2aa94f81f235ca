"""Random weights from a configuration and a seed: tensors in memory, or a model
folder (config.json + model.safetensors) that the loader reads back.

Matrices and the embedding are N(0, 0.02); norm weights are 1 + N(0, 0.02).
Each tensor has its own generator seeded from (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or in which order they are
made.  (The reference ships no weights and tests on integer patterns,
src/kernels/transformer/attention_test.zig:46-128; random folders are this
library's way to exercise the whole path.)
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Mapping

import torch

from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors

STD = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec: ParamSpec, seed: int, device, dtype: torch.dtype) -> torch.Tensor:
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    n = 1
    for s in spec.shape:
        n *= s
    # generated in fp32 in slices, so that a large matrix never needs an fp32 copy of itself
    out = torch.empty(n, dtype=dtype, device=device)
    step = 1 << 26
    for b in range(0, n, step):
        e = min(n, b + step)
        t = torch.randn(e - b, generator=g, device=device, dtype=torch.float32) * STD
        if spec.init == "one_plus_normal":
            t += 1.0
        elif spec.init != "normal":
            raise ValueError(f"unknown init '{spec.init}' for {name}")
        out[b:e] = t.to(dtype)
    return out.view(*spec.shape)


def random_tensors(expected: Mapping[str, ParamSpec], seed: int, device="cpu",
                   dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    """name -> random tensor for every expected, non-ignorable tensor.  ``dtype``
    is the storage dtype of float tensors."""
    return {n: random_tensor(n, p, seed, device, dtype) for n, p in expected.items() if not p.ignorable}


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.float32) -> None:
    """Writes ``config.json`` and ``model.safetensors`` for the typed configuration
    ``config`` (an object with to_dict() and to_model_spec())."""
    from ..parts.model import DecoderModel
    os.makedirs(folder, exist_ok=True)
    model = DecoderModel(config.to_model_spec())
    tensors = random_tensors(model.param_specs(), seed, "cpu", dtype)
    d = config.to_dict()
    d["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, {"format": "pt"})
