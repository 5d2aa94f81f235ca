"""Reading and writing the safetensors container: an 8-byte little-endian header
length, a JSON header {name: {dtype, shape, data_offsets}}, then raw
little-endian tensor bytes.  Tensors are memory-mapped and handed out one at a
time, so a model larger than host memory never sits there whole.

The reference keeps weights in its own memory-mapped image and looks tensors up
by name (src/image/zcom.zig:111-168); this is the same idea for the checkpoint
format that the architecture's own tooling writes.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: truncated (header of {hlen} bytes in a file of {size})")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        data_size = size - self._base
        for name, e in header.items():
            try:
                dt, shape, (b, end) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for '{name}'") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            n = 1
            for s in shape:
                n *= s
            if end - b != n * _DTYPES[dt][1]:
                raise SafetensorsError(f"{path}: tensor '{name}' byte range does not match its shape")
            if b < 0 or end > data_size:
                raise SafetensorsError(f"{path}: truncated (tensor '{name}' ends at byte {end} of {data_size})")
            self.entries[name] = (dt, shape, b, end)

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only memory: copy or
        move it before writing)."""
        dt, shape, b, end = self.entries[name]
        tdt = _DTYPES[dt][0]
        if end == b:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self._base + b:self._base + end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # torch warns about the read-only buffer
            t = torch.frombuffer(buf, dtype=tdt)
        return t.reshape(shape)

    def close(self) -> None:
        # tensors handed out may still view the map; let the GC end it
        self._f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] | None = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot write dtype {t.dtype} ('{name}')")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes()
                        if t.dtype != torch.bool else t.to(torch.uint8).numpy().tobytes())


def open_model_files(folder: str) -> Dict[str, SafetensorsFile]:
    """name -> the file that holds it, for ``model.safetensors`` or a sharded
    checkpoint with ``model.safetensors.index.json``.  A name found in two
    shards is an error."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    paths: List[str] = []
    if os.path.isfile(single):
        paths = [single]
    elif os.path.isfile(index):
        with open(index) as f:
            wm = json.load(f).get("weight_map", {})
        paths = sorted({os.path.join(folder, p) for p in wm.values()})
    else:
        raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")
    where: Dict[str, SafetensorsFile] = {}
    for p in paths:
        if not os.path.isfile(p):
            raise SafetensorsError(f"{folder}: shard {os.path.basename(p)} named by the index is missing")
        sf = SafetensorsFile(p)
        for n in sf.names():
            if n in where:
                raise SafetensorsError(f"tensor '{n}' appears in {where[n].path} and {p}")
            where[n] = sf
    return where
