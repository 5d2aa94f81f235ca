"""Architecture-neutral description of a decoder: which parts each layer is made
of, with which sizes and constants, and in which order the layers run.

A typed architecture configuration (for instance ``Qwen3Config``) is read from
the keys of its own ``config.json`` and lowered to a ``ModelSpec``.  Everything
below the configuration (weights, parts, cache, engine) sees only the
``ModelSpec``; no size or constant lives in code.

The reference declares a model the same way: a table of semantic instructions
per layer plus a per-layer cache declaration, not forward code
(src/architectures/core/graph.zig:167-176, src/architectures/core/kv.zig:6-38).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A configuration that is missing a key, or holds a value this library
    refuses.  The message names the key."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered ``kind`` and its parameters.

    ``prefix`` is put before the part's local tensor names (``q_proj.weight``)
    to form checkpoint names; ``rename`` maps a local name to another local name
    for checkpoints that call the tensor differently.
    """
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""
    rename: Mapping[str, str] = field(default_factory=dict)

    def tensor_name(self, local: str) -> str:
        return self.prefix + self.rename.get(local, local)


@dataclass(frozen=True)
class LayerSpec:
    """A block: how a mixer and a feed-forward are arranged around the residual
    stream, and the norms that go with them.  ``arrangement`` names a registered
    block class (``pre_norm``: h += mixer(norm(h)); h += ffn(norm(h)))."""
    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers`` (a layer may
    be named by several entries and then shares its weights).  ``cache_of`` is
    the index of the schedule entry whose cache this entry reads instead of
    keeping one of its own (None: its own)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ConfigError(f"schedule[{i}] names layer {e.layer}, model has {n}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ConfigError(
                        f"schedule[{i}].cache_of={e.cache_of} must name an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(
                        f"schedule[{i}].cache_of={e.cache_of} names an entry without a cache of its own")


def require(d: Mapping[str, Any], key: str, typ) -> Any:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing key '{key}'")
    return coerce(d[key], key, typ)


def optional(d: Mapping[str, Any], key: str, typ, default) -> Any:
    if key not in d or d[key] is None:
        return default
    return coerce(d[key], key, typ)


def coerce(v: Any, key: str, typ) -> Any:
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                return int(v)
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
        return v
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: '{key}' must be a string, got {v!r}")
        return v
    raise TypeError(typ)
