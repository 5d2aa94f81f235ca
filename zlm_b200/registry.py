"""The registries: architecture name -> typed configuration, and part kind ->
part class.  Everything that builds a model goes through these tables, so a new
mixer, feed-forward, norm, position encoding, block arrangement or whole
architecture is added by registering it; no file of the framework changes.

The reference keeps one table of architectures and looks a model up by the name
in its metadata (src/architectures/core/root.zig:23-37); an unknown name is an
error there too (src/architectures/root.zig:37-39).
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping, Type

from .config.spec import ConfigError, ModelSpec

# architecture name (config.json "architectures"[0]) -> configuration class with
# from_dict(mapping) and to_model_spec()
ARCHITECTURES: Dict[str, Any] = {}

# part registries: kind -> class
MIXERS: Dict[str, Any] = {}
FEED_FORWARDS: Dict[str, Any] = {}
NORMS: Dict[str, Any] = {}
POSITION_ENCODINGS: Dict[str, Any] = {}
ARRANGEMENTS: Dict[str, Any] = {}
EMBEDDINGS: Dict[str, Any] = {}
HEADS: Dict[str, Any] = {}


def _register(table: Dict[str, Any], what: str, name: str):
    def deco(cls):
        if name in table and table[name] is not cls:
            raise ValueError(f"{what} '{name}' is already registered")
        table[name] = cls
        return cls
    return deco


def register_architecture(name: str):
    return _register(ARCHITECTURES, "architecture", name)


def register_mixer(kind: str):
    return _register(MIXERS, "mixer", kind)


def register_feed_forward(kind: str):
    return _register(FEED_FORWARDS, "feed-forward", kind)


def register_norm(kind: str):
    return _register(NORMS, "norm", kind)


def register_position_encoding(kind: str):
    return _register(POSITION_ENCODINGS, "position encoding", kind)


def register_arrangement(kind: str):
    return _register(ARRANGEMENTS, "block arrangement", kind)


def register_embedding(kind: str):
    return _register(EMBEDDINGS, "embedding", kind)


def register_head(kind: str):
    return _register(HEADS, "head", kind)


def lookup(table: Dict[str, Any], what: str, kind: str):
    try:
        return table[kind]
    except KeyError:
        raise ConfigError(f"unknown {what} '{kind}'; registered: {sorted(table)}") from None


def architecture_name(config: Mapping[str, Any]) -> str:
    archs = config.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a list with the model class name")
    return archs[0]


def config_from_dict(config: Mapping[str, Any]):
    """The typed configuration for a config.json mapping, chosen by its
    ``architectures[0]``."""
    name = architecture_name(config)
    if name not in ARCHITECTURES:
        raise ConfigError(f"unsupported architecture '{name}'; this build knows {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[name].from_dict(config)


def config_from_folder(folder: str):
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: must hold a JSON object")
    return config_from_dict(d)
