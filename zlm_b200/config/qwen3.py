"""Typed configuration of the Qwen3 dense architecture, read from its own
``config.json`` keys, and its lowering to a ``ModelSpec``.

Keys and defaults follow the reference's typed config
(src/architectures/impl/qwen3/config.zig:26-57): layer count, width, context
length, feed-forward width and head count are required; the KV head count
defaults to the head count, the head size to width / heads, the norm epsilon to
1e-6 and the rotary base to 1,000,000 (float or integer accepted).  Tensor names
are the checkpoint's (``model.layers.N.self_attn.q_proj.weight``, ...); the role
table mirrors src/architectures/impl/qwen3/names.zig:8-26.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .spec import (ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                   optional, require)

ARCHITECTURE = "Qwen3ForCausalLM"

# keys that a ``rope_parameters`` / ``rope_scaling`` object may hold while still meaning
# plain rotary; anything else (factor, beta_fast, mrope_section, ...) changes the angles
_PLAIN_ROPE_KEYS = {"rope_theta", "rope_type", "type", "partial_rotary_factor"}


def _is_plain_rope(p: Mapping[str, Any]) -> bool:
    if not isinstance(p, Mapping):
        return False
    if any(k not in _PLAIN_ROPE_KEYS for k in p):
        return False
    kind = p.get("rope_type", p.get("type", "default"))
    if kind not in (None, "default"):
        return False
    return p.get("partial_rotary_factor", 1.0) in (1, 1.0, None)


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    # window of each layer in keys (0: all keys), from layer_types /
    # use_sliding_window / sliding_window / max_window_layers
    layer_windows: Tuple[int, ...]
    eos_token_ids: Tuple[int, ...] = ()

    # ---- reading -----------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        hidden = require(d, "hidden_size", int)
        layers = require(d, "num_hidden_layers", int)
        heads = require(d, "num_attention_heads", int)
        kv_heads = optional(d, "num_key_value_heads", int, heads)
        if heads <= 0 or kv_heads <= 0 or layers <= 0 or hidden <= 0:
            raise ConfigError("config.json: sizes must be positive")
        head_dim = optional(d, "head_dim", int, hidden // heads)
        inter = require(d, "intermediate_size", int)
        vocab = require(d, "vocab_size", int)
        max_pos = require(d, "max_position_embeddings", int)
        eps = optional(d, "rms_norm_eps", float, 1e-6)
        theta = cls._rope_theta(d)
        tied = optional(d, "tie_word_embeddings", bool, False)

        if heads % kv_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads={heads} is not a multiple of "
                f"num_key_value_heads={kv_heads}")
        if head_dim <= 0 or head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim={head_dim} must be even (rotary pairs)")
        if optional(d, "attention_bias", bool, False):
            raise ConfigError("config.json: attention_bias=true is not supported (Qwen3 dense has no bias)")
        scaling = d.get("rope_scaling")
        if scaling is not None and not _is_plain_rope(scaling):
            raise ConfigError("config.json: rope_scaling is not supported (plain rotary only)")
        if optional(d, "partial_rotary_factor", float, 1.0) != 1.0:
            raise ConfigError("config.json: partial_rotary_factor must be 1 (the whole head is rotated)")
        act = optional(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act='{act}' is not supported (silu only)")
        for k in ("num_experts", "num_local_experts", "num_experts_per_tok"):
            if d.get(k):
                raise ConfigError(f"config.json: '{k}' belongs to a mixture-of-experts model; "
                                  "this library builds Qwen3 dense only")
        if vocab <= 0 or inter <= 0 or max_pos <= 0 or eps <= 0 or theta <= 0:
            raise ConfigError("config.json: vocab_size, intermediate_size, "
                              "max_position_embeddings, rms_norm_eps and rope_theta must be positive")

        windows = cls._windows(d, layers)

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: 'eos_token_id' must be an integer or a list, got {eos!r}")

        return cls(hidden, layers, heads, kv_heads, head_dim, inter, vocab, max_pos,
                   eps, theta, tied, windows, eos_ids)

    @staticmethod
    def _rope_theta(d: Mapping[str, Any]) -> float:
        """The rotary base: the top-level ``rope_theta``, or ``rope_parameters.rope_theta``
        where a newer writer of config.json has moved it (the two must agree if both are
        there); default 1,000,000, float or integer
        (src/architectures/impl/qwen3/config.zig:39-40).  ``rope_parameters`` may say
        nothing but plain rotary: any other ``rope_type``, a ``factor`` or a partial
        rotation is refused rather than ignored."""
        top = optional(d, "rope_theta", float, None)
        params = d.get("rope_parameters")
        if params is None:
            return 1_000_000.0 if top is None else top
        if not isinstance(params, Mapping):
            raise ConfigError(f"config.json: 'rope_parameters' must be an object, got {params!r}")
        if not _is_plain_rope(params):
            raise ConfigError(
                f"config.json: rope_parameters={dict(params)!r} asks for scaled or partial rotary; "
                "plain rotary only (rope_type 'default', no factor, partial_rotary_factor 1)")
        inner = optional(params, "rope_theta", float, None)
        if top is not None and inner is not None and top != inner:
            raise ConfigError(f"config.json: rope_theta={top} and rope_parameters.rope_theta={inner} differ")
        if inner is not None:
            return inner
        return 1_000_000.0 if top is None else top

    @staticmethod
    def _windows(d: Mapping[str, Any], layers: int) -> Tuple[int, ...]:
        window = optional(d, "sliding_window", int, 0)
        use = optional(d, "use_sliding_window", bool, False)
        types = d.get("layer_types")
        if types is not None:
            if not isinstance(types, list) or len(types) != layers:
                raise ConfigError(f"config.json: 'layer_types' must list {layers} layers")
            out = []
            for i, t in enumerate(types):
                if t == "full_attention":
                    out.append(0)
                elif t == "sliding_attention":
                    if window <= 0:
                        raise ConfigError("config.json: layer_types names sliding_attention "
                                          "but 'sliding_window' is not a positive integer")
                    out.append(window)
                else:
                    raise ConfigError(f"config.json: layer_types[{i}]='{t}' is not known")
            return tuple(out)
        if use:
            if window <= 0:
                raise ConfigError("config.json: use_sliding_window=true needs a positive 'sliding_window'")
            first = optional(d, "max_window_layers", int, layers)
            return tuple(window if i >= first else 0 for i in range(layers))
        return tuple(0 for _ in range(layers))

    @classmethod
    def from_folder(cls, folder: str) -> "Qwen3Config":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_dict(json.load(f))

    # ---- writing -----------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "rope_scaling": None,
        }
        if any(self.layer_windows):
            d["use_sliding_window"] = True
            d["sliding_window"] = max(self.layer_windows)
            d["layer_types"] = ["sliding_attention" if w else "full_attention"
                                for w in self.layer_windows]
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- lowering ----------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        if len(set(w for w in self.layer_windows if w)) > 1:
            raise ConfigError("config.json: one sliding_window for all sliding layers")
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            position = {"kind": "rope_half_split", "theta": self.rope_theta,
                        "head_dim": self.head_dim, "n_rot": self.head_dim}
            mixer = PartSpec("gqa_attention", {
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qk_norm": True,
                "qk_norm_eps": self.rms_norm_eps,
                "window": self.layer_windows[i],
                "position": position,
            }, prefix=p + "self_attn.")
            ffn = PartSpec("swiglu", {"intermediate_size": self.intermediate_size},
                           prefix=p + "mlp.")
            norm_a = PartSpec("rms_norm", {"eps": self.rms_norm_eps},
                              prefix=p + "input_layernorm.")
            norm_f = PartSpec("rms_norm", {"eps": self.rms_norm_eps},
                              prefix=p + "post_attention_layernorm.")
            layers.append(LayerSpec("pre_norm", mixer, ffn, norm_a, norm_f))
        spec = ModelSpec(
            architecture=ARCHITECTURE,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_position=self.max_position_embeddings,
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            embedding=PartSpec("token_embedding", {}, prefix="model.embed_tokens."),
            final_norm=PartSpec("rms_norm", {"eps": self.rms_norm_eps}, prefix="model.norm."),
            head=PartSpec("lm_head", {"tied": self.tie_word_embeddings}, prefix="lm_head."),
        )
        spec.validate()
        return spec
