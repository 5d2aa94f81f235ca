"""Registers the Qwen3 dense architecture: ``Qwen3ForCausalLM`` -> ``Qwen3Config``.
The model itself is the generic ``DecoderModel`` built from the specification
that the configuration lowers to; there is no Qwen3 forward code.
(The reference does the same: src/architectures/impl/qwen3/arch.zig:126-139 is
a bundle of declarations, "no forward logic".)"""
from ..config.qwen3 import ARCHITECTURE, Qwen3Config
from ..registry import register_architecture

register_architecture(ARCHITECTURE)(Qwen3Config)
