from .base import (CacheRequest, CacheView, FeedForward, LayerIO, Mixer, Norm, ParamSpec, Part,
                   PositionEncoding, Runtime, StateRequest, StepContext, Workspace)
from . import norm, rope, attention, mlp, block, embedding   # register the built-in parts
from .model import DecoderModel

__all__ = ["CacheRequest", "CacheView", "FeedForward", "LayerIO", "Mixer", "Norm", "ParamSpec", "Part",
           "PositionEncoding", "Runtime", "StateRequest", "StepContext", "Workspace", "DecoderModel"]
