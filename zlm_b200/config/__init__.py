from .spec import (ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "Qwen3Config"]
