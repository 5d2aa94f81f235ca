"""zlm_b200: a small model library with generation of its own for one GPU
(NVIDIA B200, sm_100a): typed configuration and registry, weights by name,
layers put together from parts, a paged cache with slots, one step function, a
generation loop, samplers, and the CUDA kernels under them."""
from . import models as _models          # fills the architecture registry
from . import parts as _parts            # fills the part registries
from .config import ConfigError, Qwen3Config
from .engine import Engine, StepEntry, StepError
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "Qwen3Config", "Engine", "StepEntry", "StepError", "WeightError",
           "write_random_model"]
