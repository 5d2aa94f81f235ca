from .batch import StepEntry, StepError
from .engine import Engine, parse_dtype

__all__ = ["Engine", "StepEntry", "StepError", "parse_dtype"]
