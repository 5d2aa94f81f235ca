"""Architectures this build knows.  Importing the package fills the registry."""
from . import qwen3   # noqa: F401
