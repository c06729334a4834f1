"""A small, whole inference engine for one B200 GPU and one architecture family
(the Qwen2 / Qwen2.5 dense decoder), built from parts so that another can be added."""
from . import errors
from .config import load_config

__all__ = ["errors", "load_config"]
