"""A small, whole inference engine for one B200 GPU and one architecture family
(the Qwen2 / Qwen2.5 dense decoder), built from parts so that another can be added.

    from vipera_rs_b200 import Engine, SamplingParams
    engine = Engine("path/to/model", dtype="bfloat16")
    result = engine.generate([[151, 2040, 17]], SamplingParams(max_new_tokens=16))[0]
"""
from . import errors
from .config import load_config
from .engine import Engine, Generation, StepReport, load_model, random_model, write_random_model
from .sampling import SamplingParams

__all__ = ["errors", "load_config", "Engine", "Generation", "StepReport", "SamplingParams",
           "load_model", "random_model", "write_random_model"]
