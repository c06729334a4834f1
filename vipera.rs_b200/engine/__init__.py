"""The engine: model loading, the step function, the scheduler and the public API."""
from .loader import load_model, parse_dtype, random_model, write_random_model
from .runner import ModelRunner, StepInput
from .engine import Engine, Generation, StepReport

__all__ = ["load_model", "parse_dtype", "random_model", "write_random_model", "ModelRunner", "StepInput",
           "Engine", "Generation", "StepReport"]
