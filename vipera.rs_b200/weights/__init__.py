"""Weights: the safetensors container, sources of tensors, the schema check."""
from .loader import (
    AliasedSource,
    INIT,
    RandomSource,
    SafetensorsSource,
    Schema,
    TensorSpec,
    WeightSource,
    check_source,
    to_run_dtype,
    write_model_folder,
)
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = [
    "AliasedSource", "INIT", "RandomSource", "SafetensorsSource", "Schema", "TensorSpec", "WeightSource",
    "check_source", "to_run_dtype", "write_model_folder", "SafetensorsFile", "write_safetensors",
]
