"""From a model folder (or a configuration and a seed) to a built model on the GPU."""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import parts  # noqa: F401  (registers the built-in part kinds)
from ..build import build_kernels
from ..config import architecture_of, load_config, read_config_json
from ..errors import InvalidArgumentError
from ..parts.model import DecoderModel, model_schema
from ..weights import AliasedSource, RandomSource, SafetensorsSource, write_model_folder


def _kernel_families(model) -> list:
    """The kernel families the model's parts name."""
    return list(model.kernel_families())


_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise InvalidArgumentError(f"dtype must be bfloat16 or float32, got {name!r}") from None


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """Build the model that ``model_dir/config.json`` names from ``model_dir/model.safetensors``
    and compile the kernels it needs."""
    arch, config = load_config(model_dir)
    spec = arch.model_spec(config)
    source = SafetensorsSource(model_dir)
    if arch.tensor_alias is not None:
        source = AliasedSource(source, arch.tensor_alias)
    model = DecoderModel(spec, source, parse_dtype(dtype), device)
    model.config = config
    build_kernels(_kernel_families(model))
    return model


def random_model(config_dict: dict, seed: int, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """Build a model with seeded random weights made on the device, without a folder.
    (The values differ from those ``write_random_model`` stores for the same seed: the
    device's generator is not the host's.)"""
    arch = architecture_of(config_dict)
    config = arch.config_from_dict(config_dict)
    spec = arch.model_spec(config)
    run_dtype = parse_dtype(dtype)
    source = RandomSource(model_schema(spec), seed, run_dtype, device=str(device))
    model = DecoderModel(spec, source, run_dtype, device)
    model.config = config
    build_kernels(_kernel_families(model))
    return model


def write_random_model(model_dir: str, config_dict: dict, seed: int, dtype="bfloat16") -> None:
    """Random-weights mode: write ``config.json`` and ``model.safetensors`` for a configuration
    and a seed.  Linear and embedding weights ~ N(0, 0.02), biases ~ N(0, 0.02), norm weights
    1 + N(0, 0.01); norm weights are stored in 32-bit, the rest in ``dtype``."""
    arch = architecture_of(config_dict)
    config = arch.config_from_dict(config_dict)
    spec = arch.model_spec(config)
    out = config.to_dict() if hasattr(config, "to_dict") else dict(config_dict)
    write_model_folder(model_dir, out, model_schema(spec), seed, parse_dtype(dtype))
