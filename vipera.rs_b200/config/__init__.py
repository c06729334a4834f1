"""Configuration: typed per-architecture configs, the registries, the model description."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Tuple

from ..errors import IoError, ParseError, UnsupportedError
from .registry import (
    ARCHITECTURES,
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    Architecture,
    Registry,
    register_architecture,
)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .qwen2 import Qwen2Config, qwen2_model_spec


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            text = handle.read()
    except OSError as error:
        raise IoError(f"cannot read {path}: {error}") from None
    try:
        data = json.loads(text)
    except json.JSONDecodeError as error:
        raise ParseError(f"{path} is not valid JSON: {error.msg}", error.pos) from None
    if not isinstance(data, dict):
        raise ParseError(f"{path} must hold a JSON object")
    return data


def architecture_of(data: Dict[str, Any]) -> Architecture:
    """The registered architecture config.json names in ``architectures[0]``."""
    names = data.get("architectures")
    if not names or not isinstance(names, list):
        raise UnsupportedError(
            "config.json has no 'architectures' list; registered: "
            + ", ".join(ARCHITECTURES.names())
        )
    return ARCHITECTURES.find(str(names[0]))


def load_config(model_dir: str) -> Tuple[Architecture, Any]:
    """Read ``model_dir/config.json`` into its architecture's typed configuration."""
    data = read_config_json(model_dir)
    arch = architecture_of(data)
    return arch, arch.config_from_dict(data)


__all__ = [
    "ARCHITECTURES", "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "Architecture", "Registry", "register_architecture",
    "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry",
    "Qwen2Config", "qwen2_model_spec",
    "read_config_json", "architecture_of", "load_config",
]
