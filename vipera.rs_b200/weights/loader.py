"""Weights by tensor name: the schema a model declares, the sources that fill it
(a safetensors folder, or a seeded random generator), and the one check that
reports every missing, unexpected and wrongly shaped tensor together.

The reference looks tensors up by name and checks rank and exact extents, with
errors of the form ``model has no tensor "…"`` and ``tensor … is [..], expected
[..]`` (crates/vipera-backend-cpu/src/model.rs:4383-4458); optional vectors are
empty when absent (:4422-4432) and the output matrix falls back to the embedding
(:425).  It has no random-weights mode; that one is this engine's own.
"""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..errors import IoError, UnsupportedError
from .safetensors_io import SafetensorsFile, write_safetensors

# How a tensor is initialised in random-weights mode: (mean, standard deviation).
INIT = {
    "linear": (0.0, 0.02),
    "embedding": (0.0, 0.02),
    "bias": (0.0, 0.02),
    "norm": (1.0, 0.01),
}


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one tensor.

    ``init`` names the random initialisation (a key of ``INIT``).  ``store`` is the
    dtype the random-weights mode stores it in when the folder is written in
    bfloat16: ``"float32"`` for tensors that stay in 32-bit, ``"model"`` for
    tensors that follow the folder's dtype, ``"int32"`` for integer tables.
    """

    shape: Tuple[int, ...]
    init: str = "linear"
    store: str = "model"


Schema = Dict[str, TensorSpec]


class WeightSource:
    """Where tensors come from.  ``get`` returns a host tensor in its stored dtype."""

    def names(self) -> List[str]:
        raise NotImplementedError

    def shape(self, name: str) -> Tuple[int, ...]:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def describe(self) -> str:
        return type(self).__name__


class SafetensorsSource(WeightSource):
    """``model.safetensors`` of a folder, or the shards its index file names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        paths: List[str]
        if os.path.exists(single):
            paths = [single]
        elif os.path.exists(index_path):
            with open(index_path, "r", encoding="utf-8") as handle:
                index = json.load(handle)
            paths = sorted({os.path.join(model_dir, f) for f in index["weight_map"].values()})
        else:
            paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
            if not paths:
                raise IoError(f"{model_dir} holds no model.safetensors")
        self._files = [SafetensorsFile(path) for path in paths]
        self._where: Dict[str, SafetensorsFile] = {}
        for handle in self._files:
            for name in handle.names():
                self._where[name] = handle

    def names(self) -> List[str]:
        return list(self._where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].shape(name)

    def stored_dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def get(self, name: str) -> torch.Tensor:
        return self._where[name].get(name)

    def describe(self) -> str:
        return self.model_dir


class AliasedSource(WeightSource):
    """A source seen under the names the parts ask for: a tensor the file stores under another
    name the architecture knows (``alias(name_in_file)`` gives the name asked for) appears under
    that name.  A name that is not an alias stays as it is, so that the check still reports it
    when nothing asks for it."""

    def __init__(self, source: WeightSource, alias):
        self._source = source
        self._stored: Dict[str, str] = {}
        for name in source.names():
            wanted = alias(name) or name
            if wanted in self._stored:
                raise UnsupportedError(f"{source.describe()} holds both {self._stored[wanted]!r} and {name!r} for {wanted!r}")
            self._stored[wanted] = name

    def names(self) -> List[str]:
        return list(self._stored)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._source.shape(self._stored[name])

    def stored_dtype(self, name: str) -> torch.dtype:
        return self._source.stored_dtype(self._stored[name])

    def get(self, name: str) -> torch.Tensor:
        return self._source.get(self._stored[name])

    def describe(self) -> str:
        return self._source.describe()


def _fnv1a64(text: str) -> int:
    value = 0xCBF29CE484222325
    for byte in text.encode("utf-8"):
        value ^= byte
        value = (value * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return value


class RandomSource(WeightSource):
    """Seeded random tensors for a schema.  A tensor's values depend on the seed and
    on its name only, not on the order in which tensors are asked for."""

    def __init__(self, schema: Schema, seed: int, dtype: torch.dtype = torch.bfloat16,
                 device: str = "cpu"):
        self._schema = schema
        self._seed = int(seed)
        self._dtype = dtype
        self._device = device

    def names(self) -> List[str]:
        return list(self._schema)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._schema[name].shape

    def get(self, name: str) -> torch.Tensor:
        spec = self._schema[name]
        generator = torch.Generator(device=self._device)
        generator.manual_seed((self._seed * 0x9E3779B97F4A7C15 ^ _fnv1a64(name)) & 0x7FFFFFFFFFFFFFFF)
        if spec.store == "int32":
            return torch.randint(0, 2**31 - 1, spec.shape, generator=generator,
                                 device=self._device, dtype=torch.int32)
        mean, std = INIT[spec.init]
        values = torch.randn(spec.shape, generator=generator, device=self._device,
                             dtype=torch.float32)
        values.mul_(std).add_(mean)
        return values.to(torch.float32 if spec.store == "float32" else self._dtype)

    def describe(self) -> str:
        return f"random weights (seed {self._seed})"


def check_source(schema: Schema, source: WeightSource) -> None:
    """One error that lists every missing tensor, every unexpected tensor and every
    wrong shape, or nothing."""
    have = set(source.names())
    want = set(schema)
    missing = sorted(want - have)
    unexpected = sorted(have - want)
    wrong = []
    for name in sorted(want & have):
        got = tuple(source.shape(name))
        if got != tuple(schema[name].shape):
            wrong.append(f"{name}: is {list(got)}, expected {list(schema[name].shape)}")
    if not (missing or unexpected or wrong):
        return
    lines = [f"weights in {source.describe()} do not match the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(wrong))
    error = UnsupportedError("\n".join(lines))
    error.missing, error.unexpected, error.wrong_shape = missing, unexpected, wrong
    raise error


def to_run_dtype(tensor: torch.Tensor, run_dtype: torch.dtype) -> torch.Tensor:
    """The dtype a stored tensor is kept in while the model runs.

    Float tensors follow the run dtype, except that a tensor stored in 32-bit stays
    in 32-bit; integer tables become int32.  In a float32 run everything is float32.
    """
    if tensor.dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return tensor.to(torch.int32)
    if run_dtype == torch.float32 or tensor.dtype in (torch.float32, torch.float64):
        return tensor.to(torch.float32)
    return tensor.to(run_dtype)


def write_model_folder(model_dir: str, config_dict: dict, schema: Schema, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Random-weights mode: write ``config.json`` and ``model.safetensors``."""
    os.makedirs(model_dir, exist_ok=True)
    source = RandomSource(schema, seed, dtype)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config_dict, handle, indent=2)
        handle.write("\n")
    write_safetensors(
        os.path.join(model_dir, "model.safetensors"),
        ((name, source.get(name)) for name in schema),
        metadata={"format": "pt", "seed": seed},
    )
