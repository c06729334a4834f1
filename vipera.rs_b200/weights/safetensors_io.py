"""Reading and writing the safetensors container: an 8-byte little-endian header
length, a JSON header ``{name: {dtype, shape, data_offsets}}``, then the raw bytes.

The reference's model file reader is a bounded little-endian reader over a
memory-mapped file with a tensor table of ``{name, dims, type, offset}``
(crates/vipera-core/src/gguf/mod.rs:90-99, reader.rs); this is the same idea
for the container the Qwen2 checkpoints come in.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

from ..errors import IoError, ParseError, UnsupportedError

_DTYPES = {
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F32": torch.float32,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {value: key for key, value in _DTYPES.items()}


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are views until copied."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._handle = open(path, "rb")
            size = os.fstat(self._handle.fileno()).st_size
        except OSError as error:
            raise IoError(f"cannot read {path}: {error}") from None
        if size < 8:
            raise ParseError(f"{path} is too short for a safetensors header", 0)
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len > size - 8:
            raise ParseError(f"{path}: header length {header_len} exceeds the file", 0)
        try:
            header = json.loads(self._map[8 : 8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise ParseError(f"{path}: header is not valid JSON ({error})", 8) from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + header_len
        self._table: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, entry in header.items():
            try:
                dtype = _DTYPES[entry["dtype"]]
            except KeyError:
                raise UnsupportedError(
                    f"{path}: tensor {name!r} has dtype {entry.get('dtype')!r}, which is not supported"
                ) from None
            shape = tuple(int(x) for x in entry["shape"])
            begin, end = (int(x) for x in entry["data_offsets"])
            count = 1
            for extent in shape:
                count *= extent
            if end - begin != count * _element_size(dtype) or self._base + end > size or begin < 0:
                raise ParseError(
                    f"{path}: tensor {name!r} claims bytes [{begin}, {end}) that do not match "
                    f"its shape {list(shape)} or lie outside the file",
                    self._base + begin,
                )
            self._table[name] = (dtype, shape, begin, end)

    def names(self) -> List[str]:
        return list(self._table)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._table[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._table[name][0]

    def __contains__(self, name: str) -> bool:
        return name in self._table

    def get(self, name: str) -> torch.Tensor:
        """A copy of the tensor in host memory, in the dtype it is stored in."""
        dtype, shape, begin, end = self._table[name]
        count = 1
        for extent in shape:
            count *= extent
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=end - begin, offset=self._base + begin).copy()
        return torch.from_numpy(raw).view(dtype).reshape(shape)

    def close(self) -> None:
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass  # a view is still alive; the map goes with it
        self._handle.close()


def _element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None) -> None:
    """Write named tensors in the order given; ``tensors`` may be a generator."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    staged: List[torch.Tensor] = []
    for name, tensor in tensors:
        tensor = tensor.detach().contiguous().cpu()
        if tensor.dtype not in _NAMES:
            raise UnsupportedError(f"cannot store dtype {tensor.dtype} of {name!r}")
        size = tensor.numel() * tensor.element_size()
        header[name] = {
            "dtype": _NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + size],
        }
        offset += size
        staged.append(tensor)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    try:
        with open(path, "wb") as handle:
            handle.write(struct.pack("<Q", len(blob)))
            handle.write(blob)
            for tensor in staged:
                if tensor.numel():
                    handle.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())
    except OSError as error:
        raise IoError(f"cannot write {path}: {error}") from None
