"""Rotary position encoding, NeoX pairing ``(i, i + d/2)``.

Angles as the reference computes them, in 32-bit: ``inv_i = 1 / base^(2i/d)``,
``angle = position * inv_i`` (crates/vipera-backend-cpu/src/model.rs:4204-4206).  The
reference builds the table once per position and step and shares it between layers
(model.rs:970-973); here one table is built on the host for the positions the engine can
reach (``prepare``; the model's own limit where nobody says) and shared by every layer with
the same head size and base.  Tables live as long as a part holds them.
"""
from __future__ import annotations

import weakref

import torch

from ..config.registry import POSITION_ENCODINGS
from ..kernels import ops
from .base import PositionEncoding

class _Tables:
    """(cos, sin) held by the parts that use them; the shared table forgets them with the last part."""

    def __init__(self, cos, sin):
        self.pair = (cos, sin)


_TABLES = weakref.WeakValueDictionary()


def rotary_tables(head_dim: int, theta: float, max_positions: int, device) -> _Tables:
    """cos and sin, each float32 [max_positions, head_dim / 2], on ``device``."""
    key = (head_dim, float(theta), max_positions, str(device))
    cached = _TABLES.get(key)
    if cached is not None:
        return cached
    half = head_dim // 2
    index = torch.arange(half, dtype=torch.float32)
    exponent = 2.0 * index / torch.tensor(float(head_dim), dtype=torch.float32)
    inverse = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    position = torch.arange(max_positions, dtype=torch.float32)
    angle = position[:, None] * inverse[None, :]
    tables = _Tables(torch.cos(angle).contiguous().to(device), torch.sin(angle).contiguous().to(device))
    _TABLES[key] = tables
    return tables


class RopeNeox(PositionEncoding):
    """params: ``head_dim``, ``theta``, ``max_positions``.  No tensors."""

    style = ops.ROPE_NEOX
    kernels = ("rope_cache",)

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        self.reach = None   # positions the tables cover; the model's own limit where nobody says
        self._tables = None

    def prepare(self, max_positions: int) -> None:
        """An engine reaches positions below `max_positions` only: the tables are sized for the
        furthest any engine on this model has asked for, and never shrink."""
        reach = min(self.max_positions, int(max_positions))
        if self.reach is not None and reach <= self.reach:
            return
        self.reach = reach
        if self._tables is not None:
            # Tables in use move: graphs that captured their addresses are stale.
            self._tables = None
            ops.buffer_generation += 1

    def tables(self):
        if self._tables is None:
            if self.reach is None:
                self.reach = self.max_positions
            self._tables = rotary_tables(self.head_dim, self.theta, self.reach, self.device)
        return self._tables.pair


class RopeInterleaved(RopeNeox):
    """The same angles with the other pairing: values ``(2i, 2i + 1)`` turn together.  No fused
    ending knows it; the rotation kernel behind the q/k/v product does (so it runs unfused)."""

    style = ops.ROPE_INTERLEAVED


class NoPositions(PositionEncoding):
    """Leaves q and k as they are."""

    style = ops.ROPE_NONE

    def tables(self):
        return (None, None)


POSITION_ENCODINGS.register("rope_neox", RopeNeox)
POSITION_ENCODINGS.register("rope_interleaved", RopeInterleaved)
POSITION_ENCODINGS.register("none", NoPositions)
