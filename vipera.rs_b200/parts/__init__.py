"""Parts a decoder is put together from.  Importing this package registers the built-in
kinds: ``rmsnorm``; ``rope_neox``, ``rope_interleaved`` and ``none``; ``gqa_attention``; ``swiglu``; ``prenorm``."""
from . import attention, block, mlp, norm, rotary  # noqa: F401  (registration)
from .base import (
    FeedForward,
    FixedState,
    Mixer,
    Norm,
    PagedKV,
    PagedKVView,
    Part,
    PositionEncoding,
    StateView,
    StepContext,
    Workspace,
)
from .block import Block
from .linear import Linear, NormedInput, interleave_gate_up
from .model import DecoderModel, model_schema

__all__ = [
    "FeedForward", "FixedState", "Mixer", "Norm", "PagedKV", "PagedKVView", "Part", "PositionEncoding",
    "StateView", "StepContext", "Workspace", "Block", "Linear", "NormedInput", "interleave_gate_up", "DecoderModel", "model_schema",
]
