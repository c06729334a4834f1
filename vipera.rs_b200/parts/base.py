"""What every part looks like to the builder and to the step function.

A part is built from ``params`` (its sizes and constants), a ``prefix`` (where its tensors
live in the weight file) and the tensors themselves.  It never learns which model it is in.

Interfaces
----------
Norm            ``forward(ctx, x, out, rows=None)``: x is the float32 residual stream
                [tokens, hidden]; ``out`` receives the normalised rows in the activation dtype.
PositionEncoding  ``style`` and ``tables(device)`` for encodings the fused kernel knows
                (rotary pairs), or ``apply(ctx, q, k)`` for anything else.
Mixer           ``cache_request()`` says what the mixer keeps between steps (paged keys and
                values, a fixed-size state, or nothing); ``forward(ctx, h, residual, cache,
                writes_cache)`` adds the mixer's output into ``residual`` in place.
FeedForward     ``forward(ctx, h, residual)`` adds its output into ``residual`` in place.
Block           ``forward(ctx, residual, cache, writes_cache)`` arranges the four.

The reference's seam between runtime and backend is the same in spirit: the backend turns
(tokens, positions, block table, cache buffer) into logits and writes keys and values into
the runtime's buffer (crates/vipera-runtime/src/pipeline.rs:107-130, 187-230), and "what it
stores inside that slot is its own business" (pipeline.rs:107-113).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..weights import Schema


@dataclass(frozen=True)
class PagedKV:
    """The mixer keeps keys and values of every position (or of a window of them) in pages."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: all keys; w: a query at p reads p-w+1 .. p


@dataclass(frozen=True)
class FixedState:
    """The mixer keeps one tensor of fixed shape per request, whatever its length."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class PagedKVView:
    """The pages of one cache slot: ``k`` and ``v`` are [pages, page_size, kv_heads, d]."""

    def __init__(self, group: int, k: torch.Tensor, v: torch.Tensor, page_size: int, window: Optional[int]):
        self.group = group
        self.k = k
        self.v = v
        self.page_size = page_size
        self.window = window


class StateView:
    """The state of one cache slot: ``data`` is [state_slots, *shape]; a request's row is
    ``ctx.state_slots[entry]``, and ``ctx.fresh[entry]`` says that it must start anew."""

    def __init__(self, data: torch.Tensor):
        self.data = data


class Workspace:
    """Named device buffers that live across steps, so that a step allocates nothing once
    its sizes have been seen (and a captured CUDA graph keeps valid addresses)."""

    def __init__(self, device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}  # (name, dtype, shape) -> the view handed out last time
        self.frozen = False
        self.generation = 0  # goes up whenever a buffer moves; captured graphs are then stale

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(shape)
        view = self._views.get((name, dtype, shape))
        if view is not None:
            return view
        count = 1
        for extent in shape:
            count *= int(extent)
        key = (name, dtype)
        buffer = self._buffers.get(key)
        if buffer is None or buffer.numel() < count:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would grow while frozen")
            buffer = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buffer
            self.generation += 1
            # views of the buffer that was replaced are no longer handed out
            self._views = {k: v for k, v in self._views.items() if (k[0], k[1]) != key}
        view = buffer[:count].view(*shape)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[(name, dtype, shape)] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class StepContext:
    """Everything a part may read about the step it runs in.  Device tensors are int32."""

    num_tokens: int
    num_entries: int
    tokens: torch.Tensor        # [tokens]
    positions: torch.Tensor     # [tokens]
    token_entry: torch.Tensor   # [tokens] index of the token's entry (row of the block tables)
    entry_starts: torch.Tensor  # [entries + 1] cumulative token counts
    entry_pos0: torch.Tensor    # [entries] position of the entry's first token
    state_slots: torch.Tensor   # [entries]
    fresh: torch.Tensor         # [entries] 1 where per-request state must start anew
    block_tables: List[torch.Tensor]  # per group: [entries, width], -1 where no page is held
    logit_rows: Optional[torch.Tensor]  # [rows] token indices whose logits are wanted
    num_logit_rows: int
    # host copies for launch decisions
    host_counts: List[int]
    host_pos0: List[int]
    max_count: int
    max_kv_len: int
    all_single: bool            # every entry brings exactly one token
    any_single: bool            # some entry brings exactly one token (beside entries that bring more)
    dtype: torch.dtype          # activation dtype of the run
    workspace: Workspace
    logits_all_rows: bool = False  # the wanted rows are all the step's tokens, in order
    extras: Dict[str, Any] = field(default_factory=dict)


class Part:
    """Base of all parts."""

    kernels: Tuple[str, ...] = ()  # kernel families this part launches
    graph_safe: bool = True         # False: forward() talks to the host, so it cannot be captured in a CUDA graph

    @classmethod
    def schema(cls, params: Dict[str, Any], prefix: str) -> Schema:
        """The tensors this part reads, by full name."""
        return {}

    def __init__(self, params: Dict[str, Any], prefix: str, tensors: Dict[str, torch.Tensor],
                 dtype: torch.dtype, device):
        self.params = params
        self.prefix = prefix
        self.dtype = dtype
        self.device = device

    def kernel_families(self) -> Tuple[str, ...]:
        return self.kernels

    @classmethod
    def workspace_bytes(cls, params: Dict[str, Any], tokens: int, element_bytes: int) -> int:
        """Device bytes of the buffers this part asks the workspace for in a step of `tokens`
        tokens (for the memory plan; parts of one kind share their buffers between layers)."""
        return 0


class Norm(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    style: Optional[int] = None  # a rotary style of the fused kernel, or None

    def tables(self):
        """(cos, sin) float32 [positions, d/2] for the fused styles."""
        raise NotImplementedError

    def apply(self, ctx: StepContext, q: torch.Tensor, k: torch.Tensor) -> None:
        """Encode positions into float32 q [tokens, heads, d] and k [tokens, kv_heads, d] in place."""
        raise NotImplementedError


class Mixer(Part):
    @classmethod
    def cache_request_for(cls, params: Dict[str, Any]):
        """What a mixer with these sizes keeps between steps: PagedKV, FixedState or None.  A
        class method, so that memory can be planned from a description alone, without weights."""
        return None

    def cache_request(self):
        return type(self).cache_request_for(self.params)

    def forward(self, ctx: StepContext, h: torch.Tensor, residual: torch.Tensor, cache, writes_cache: bool) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: StepContext, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError
