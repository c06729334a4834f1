"""Device memory of the cache and its grouping.

Layers whose mixers ask for the same kind of paged memory (KV head count, head size,
window) form a group.  A group has pages of its own: one page number addresses the same
page in every layer of the group, as one block addresses every layer in the reference
(crates/vipera-backend-cpu/src/model.rs:63-70, crates/vipera-runtime/src/pipeline.rs:128-129).
Inside a group the memory is [slot in group][k or v][page][position in page][kv head][d],
the reference's layer-major order lifted to the pool (model.rs:1451-1469), so that each
layer's keys are one dense [pages * page_size, kv_heads * d] matrix.

Mixers that keep a fixed-size state get one tensor [state slots, *shape] per cache slot.
The bookkeeping (which request holds which page and which state slot) is the native
``CacheManager``; this module owns only the memory.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..build import runtime_module
from ..errors import InvalidArgumentError
from ..parts.base import FixedState, PagedKV, PagedKVView, StateView


GUARD_WORD = 0x5A5A   # fits 16 bits: the guard regions are viewed as integers of the element's width


@dataclass
class CacheGroup:
    num_kv_heads: int
    head_dim: int
    window: Optional[int]
    slots: List[int] = field(default_factory=list)  # cache slots (of the schedule) in this group

    def bytes_per_token(self, element_bytes: int) -> int:
        return 2 * len(self.slots) * self.num_kv_heads * self.head_dim * element_bytes


def plan_groups(cache_requests: Dict[int, object]) -> Tuple[List[CacheGroup], Dict[int, FixedState]]:
    """Sort the cache slots of a model into paged groups and fixed-state slots."""
    groups: Dict[Tuple[int, int, Optional[int]], CacheGroup] = {}
    states: Dict[int, FixedState] = {}
    for slot in sorted(cache_requests):
        request = cache_requests[slot]
        if request is None:
            continue
        if isinstance(request, PagedKV):
            key = (request.num_kv_heads, request.head_dim, request.window)
            if key not in groups:
                groups[key] = CacheGroup(*key)
            groups[key].slots.append(slot)
        elif isinstance(request, FixedState):
            states[slot] = request
        else:
            raise InvalidArgumentError(f"cache slot {slot}: unknown kind of cache request {request!r}")
    return list(groups.values()), states


class CachePools:
    """Allocates the pools and the native manager for one engine."""

    def __init__(self, cache_requests: Dict[int, object], *, page_size: int, num_pages, num_state_slots: int,
                 dtype: torch.dtype, device, reuse_prefixes: bool = False):
        self.groups, self.states = plan_groups(cache_requests)
        self.page_size = int(page_size)
        self.dtype = dtype
        self.device = device
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        if len(num_pages) != len(self.groups):
            raise InvalidArgumentError("one page count is needed for each group of layers")
        self.num_pages = [int(n) for n in num_pages]
        runtime = runtime_module()
        self.manager = runtime.CacheManager(
            [(self.page_size, pages, group.window or 0) for group, pages in zip(self.groups, self.num_pages)],
            int(num_state_slots),
            # pages of a prompt prefix can be shared only where the pages are all a request keeps:
            # a mixer with a state of its own would have to store that state at every page's end
            bool(reuse_prefixes) and not self.states)
        self.pool_tensors: List[torch.Tensor] = []
        self.views: Dict[int, object] = {}
        # One page beyond those the manager hands out, per group: the scratch page.  No request
        # ever holds it; tokens that pad a captured step to its size class write there.
        self.scratch_pages: List[int] = list(self.num_pages)
        # Each pool lies between two guard regions of one page each, filled with a fixed word that
        # no kernel ever writes: `guards_intact()` (the tests call it after they ran) shows a write
        # that went past either end of a pool.
        self._guards: List[torch.Tensor] = []
        for index, (group, pages) in enumerate(zip(self.groups, self.num_pages)):
            shape = (len(group.slots), 2, pages + 1, self.page_size, group.num_kv_heads, group.head_dim)
            count = 1
            for extent in shape:
                count *= extent
            guard = self.page_size * group.num_kv_heads * group.head_dim
            storage = torch.zeros(count + 2 * guard, dtype=dtype, device=device)
            storage[:guard].view(torch.int16 if storage.element_size() == 2 else torch.int32).fill_(GUARD_WORD)
            storage[guard + count:].view(torch.int16 if storage.element_size() == 2 else torch.int32).fill_(GUARD_WORD)
            self._guards.extend([storage[:guard], storage[guard + count:]])
            pool = storage[guard:guard + count].view(shape)
            self.pool_tensors.append(pool)
            for position, slot in enumerate(group.slots):
                self.views[slot] = PagedKVView(index, pool[position, 0], pool[position, 1], self.page_size,
                                               group.window)
        for slot, request in self.states.items():
            data = torch.zeros((int(num_state_slots), *request.shape), dtype=request.dtype, device=device)
            self.views[slot] = StateView(data)

    def guards_intact(self) -> bool:
        """Whether the guard regions in front of and behind every pool still hold their word."""
        for guard in self._guards:
            words = guard.view(torch.int16 if guard.element_size() == 2 else torch.int32)
            if not bool((words == GUARD_WORD).all()):
                return False
        return True

    def audit(self) -> str:
        """"" when the manager's books are sound (no page lost, held twice or freed twice) and
        the guard regions are intact; else what is wrong."""
        problem = self.manager.audit()
        if not problem and not self.guards_intact():
            problem = "a guard region beside a cache pool was written"
        return problem

    def bytes(self) -> int:
        total = sum(p.numel() * p.element_size() for p in self.pool_tensors)
        for view in self.views.values():
            if isinstance(view, StateView):
                total += view.data.numel() * view.data.element_size()
        return total

    def poison(self, value: float = float("nan")) -> None:
        """Fill every page with a value that shows when read (tests use NaN)."""
        for pool in self.pool_tensors:
            pool.fill_(value)
