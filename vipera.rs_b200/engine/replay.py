"""Replay of given tokens through the engine's own step function (no sampling).

Used by ``bin/trace_run``.  It owns nothing but the mapping from a trace's request names
to the cache manager's request numbers: pages come from the engine's cache manager, the
step from the engine's runner, the model and kernels are the ones generation uses.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import numpy as np
import torch

from ..cache import CachePools
from ..errors import InvalidArgumentError
from ..kernels import ops
from .loader import load_model
from .runner import ModelRunner, StepInput


class Replayer:
    def __init__(self, model_dir: str, dtype: str, *, max_tokens: int, page_size: int = 64,
                 device: str = "cuda:0", max_live: int = 8):
        self.model = load_model(model_dir, dtype, device)
        pages = max(1, (int(max_tokens) + page_size - 1) // page_size)
        self.pools = CachePools(self.model.cache_requests, page_size=page_size, num_pages=pages,
                                num_state_slots=max_live, dtype=self.model.dtype, device=self.model.device)
        if os.environ.get("VIPERA_POISON_CACHE") == "1":
            # Unwritten cache memory reads as NaN, so a key that was never stored shows.
            self.pools.poison()
        self.runner = ModelRunner(self.model, self.pools,
                                  max_model_len=self.model.spec.max_position_embeddings)
        self._ids: Dict[str, int] = {}
        self._next = 0

    def step(self, entries: List[dict], end: List[str]) -> Optional[np.ndarray]:
        manager = self.pools.manager
        requests, counts, pos0, fresh, tokens, rows = [], [], [], [], [], []
        offset = 0
        for entry in entries:
            name = str(entry["id"])
            ids = [int(t) for t in entry["tokens"]]
            if not ids:
                raise InvalidArgumentError(f"request {name!r} brings no tokens in this step")
            if name not in self._ids:
                self._ids[name] = self._next
                self._next += 1
                manager.open(self._ids[name])
            number = self._ids[name]
            done = manager.computed(number)
            manager.reserve(number, done + len(ids))
            requests.append(number)
            counts.append(len(ids))
            pos0.append(done)
            fresh.append(1 if done == 0 else 0)
            tokens.extend(ids)
            for place in entry.get("want", []):
                if not 0 <= int(place) < len(ids):
                    raise InvalidArgumentError(f"request {name!r}: wanted place {place} is outside its tokens")
                rows.append(offset + int(place))
            offset += len(ids)
        result = None
        if requests:
            step = StepInput(requests=requests, tokens=np.asarray(tokens, dtype=np.int32), counts=counts,
                             pos0=pos0, fresh=fresh, logit_rows=np.asarray(rows, dtype=np.int32))
            logits = self.runner.run(step)
            if logits is not None:
                result = logits.cpu().numpy()
            else:
                torch.cuda.synchronize(self.model.device)
            ops.check_kernel_status(self.model.device)
            for number, count, first in zip(requests, counts, pos0):
                manager.commit(number, first + count)
        for name in end:
            number = self._ids.pop(str(name), None)
            if number is not None:
                manager.close(number)
        return result
