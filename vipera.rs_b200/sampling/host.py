"""The host sampler (native code): the reference's semantics on a row of float32 logits.
It is what the device sampler is held to in the tests, and what draws the one case the
device kernel leaves out (no top-k cut and a top-p head longer than 4096 candidates)."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from ..build import runtime_module


def Rng(seed: int = 0):
    """xorshift64* seeded through SplitMix64 (crates/vipera-sampler/src/rng.rs:13-57)."""
    return runtime_module().Rng(int(seed))


def _config(params) -> dict:
    if hasattr(params, "to_native"):
        return params.to_native()
    return dict(params)


def draw_greedy(logits, params=None, recent: Sequence[int] = ()) -> int:
    return int(runtime_module().draw_greedy(np.asarray(logits, dtype=np.float32),
                                            _config(params or {}), list(recent)))


def draw_temperature(logits, params, recent: Sequence[int], uniform: float) -> int:
    return int(runtime_module().draw_temperature(np.asarray(logits, dtype=np.float32), _config(params),
                                                 list(recent), float(uniform)))


class HostSampler:
    """Options and generator of one request (crates/vipera-sampler/src/lib.rs:269-417)."""

    def __init__(self, params):
        self._native = runtime_module().Sampler(_config(params))

    def sample(self, logits, recent: Sequence[int] = ()) -> int:
        return int(self._native.sample(np.asarray(logits, dtype=np.float32), list(recent)))
