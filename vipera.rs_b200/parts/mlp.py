"""SwiGLU feed-forward: ``down(up(h) * silu(gate(h)))``, no biases
(crates/vipera-backend-cpu/src/model.rs:1154-1198, 4368-4374).

The reference runs gate and up as two products and the activation as its own pass
(model.rs:1159-1183).  Here the two matrices are interleaved at load so that one product
yields both halves of every feature in one tile, the activation is that product's ending,
and the down product adds into the 32-bit residual stream.
"""
from __future__ import annotations

import torch

from ..config.registry import FEED_FORWARDS
from ..kernels import ops
from ..weights import TensorSpec
from .base import FeedForward
from .linear import Linear, interleave_gate_up


class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size and, optionally, ``projection_names``
    (defaults gate_proj, up_proj, down_proj)."""

    takes_lazy_input = True

    @staticmethod
    def _names(params):
        return params.get("projection_names", ("gate_proj", "up_proj", "down_proj"))

    @classmethod
    def schema(cls, params, prefix):
        hidden, inter = params["hidden_size"], params["intermediate_size"]
        gate, up, down = cls._names(params)
        return {
            f"{prefix}.{gate}.weight": TensorSpec((inter, hidden)),
            f"{prefix}.{up}.weight": TensorSpec((inter, hidden)),
            f"{prefix}.{down}.weight": TensorSpec((hidden, inter)),
        }

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        return tokens * params["intermediate_size"] * element_bytes

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        gate, up, down = self._names(params)
        fused = interleave_gate_up(tensors[f"{prefix}.{gate}.weight"], tensors[f"{prefix}.{up}.weight"])
        self.gate_up = Linear(fused, dtype, device)
        self.down = Linear(tensors[f"{prefix}.{down}.weight"], dtype, device)

    def kernel_families(self):
        return tuple(dict.fromkeys(self.gate_up.kernel_families() + self.down.kernel_families()))

    def forward(self, ctx, h, residual):
        act = ctx.workspace.get("swiglu.act", (ctx.num_tokens, self.inter), ctx.dtype)
        self.gate_up(ctx, h, epilogue=ops.EPI_SWIGLU, out=act)
        self.down(ctx, act, epilogue=ops.EPI_RESIDUAL, resid=residual)


FEED_FORWARDS.register("swiglu", SwiGLU)
