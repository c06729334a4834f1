"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` with 32-bit statistics
(crates/vipera-backend-cpu/src/model.rs:4282-4288)."""
from __future__ import annotations

import torch

from ..config.registry import NORMS
from ..kernels import ops
from ..weights import TensorSpec
from .base import Norm


class RMSNorm(Norm):
    """params: ``size`` (width of a row), ``eps``.  Tensor: ``<prefix>.weight`` [size]."""

    kernels = ("rowwise",)
    fused_kind = "rmsnorm"  # products that can compute a norm on the way recognise it by this

    @classmethod
    def schema(cls, params, prefix):
        return {f"{prefix}.weight": TensorSpec((params["size"],), init="norm", store="float32")}

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        # The weight is used in 32-bit whatever it was stored in (bfloat16 widens exactly).
        self.weight = tensors[f"{prefix}.weight"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, ctx, x, out, rows=None):
        ops.rmsnorm(x, self.weight, out, self.eps, rows)


NORMS.register("rmsnorm", RMSNorm)
