"""A weight matrix and the product with it, used by mixers and feed-forwards.

The product is ``a[M, K] . w[N, K]^T`` with one of three endings: store (with an optional
bias), add into the 32-bit residual stream, or SwiGLU over interleaved gate and up rows.
Which kernel runs is decided here, by dtype and size: the 32-bit path always uses the
CUDA-core kernel; the bfloat16 path uses the tensor-core kernel where it takes the sizes
and the CUDA-core kernel elsewhere.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..errors import UnsupportedError
from ..kernels import ops

SWIGLU_GROUP = 16  # gate rows and up rows alternate in groups of this many


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, H] gate and up matrices as one [2I, H] matrix: 16 gate rows, then the 16 up rows
    of the same features, and so on, so that one tile of the product holds both halves of
    every feature it covers."""
    inter, hidden = gate.shape
    if up.shape != gate.shape:
        raise UnsupportedError("gate and up matrices differ in shape")
    if inter % SWIGLU_GROUP:
        raise UnsupportedError(
            f"intermediate size {inter} is not a multiple of {SWIGLU_GROUP}; the SwiGLU kernels refuse it")
    groups = inter // SWIGLU_GROUP
    stacked = torch.stack(
        [gate.view(groups, SWIGLU_GROUP, hidden), up.view(groups, SWIGLU_GROUP, hidden)], dim=1)
    return stacked.reshape(2 * inter, hidden).contiguous()


class Linear:
    """``weight`` is [N, K] in the run dtype on the device; ``bias`` float32 [N] or None."""

    kernels = ("gemm_simt",)

    def __init__(self, weight: torch.Tensor, dtype: torch.dtype, device, bias: Optional[torch.Tensor] = None):
        self.weight = weight.to(device=device, dtype=dtype).contiguous()
        self.bias = None if bias is None else bias.to(device=device, dtype=torch.float32).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self._tensor_core = None
        if dtype == torch.bfloat16:
            from . import tensor_core

            self._tensor_core = tensor_core.plan_for(self.weight)

    def kernel_families(self):
        if self._tensor_core is not None:
            return ("gemm_simt", "gemm_tc")
        return ("gemm_simt",)

    def __call__(self, ctx, a: torch.Tensor, *, epilogue: int = ops.EPI_STORE,
                 out: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None) -> None:
        bias = self.bias if epilogue == ops.EPI_STORE else None
        if self._tensor_core is not None and self._tensor_core.takes(a, epilogue, out):
            self._tensor_core.run(ctx, a, epilogue=epilogue, bias=bias, out=out, resid=resid)
            return
        ops.gemm_simt(a, self.weight, epilogue=epilogue, bias=bias, out=out, resid=resid)
