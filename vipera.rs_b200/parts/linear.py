"""A weight matrix and the product with it, used by mixers and feed-forwards.

The product is ``a[M, K] . w[N, K]^T`` with one of three endings: store (with an optional
bias), add into the 32-bit residual stream, or SwiGLU over interleaved gate and up rows.
Which kernel runs is decided here, by dtype and size: the 32-bit path always uses the
CUDA-core kernel; the bfloat16 path uses the tensor-core kernel where it takes the sizes
and the CUDA-core kernel elsewhere.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..errors import UnsupportedError
from ..kernels import ops

SWIGLU_GROUP = 16  # gate rows and up rows alternate in groups of this many
SMALL_KERNEL_MAX_ROWS = int(os.environ.get("VIPERA_GEMV_MAX_ROWS", 4096))
SMALL_KERNEL_MAX_INNER = int(os.environ.get("VIPERA_GEMV_MAX_INNER", 4096))


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


class NormedInput:
    """The normalised residual stream as an input that may not have been computed yet.

    A product that can take the norm with it (the small-token kernel) reads ``residual``,
    ``norm.weight`` and ``norm.eps`` itself; everything else calls ``tensor()``, which runs
    the norm once and keeps the result for the other products of the same part."""

    def __init__(self, ctx, norm, residual: torch.Tensor, rows: Optional[torch.Tensor] = None,
                 num_rows: Optional[int] = None, name: str = "block.h"):
        self.ctx, self.norm, self.residual, self.rows = ctx, norm, residual, rows
        self.num_rows = int(num_rows if num_rows is not None else residual.shape[0])
        self.name = name
        self._tensor = None

    @property
    def fusable(self) -> bool:
        weight = getattr(self.norm, "weight", None)
        return (getattr(self.norm, "fused_kind", None) == "rmsnorm" and weight is not None
                and weight.dtype == torch.float32)

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            out = self.ctx.workspace.get(self.name, (self.num_rows, self.residual.shape[1]), self.ctx.dtype)
            self.norm.forward(self.ctx, self.residual, out, rows=self.rows)
            self._tensor = out
        return self._tensor


class Linear:
    """``weight`` is [N, K] in the run dtype on the device; ``bias`` float32 [N] or None."""

    kernels = ("gemm_simt",)

    def __init__(self, weight: torch.Tensor, dtype: torch.dtype, device, bias: Optional[torch.Tensor] = None):
        self.weight = weight.to(device=device, dtype=dtype).contiguous()
        self.bias = None if bias is None else bias.to(device=device, dtype=torch.float32).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self._small_ok = {}
        # The tcgen05 kernel reads the matrix by TMA: bfloat16, rows a multiple of 16 bytes long
        # and a 16-byte aligned base.  Other matrices run on the CUDA cores.
        self.tensor_core = (dtype == torch.bfloat16 and self.weight.shape[1] % 8 == 0
                            and self.weight.data_ptr() % 16 == 0)

    def kernel_families(self):
        if self.tensor_core:
            return ("gemm_simt", "gemm_tc", "gemv_small")
        return ("gemm_simt",)

    def takes_small(self, tokens: int) -> bool:
        """Whether the small-token kernel runs this product for `tokens` tokens."""
        # The small-token kernel wins where a product is small (its fixed cost is low and it
        # fuses the norm in front); wide or deep products stream better through TMA.
        if (not self.tensor_core or self.out_features > SMALL_KERNEL_MAX_ROWS
                or self.in_features > SMALL_KERNEL_MAX_INNER):
            return False
        known = self._small_ok.get(tokens)
        if known is None:
            most = min(int(os.environ.get("VIPERA_GEMV_MAX_TOKENS", ops.GEMV_MAX_TOKENS)), ops.GEMV_MAX_TOKENS)
            known = self._small_ok[tokens] = (tokens <= most and
                                              ops.gemv_small_takes(tokens, self.in_features, self.out_features))
        return known

    def __call__(self, ctx, a, *, epilogue: int = ops.EPI_STORE,
                 out: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None) -> None:
        """``a`` is a tensor [tokens, K] in the run dtype, or a NormedInput."""
        bias = self.bias if epilogue == ops.EPI_STORE else None
        lazy = a if isinstance(a, NormedInput) else None
        tokens = lazy.num_rows if lazy is not None else a.shape[0]
        if self.takes_small(tokens):
            if lazy is not None and lazy.fusable and lazy._tensor is None:
                ops.gemv_small(self.weight, x=lazy.residual, norm_weight=lazy.norm.weight, eps=lazy.norm.eps,
                               rows=lazy.rows, tokens=tokens, epilogue=epilogue, bias=bias, out=out, resid=resid)
            else:
                ops.gemv_small(self.weight, a=lazy.tensor() if lazy is not None else a, epilogue=epilogue,
                               bias=bias, out=out, resid=resid)
            return
        if lazy is not None:
            a = lazy.tensor()
        if self.tensor_core and a.dtype == torch.bfloat16 and a.is_contiguous() and a.data_ptr() % 16 == 0:
            ops.gemm_tc(a, self.weight, epilogue=epilogue, bias=bias, out=out, resid=resid)
            return
        ops.gemm_simt(a, self.weight, epilogue=epilogue, bias=bias, out=out, resid=resid)
