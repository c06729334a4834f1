"""Choice of the tensor-core product kernel for a bfloat16 weight matrix."""
from __future__ import annotations

import torch

from ..kernels import ops


class TensorCorePlan:
    """Runs products with one [N, K] bfloat16 matrix through the tcgen05 kernel."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight

    def takes(self, a: torch.Tensor, epilogue: int, out) -> bool:
        return a.dtype == torch.bfloat16 and a.is_contiguous() and a.data_ptr() % 16 == 0

    def run(self, ctx, a, *, epilogue, bias, out, resid) -> None:
        ops.gemm_tc(a, self.weight, epilogue=epilogue, bias=bias, out=out, resid=resid)


def plan_for(weight: torch.Tensor):
    """A plan that runs products with ``weight`` on the tensor cores, or None where the
    tensor-core kernel does not take the matrix: TMA needs rows that are a multiple of 16
    bytes long and a 16-byte aligned base."""
    if weight.dtype != torch.bfloat16 or weight.shape[1] % 8 or weight.data_ptr() % 16:
        return None
    return TensorCorePlan(weight)
