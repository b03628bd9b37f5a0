"""y = x . W^T with a fused epilogue.

W is stored (outputs x inputs) row-major, as in the reference (src/math.br:66-68) and in
checkpoints, so nothing is transposed at load. Which kernel runs is the kernel library's business
(`ops.gemm`): float32 operands always take the plain CUDA-core kernel (true 32-bit), bfloat16
operands a tensor-core kernel chosen by the product's shape.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..kernels.ops import EPI_NONE, EPI_BIAS, EPI_RESIDUAL, EPI_SWIGLU


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T)."""
    ops.gemm(x, w, out, bias, epilogue, fast=ctx.fast)
