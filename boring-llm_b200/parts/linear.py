"""y = x . W^T with a fused epilogue: the one place that chooses between the matrix-product kernels.

W is stored (outputs x inputs) row-major, as in the reference (src/math.br:66-68) and in
checkpoints, so nothing is transposed at load.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..kernels.ops import EPI_NONE, EPI_BIAS, EPI_RESIDUAL, EPI_SWIGLU


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T). float32 operands always take the plain CUDA-core kernel (true 32-bit)."""
    ops.gemm_plain(x, w, out, bias, epilogue)
