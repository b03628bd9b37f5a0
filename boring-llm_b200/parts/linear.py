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


def linear(ctx, x, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T).

    Two products of a layer may share an RMS norm between them without a pass over the rows (bfloat16; many rows: the
    kernels on pairs of SMs; a decode step's few rows: the register-streaming kernel). The product that adds into the residual stream, when the step says which norm reads the
    stream next (`ctx.next_norm`), also leaves that norm's rows pending in the step's memo; a product that is handed
    `PendingNormRows` as its x finishes the norm in its epilogue, or has them normed the ordinary way."""
    from .base import PendingNormRows
    from .norm import RMSNorm
    if isinstance(x, PendingNormRows):
        if epilogue == EPI_SWIGLU and bias is None and ops.gemm_on_pairs(x.rows, w, out.shape[1], epilogue, ctx.fast):
            ops.gemm_swiglu_scaled(x.rows, w, out, x.sums, x.eps)
            return
        if epilogue != EPI_RESIDUAL and ops.gemm_skinny_links_norm(x.rows, w, out.shape[1], epilogue, ctx.fast):
            ops.gemm_skinny_scaled(x.rows, w, out, x.sums, x.eps, bias, epilogue)
            return
        x = x.normed(ctx)
    norm = ctx.next_norm
    if (epilogue == EPI_RESIDUAL and bias is None and isinstance(norm, RMSNorm) and norm.weight is not None
            and out.dtype == torch.float32 and out.shape[1] % 4 == 0 and norm.dim == out.shape[1]):
        if ops.gemm_on_pairs(x, w, out.shape[1], epilogue, ctx.fast):
            hw, ss = ops.gemm_residual_norm(x, w, out, norm.weight)
            ctx.memo[("pending norm", id(out))] = PendingNormRows(hw, ss, norm, out)
            return
        if out.shape[1] % 8 == 0 and ops.gemm_skinny_links_norm(x, w, out.shape[1], epilogue, ctx.fast):
            hw, ss = ops.gemm_skinny_residual_norm(x, w, out, norm.weight)
            ctx.memo[("pending norm", id(out))] = PendingNormRows(hw, ss, norm, out)
            return
    ops.gemm(x, w, out, bias, epilogue, fast=ctx.fast)
