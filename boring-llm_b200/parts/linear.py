"""y = x . W^T with a fused epilogue: the one place that chooses between the matrix-product kernels.

W is stored (outputs x inputs) row-major, as in the reference (src/math.br:66-68) and in
checkpoints, so nothing is transposed at load.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..kernels.ops import EPI_NONE, EPI_BIAS, EPI_RESIDUAL, EPI_SWIGLU

SKINNY_MAX_ROWS = 64      # up to here W streams through registers (measured faster than 128-row tcgen05 tiles at 64 rows)
TC_MIN_COLUMNS_FEW_ROWS = 4096   # 17..64 rows: wide products have enough 128-column tiles for TMA to stream W at full rate
TC_MIN_COLUMNS_VERY_FEW_ROWS = 32768   # an output head: up to 64 rows take the kernel made for it; without it the 128-row tiles win from 9 rows
PAIR_MIN_ROWS = 256       # from here on pairs of SMs share 256 x 256 tiles (tcgen05 cta_group::2)


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T). float32 operands always take the plain CUDA-core kernel (true 32-bit);
    bfloat16 operands take a tensor-core kernel chosen by the number of rows."""
    if ctx.fast and ops.gemm_skinny_supported(x, w):
        M, N = x.shape[0], out.shape[1]
        few_rows_tc = (M > 16 and N >= TC_MIN_COLUMNS_FEW_ROWS) or (M > 8 and N >= TC_MIN_COLUMNS_VERY_FEW_ROWS)
        if (N >= TC_MIN_COLUMNS_VERY_FEW_ROWS and bias is None and epilogue == EPI_NONE and M <= 64
                and ops.gemm_tc_cols_supported(x, w)):
            ops.gemm_tc_cols(x, w, out)            # an output head at decode time: W streams once, as the M side of the product
        elif M <= SKINNY_MAX_ROWS and not few_rows_tc:
            ops.gemm_skinny(x, w, out, bias, epilogue)
        elif x.shape[0] < PAIR_MIN_ROWS:
            ops.gemm_tc(x, w, out, bias, epilogue)
        else:
            ops.gemm_tc_pair(x, w, out, bias, epilogue)
    else:
        ops.gemm_plain(x, w, out, bias, epilogue)
