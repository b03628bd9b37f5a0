"""Feed-forward parts: rows in, rows out, no cache."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights import TensorSpec, MATRIX
from .base import Part, to_device_matrix
from .linear import linear, EPI_RESIDUAL, EPI_SWIGLU


FF_FUSED_MAX_ROWS = 16    # more rows: a separate norm and the tcgen05 product are faster (measured: 6% of a step at 24 and 32 rows)


class FeedForward(Part):
    """Interface: `forward(ctx, h, residual)` reads the normed rows `h` [T, dim] and adds its
    result into the 32-bit `residual` [T, dim] in place. `graph_safe` as for mixers."""
    graph_safe = False

    def forward(self, ctx, h, residual) -> None:
        raise NotImplementedError

    def forward_fused_norm(self, ctx, x, norm) -> bool:
        """Optional: run `norm` and this feed-forward on the residual stream `x` in fused kernels and return
        True, or return False to be called with the normed rows as usual."""
        return False


class SwiGLU(FeedForward):
    """down(silu(gate(h)) * up(h)), no biases (src/math.br:232-233, 246-261). Gate and up run as
    one joined product over [Wg; Wu] (src/model.br:788-792) whose epilogue combines them
    (src/math_gpu.br:2673-2692); the down product adds into the residual stream."""
    graph_safe = True
    takes_pending_norm = True            # its first product can finish an RMS norm that the product before has begun

    def __init__(self, dim: int, hidden: int, names: Dict[str, str]):
        super().__init__(names)
        self.dim, self.hidden = dim, hidden
        self.w_gate_up = self.w_down = None

    def local_specs(self):
        return {"w_gate": TensorSpec((self.hidden, self.dim), MATRIX),
                "w_up": TensorSpec((self.hidden, self.dim), MATRIX),
                "w_down": TensorSpec((self.dim, self.hidden), MATRIX)}

    def place(self, local, dtype, device):
        self.w_gate_up = to_device_matrix(torch.cat([local["w_gate"], local["w_up"]], dim=0), dtype, device)
        self.w_down = to_device_matrix(local["w_down"], dtype, device)

    def takes_pending_norm_at(self, rows: int) -> bool:
        """gate/up finishes a norm that the product before has begun where it runs on pairs of SMs (many rows) or on the
        register-streaming kernel (a decode step's 2 to 16 rows, a matrix of up to 592 blocks of 16 columns that does
        not stream better through TMA); elsewhere the product before need not begin one."""
        if rows >= ops.PAIR_MIN_ROWS:
            return True
        return (ops.SKINNY_LINK_MIN_ROWS <= rows <= ops.SKINNY_LINK_MAX_ROWS and self.w_gate_up is not None
                and -(-self.hidden // 16) <= ops.SKINNY_LINK_MAX_BLOCKS and not ops.gemm_streams_better(self.w_gate_up))

    def forward_fused_norm(self, ctx, x, norm) -> bool:
        from .norm import RMSNorm
        if not (ctx.fast and ctx.dtype == torch.bfloat16 and x.shape[0] <= FF_FUSED_MAX_ROWS and isinstance(norm, RMSNorm)
                and ops.norm_gemm_supported(x, self.w_gate_up) and not ops.gemm_streams_better(self.w_gate_up)):
            return False
        held = ctx.memo.get(("pending norm", id(x)))
        if held is not None and held.norm is norm:
            return False                # the product before has begun this norm: `forward` finishes it in gate/up's epilogue
        act = ctx.empty((x.shape[0], self.hidden))
        ops.norm_gemm(x, norm.weight, norm.eps, self.w_gate_up, act, None, EPI_SWIGLU)
        linear(ctx, act, self.w_down, x, None, EPI_RESIDUAL)
        return True

    def forward(self, ctx, h, residual):
        act = ctx.empty((h.shape[0], self.hidden))
        linear(ctx, h, self.w_gate_up, act, None, EPI_SWIGLU)
        linear(ctx, act, self.w_down, residual, None, EPI_RESIDUAL)
