"""Normalisation parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..weights import TensorSpec, NORM
from .base import Part


class RMSNorm(Part):
    """y = x / sqrt(mean(x^2) + eps) * weight, statistics in 32-bit, the weight used as stored
    (src/math.br:18-36). Input: the 32-bit residual stream; output: the engine's activation dtype."""

    def __init__(self, dim: int, eps: float, names: Dict[str, str]):
        super().__init__(names)
        self.dim, self.eps = dim, float(eps)
        self.weight: Optional[torch.Tensor] = None

    def local_specs(self):
        return {"weight": TensorSpec((self.dim,), NORM)}

    def forward(self, ctx, x: torch.Tensor, row_idx: Optional[torch.Tensor] = None, pending_ok: bool = False):
        """The normed rows. `pending_ok`: the caller can finish a norm that the product before it has begun; it then
        gets `PendingNormRows` when the step holds them for this stream and this norm."""
        if pending_ok and row_idx is None:
            held = ctx.memo.get(("pending norm", id(x)))
            if held is not None and held.norm is self:
                return held
        rows = x.shape[0] if row_idx is None else row_idx.shape[0]
        out = ctx.empty((rows, self.dim))
        ops.rmsnorm(x, self.weight, self.eps, out, row_idx)
        return out
