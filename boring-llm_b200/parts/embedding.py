"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..weights import TensorSpec, MATRIX
from .base import Part, to_device_matrix
from .linear import linear, EPI_NONE


FUSED_MAX_COLUMNS = 16384


class Embedding(Part):
    """x[t] = table[token[t]] (src/model.br:1286-1295; the reference's embedding scale is 1 here),
    widened to the 32-bit residual stream."""

    def __init__(self, vocab: int, dim: int, names: Dict[str, str]):
        super().__init__(names)
        self.vocab, self.dim = vocab, dim
        self.table: Optional[torch.Tensor] = None

    def local_specs(self):
        return {"table": TensorSpec((self.vocab, self.dim), MATRIX)}

    def place(self, local, dtype, device):
        self.table = to_device_matrix(local["table"], dtype, device)

    def forward(self, ctx) -> torch.Tensor:
        x = ctx.empty((ctx.T, self.dim), torch.float32)
        ops.embed(self.table, ctx.token_ids, x)
        return x


class OutputHead(Part):
    """logits = y . W^T in 32-bit, no bias (src/model.br:1360-1362). Tied to an embedding: the
    table is shared, not copied (src/model.br:686-690)."""

    def __init__(self, vocab: int, dim: int, names: Dict[str, str], tied_to: Optional[Embedding] = None):
        super().__init__(names)
        self.vocab, self.dim, self.tied_to = vocab, dim, tied_to
        self.weight: Optional[torch.Tensor] = None

    def local_specs(self):
        return {} if self.tied_to is not None else {"weight": TensorSpec((self.vocab, self.dim), MATRIX)}

    def place(self, local, dtype, device):
        if self.tied_to is None:
            self.weight = to_device_matrix(local["weight"], dtype, device)

    def matrix(self) -> torch.Tensor:
        return self.tied_to.table if self.tied_to is not None else self.weight

    def forward_fused_norm(self, ctx, x: torch.Tensor, norm, row_idx: torch.Tensor) -> Optional[torch.Tensor]:
        """Final norm and output product in one kernel for few rows; None when that is not possible."""
        from .attention import FUSED_MAX_ROWS
        from .norm import RMSNorm
        # every block of the fused kernel normalises the rows again: worth it for a few hundred blocks, not for
        # the thousands that a large vocabulary makes
        if not (ctx.fast and ctx.dtype == torch.bfloat16 and row_idx.shape[0] <= FUSED_MAX_ROWS
                and self.vocab <= FUSED_MAX_COLUMNS
                and isinstance(norm, RMSNorm) and ops.norm_gemm_supported(x, self.matrix())):
            return None
        logits = ctx.empty((row_idx.shape[0], self.vocab), torch.float32)
        ops.norm_gemm(x, norm.weight, norm.eps, self.matrix(), logits, None, EPI_NONE, row_idx)
        return logits

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        logits = ctx.empty((y.shape[0], self.vocab), torch.float32)
        linear(ctx, y, self.matrix(), logits, None, EPI_NONE)
        return logits
