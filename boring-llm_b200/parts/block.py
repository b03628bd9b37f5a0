"""How a norm, a mixer and a feed-forward are arranged in one layer."""
from __future__ import annotations

from typing import Optional

from .base import Part, takes_pending_norm


class PreNormBlock(Part):
    """x += mixer(norm1(x)); x += ffn(norm2(x)): sequential residuals around pre-norms, the
    arrangement of the reference's plain layer (src/model.br:1297-1358 with residual_type 0)."""

    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        super().__init__()
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def children(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.mixer, "graph_safe", False) and getattr(self.ffn, "graph_safe", False))

    def forward(self, ctx, x, cache_layer: Optional[int], write_cache: bool = True) -> None:
        # a mixer or feed-forward may take the norm in front of it into its first kernel (steps with few rows)
        # (and the product that adds into the stream may begin the norm that reads it next: ctx.next_norm says which,
        # and a part that can finish such a norm says so with `takes_pending_norm`, or, by the step's number of rows,
        # with `takes_pending_norm_at`)
        ctx.next_norm = self.ffn_norm if takes_pending_norm(self.ffn, x.shape[0]) else None
        if not self.mixer.forward_fused_norm(ctx, x, self.mixer_norm, cache_layer, write_cache):
            h = self._normed(ctx, self.mixer_norm, x, self.mixer)
            self.mixer.forward(ctx, h, x, cache_layer, write_cache)
        ctx.next_norm = ctx.norm_after_block
        if not self.ffn.forward_fused_norm(ctx, x, self.ffn_norm):
            h = self._normed(ctx, self.ffn_norm, x, self.ffn)
            self.ffn.forward(ctx, h, x)
        ctx.next_norm = None

    @staticmethod
    def _normed(ctx, norm, x, reader):
        if takes_pending_norm(reader, x.shape[0]) and hasattr(norm, "dim"):
            try:
                return norm.forward(ctx, x, pending_ok=True)
            except TypeError:                    # a norm part without the option
                pass
        return norm.forward(ctx, x)
