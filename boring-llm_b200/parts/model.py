"""A decoder put together from parts, with the order of its layers as data."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..weights import TensorSpec
from .base import Part, takes_pending_norm


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run block `block` on cache layer `cache`. A block may be named
    by several entries (its weights run twice), and an entry with `write_cache` false reads the
    cache layer that an earlier entry wrote instead of writing one of its own."""
    block: int
    cache: Optional[int]
    write_cache: bool = True


class DecoderModel(Part):
    """embedding -> blocks in `schedule` order -> final norm -> output head.

    The reference runs its layers in a fixed loop (src/model.br:1297-1358); here the loop's order is
    a list so that models which repeat layers or share caches need no new code.
    """

    def __init__(self, embedding, blocks: Sequence[Part], final_norm, head,
                 schedule: Optional[Sequence[LayerCall]] = None, ignorable_tensors: Sequence[str] = ()):
        super().__init__()
        self.embedding, self.blocks, self.final_norm, self.head = embedding, list(blocks), final_norm, head
        self.schedule: List[LayerCall] = list(schedule) if schedule is not None else [
            LayerCall(i, i if b.cache_spec() is not None else None) for i, b in enumerate(self.blocks)]
        self.ignorable_tensors = tuple(ignorable_tensors)
        written = set()
        for call in self.schedule:
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"run order names block {call.block}, but there are {len(self.blocks)}")
            if call.cache is not None:
                if call.write_cache:
                    if call.cache in written:
                        raise ValueError(f"cache layer {call.cache} is written by two entries of the run order")
                    written.add(call.cache)
                elif call.cache not in written:
                    raise ValueError(f"an entry reads cache layer {call.cache} before any entry writes it")

    def children(self):
        return (self.embedding, *self.blocks, self.final_norm, self.head)

    @property
    def vocab_size(self) -> int:
        return self.head.vocab

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be captured in a CUDA graph and replayed."""
        return all(getattr(b, "graph_safe", False) for b in self.blocks)

    def cache_specs(self) -> list:
        """What each cache layer needs, indexed by cache layer (None where unused)."""
        n = 1 + max([c.cache for c in self.schedule if c.cache is not None], default=-1)
        specs = [None] * n
        for call in self.schedule:
            if call.cache is None:
                continue
            spec = self.blocks[call.block].cache_spec()
            if specs[call.cache] is not None and specs[call.cache] != spec:
                raise ValueError(f"cache layer {call.cache} is shared by layers with different needs")
            specs[call.cache] = spec
        return specs

    def forward(self, ctx) -> torch.Tensor:
        """Runs the tokens of `ctx` through every layer and returns 32-bit logits at `ctx.logit_rows`."""
        ctx.memo.clear()                        # a context may be run again (before a capture, at a replay's capture): nothing is carried over
        x = self.embedding.forward(ctx)
        for i, call in enumerate(self.schedule):
            # the norm that reads the stream after this block: the next block's first (the final norm reads a few rows only)
            after = self.blocks[self.schedule[i + 1].block] if i + 1 < len(self.schedule) else None
            reader = getattr(after, "mixer", None)
            ctx.norm_after_block = getattr(after, "mixer_norm", None) if takes_pending_norm(reader, x.shape[0]) else None
            self.blocks[call.block].forward(ctx, x, call.cache, call.write_cache)
        ctx.norm_after_block = None
        if ctx.logit_rows.shape[0] == 0:
            return ctx.empty((0, self.vocab_size), torch.float32)
        fused = getattr(self.head, "forward_fused_norm", None)
        logits = fused(ctx, x, self.final_norm, ctx.logit_rows) if fused is not None else None
        if logits is None:
            logits = self.head.forward(ctx, self.final_norm.forward(ctx, x, ctx.logit_rows))
        return logits
