"""Device tensors behind the cache manager's page and slot numbers.

For every paged group one tensor `[layers in group, 2 (keys, values), pages + 1, kv heads, page size,
head size]`: the rows of one (page, kv head) lie together, so a kernel reads a page of one head as
one contiguous tile. For every state group one tensor `[layers in group, request slots, *shape]`.
Keys are stored after rotation, values as projected (src/model.br:1814-1820).
"""
from __future__ import annotations

from typing import List

import torch

from .manager import CacheManager

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class CacheStorage:
    def __init__(self, manager: CacheManager, kv_dtype: torch.dtype, device):
        self.manager = manager
        self.kv_dtype = kv_dtype
        self.device = torch.device(device)
        # One page and one slot more than the manager hands out: rows that only pad a batch to a fixed
        # size (captured CUDA graphs) write there, where no request ever reads.
        self.trash_page = manager.num_pages
        self.trash_slot = manager.max_requests
        self.kv: List[torch.Tensor] = []
        for g in manager.paged_groups:
            self.kv.append(torch.zeros(
                (len(g.cache_layers), 2, manager.num_pages + 1, g.spec.n_kv_heads, manager.page_size,
                 g.spec.head_dim), dtype=kv_dtype, device=self.device))
        self.state: List[torch.Tensor] = []
        for sg in manager.state_groups:
            self.state.append(torch.zeros(
                (len(sg.cache_layers), manager.max_requests + 1) + tuple(sg.spec.shape),
                dtype=_TORCH_DTYPES[sg.spec.dtype], device=self.device))
        manager._on_slot_assigned = self.zero_slot

    def poison_freed_pages(self) -> int:
        """Debugging aid: fills every page that was given back since the last call (and, the first time, every page
        that no request holds, the spare page included) with NaN, keys and values in all layers. Freed pages are
        otherwise left as they are, because nothing may read a request's cache past its length; with poison a
        kernel that does read there, even with weight zero, turns its output into NaN. Returns the pages filled."""
        n = 0
        for g, kv in zip(self.manager.paged_groups, self.kv):
            if g.pool.freed_log is None:
                g.pool.freed_log = []
                pages = [p for p in range(g.pool.num_pages) if g.pool.owner_of(p) is None] + [self.trash_page]
            else:
                pages, g.pool.freed_log = [p for p in set(g.pool.freed_log) if g.pool.owner_of(p) is None], []
            if pages and kv.dtype.is_floating_point:
                kv[:, :, torch.tensor(pages, dtype=torch.long, device=self.device)] = float("nan")
                n += len(pages)
        return n

    def zero_slot(self, slot: int) -> None:
        for t in self.state:
            t[:, slot].zero_()

    def keys(self, cache_layer: int) -> torch.Tensor:
        kind, gi, li = self.manager.layer_location[cache_layer]
        assert kind == "paged"
        return self.kv[gi][li, 0]

    def values(self, cache_layer: int) -> torch.Tensor:
        kind, gi, li = self.manager.layer_location[cache_layer]
        assert kind == "paged"
        return self.kv[gi][li, 1]

    def layer_state(self, cache_layer: int) -> torch.Tensor:
        """`[request slots, *shape]` of one cache layer with fixed-size state."""
        kind, gi, li = self.manager.layer_location[cache_layer]
        assert kind == "state"
        return self.state[gi][li]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv + self.state)
