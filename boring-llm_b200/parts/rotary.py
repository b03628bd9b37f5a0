"""Position encodings applied between projection and cache write."""
from __future__ import annotations

import numpy as np
import torch


class RotaryTable:
    """Per-pair rotation table, as the reference builds it (src/math.br:107-113, 161-171):
    `inv_freq[j] = 1 / base^(2j / n_rot)` in 32-bit for the n_rot/2 rotated pairs, zero past them, a
    magnitude scale for cos/sin, the number of rotated pairs, and which dimensions form a pair:
    "halves" (j, j + n_rot/2) inside each head, the NEOX style of this architecture, or "interleaved"
    (2j, 2j + 1) (src/math.br:128-157, the `neox` argument). Every variant of rotary scaling is just
    another table, so the kernel never branches on the variant.
    """

    PAIR_LAYOUTS = {"halves": 0, "interleaved": 1}

    def __init__(self, head_dim: int, base: float, n_rot: int | None = None, mscale: float = 1.0,
                 pairs: str = "halves"):
        n_rot = head_dim if n_rot is None else n_rot
        if pairs not in self.PAIR_LAYOUTS:
            raise ValueError(f"rotary: pairs must be one of {sorted(self.PAIR_LAYOUTS)}, got {pairs!r}")
        self.pairs, self.pair_layout = pairs, self.PAIR_LAYOUTS[pairs]
        if n_rot % 2 != 0 or n_rot > head_dim or n_rot < 0:
            raise ValueError(f"rotary: {n_rot} rotated dimensions do not fit a head of {head_dim}")
        self.head_dim, self.base, self.n_rot, self.mscale = head_dim, float(base), n_rot, float(mscale)
        self.rot_half = n_rot // 2
        f = np.zeros(head_dim // 2, dtype=np.float32)
        j = np.arange(self.rot_half, dtype=np.float32)
        if self.rot_half:
            expo = (np.float32(2.0) * j) / np.float32(n_rot)
            f[: self.rot_half] = np.float32(1.0) / np.power(np.float32(base), expo, dtype=np.float32)
        self.inv_freq_host = f
        self.inv_freq: torch.Tensor | None = None

    def to(self, device):
        self.inv_freq = torch.from_numpy(self.inv_freq_host).to(device)
        return self

    def step_table(self, ctx):
        """(cos, sin), float32 [T, rot_half] each, of the step's tokens: worked out by the first layer that asks and
        kept in the step's memo for the others (the positions are the same for every layer)."""
        key = ("rotary table", self.head_dim, self.base, self.n_rot, self.mscale)     # the layers' tables are equal, not the same object
        if key not in ctx.memo:
            from ..kernels import ops
            ctx.memo[key] = ops.rope_table(ctx.positions, self.inv_freq, self.rot_half, self.mscale)
        return ctx.memo[key]
