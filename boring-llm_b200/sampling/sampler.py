"""Turns the step's logits into one token per row with the device kernels."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams, XorShift64, penalty_window


class Sampler:
    """`sample(logits, rows)`: `rows` is a list of (params, generator, history) per logits row; `history` is a
    list of token ids or an object with a `tokens` attribute (read only when a penalty is on).
    Greedy rows do not advance their generator (src/sampling.br:496-497); every other row draws
    one number per token. The choice itself runs in `bl_sample` on the device."""

    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, rows: Sequence[tuple]) -> List[int]:
        n = len(rows)
        if n == 0:
            return []
        assert logits.shape[0] == n
        f = np.zeros((4, n), dtype=np.float32)        # temperature, top_p, min_p, uniform
        k = np.zeros(n, dtype=np.int32)
        pen_tokens: List[int] = []
        pen_offsets = [0]
        pen = np.ones(n, dtype=np.float32)
        for i, (p, rng, history) in enumerate(rows):
            f[0, i], f[1, i], f[2, i] = p.temperature, p.top_p, p.min_p
            k[i] = p.top_k
            if p.temperature > 0:
                f[3, i] = rng.next_f32()
            if p.repeat_penalty != 1.0:
                pen[i] = p.repeat_penalty
                tokens = history.tokens if hasattr(history, "tokens") else history
                pen_tokens.extend(penalty_window(tokens, p.repeat_last_n))
            pen_offsets.append(len(pen_tokens))
        if pen_tokens:
            logits = logits.clone()
            ops.repeat_penalty(logits, torch.tensor(pen_tokens, dtype=torch.int32, device=self.device),
                               torch.tensor(pen_offsets, dtype=torch.int32, device=self.device),
                               torch.from_numpy(pen).to(self.device))
        fd = torch.from_numpy(f).to(self.device)
        kd = torch.from_numpy(k).to(self.device)
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        ops.sample(logits, fd[0], kd, fd[1], fd[2], fd[3], out)
        return out.cpu().tolist()
