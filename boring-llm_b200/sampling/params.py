"""Sampling options of one request and the host's random number generator.

Names and defaults follow the reference's command line (src/main.br:568-590) and its
`SamplingParams` (src/model.br:1565-1589): greedy unless a temperature is given; top_k 0, top_p 1,
min_p 0 and repeat_penalty 1 switch their filter off; seed 0.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Sequence, Tuple

_MASK64 = (1 << 64) - 1
_SEED_CONSTANT = 88172645463325252


@dataclass
class SamplingParams:
    n_predict: int = 40                 # -n / --n-predict: tokens to generate (src/main.br:563-565)
    temperature: float = 0.0            # --temp: 0 is greedy (:568-569)
    seed: int = 0                       # -s / --seed (:583)
    top_k: int = 0                      # --top-k, 0 keeps every candidate
    top_p: float = 1.0                  # --top-p
    min_p: float = 0.0                  # --min-p
    repeat_penalty: float = 1.0         # --repeat-penalty
    repeat_last_n: int = 64             # --repeat-last-n: -1 the whole history, 0 off
    eos_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False

    def __post_init__(self):
        self.eos_token_ids = tuple(self.eos_token_ids)
        if self.top_k < 0:
            self.top_k = 0
        if not 0.0 < self.top_p:
            raise ValueError(f"top_p must be positive, got {self.top_p}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must lie in [0, 1], got {self.min_p}")
        if not self.repeat_penalty > 0:
            raise ValueError(f"repeat_penalty must be positive, got {self.repeat_penalty}")


class XorShift64:
    """The reference's generator (src/sampling.br:18-54): state = seed ^ constant (seed 0: the
    constant itself), x ^= x << 13; x ^= x >> 7; x ^= x << 17; a uniform number is float32(x) / 2^64."""

    def __init__(self, seed: int):
        self.state = _SEED_CONSTANT if seed == 0 else ((seed & _MASK64) ^ _SEED_CONSTANT)

    def next_u64(self) -> int:
        x = self.state
        x ^= (x << 13) & _MASK64
        x ^= x >> 7
        x ^= (x << 17) & _MASK64
        self.state = x
        return x

    def next_f32(self) -> float:
        x = self.next_u64()
        as_f32 = struct.unpack("<f", struct.pack("<f", float(x)))[0]   # uint64 -> float32, rounded to nearest
        return as_f32 / 18446744073709551616.0


def penalty_window(history: Sequence[int], repeat_last_n: int):
    """Distinct tokens of the window the repeat penalty looks at (src/sampling.br:71-84)."""
    if repeat_last_n == 0 or not history:
        return []
    window = history[-repeat_last_n:] if 0 < repeat_last_n < len(history) else history
    return list(dict.fromkeys(window))
