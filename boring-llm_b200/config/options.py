"""Run-time settings that are not model configuration.

The reference sets these as module statics before loading (src/main.br:1212-1216: KV types,
context size, prefill chunk); here they are one value passed to the engine.
"""
from __future__ import annotations

from dataclasses import dataclass

DTYPES = ("bfloat16", "float32")


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"             # "bfloat16": serving kernels; "float32": true 32-bit everywhere
    page_size: int = 16                 # tokens per cache page
    max_tokens: int = 0                 # cache capacity in tokens (0: ctx_size * max_num_seqs)
    ctx_size: int = 4096                # prompt + reply limit of one request (-c, src/main.br:638-639)
    max_num_seqs: int = 64              # live requests (slots of per-request state)
    max_num_batched_tokens: int = 2048  # token budget of one step (-b, src/main.br:674-676)
    prefill_chunk: int = 512            # most prompt tokens of one request in a step (-ub, :677-679)
    cuda_graphs: bool = True            # replay captured decode steps
    step_graph_after: int = 2           # capture a general step's padded shape when it comes this many times (0: never)
    lookahead: bool = True              # launch the next decode step (its tokens taken on the device) before this one's are read
    debug_poison: bool = False          # fill pages with NaN when they are given back: a read past a request's length shows
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype in ("bf16",):
            self.dtype = "bfloat16"
        if self.dtype in ("fp32", "f32"):
            self.dtype = "float32"
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        for name in ("page_size", "ctx_size", "max_num_seqs", "max_num_batched_tokens", "prefill_chunk"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive, got {getattr(self, name)}")
        if self.max_tokens < 0:
            raise ValueError(f"max_tokens must not be negative, got {self.max_tokens}")

    @property
    def effective_prefill_chunk(self) -> int:
        """min(batch, ubatch), as `effective_prefill_chunk` (src/cli_config.br:24-25)."""
        return min(self.max_num_batched_tokens, self.prefill_chunk)

    @property
    def capacity_tokens(self) -> int:
        return self.max_tokens if self.max_tokens > 0 else self.ctx_size * self.max_num_seqs
