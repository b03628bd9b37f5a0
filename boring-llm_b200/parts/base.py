"""What every part shares: the declaration of its tensors, and the step context it runs in.

A part (a norm, a position encoding, a mixer, a feed-forward, a block, an embedding, an output
head) takes every size and constant as a constructor argument and never learns which model it is
in. It declares its tensors under local names; the architecture's builder maps local names to
checkpoint names (role of the reference's per-architecture tensor names, src/model.br:614-690).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..weights import TensorSpec


class Part:
    """Base of all parts. `names` maps each local tensor name to its checkpoint name."""

    def __init__(self, names: Optional[Dict[str, str]] = None):
        self.names: Dict[str, str] = dict(names or {})

    # -- tensors ---------------------------------------------------------------------------------
    def local_specs(self) -> Dict[str, TensorSpec]:
        """Local tensor name -> what it must look like."""
        return {}

    def children(self) -> Sequence["Part"]:
        return ()

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Checkpoint tensor name -> spec, for this part and the parts inside it."""
        out: Dict[str, TensorSpec] = {}
        for local, spec in self.local_specs().items():
            if local not in self.names:
                raise KeyError(f"{type(self).__name__}: no checkpoint name given for tensor '{local}'")
            out[self.names[local]] = spec
        for c in self.children():
            for k, v in c.tensor_specs().items():
                if k in out and out[k] != v:
                    raise ValueError(f"tensor {k} is declared twice with different shapes")
                out[k] = v
        return out

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Takes this part's tensors (by checkpoint name) to the device. `dtype` is the engine's
        matrix dtype: bfloat16 matrices stay, float32 mode widens everything to 32-bit."""
        local = {l: tensors[self.names[l]] for l in self.local_specs()}
        self.place(local, dtype, device)
        for c in self.children():
            c.load(tensors, dtype, device)

    # -- per-step plans ----------------------------------------------------------------------------
    def plan_step(self, q_lens: Sequence[int], ctx_lens: Sequence[int], filler: Optional[int] = None):
        """Optional: what this part wants worked out on the host before a step runs (lists of work items that its
        kernels walk, launch shapes), as `(key, StepPlan)` or None. The step function asks every part, keeps one
        plan per key (layers of one kind share theirs), copies the plan's arrays to the device with the step's own
        index arrays and hands them back as `ctx.plans[key]`. `q_lens[r]` new tokens bring request r to
        `ctx_lens[r]` tokens. `filler` is None for a step that runs once; for a step that is captured and
        replayed with other batches of the same shape it is the index of a request without tokens: the plan's
        arrays must then have sizes that `StepPlan.shape` determines, padded with entries that point at the
        filler, and everything that decides a launch must come from `shape` alone."""
        return None

    def collect_plans(self, q_lens, ctx_lens, filler=None, into: Optional[dict] = None) -> dict:
        """The plans of this part and of the parts inside it, one per key."""
        into = {} if into is None else into
        got = self.plan_step(q_lens, ctx_lens, filler)
        if got is not None and got[0] not in into:
            into[got[0]] = got[1]
        for c in self.children():
            c.collect_plans(q_lens, ctx_lens, filler, into)
        return into

    def place(self, local: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Default: each local tensor becomes an attribute of the same name."""
        for name, t in local.items():
            setattr(self, name, to_device_matrix(t, dtype, device) if t.dim() >= 2 else to_device_vector(t, dtype, device))


def to_device_matrix(t: torch.Tensor, dtype: torch.dtype, device) -> torch.Tensor:
    """Matrices take the engine's dtype (the tensor cores want bfloat16; the 32-bit path wants float32)."""
    return t.to(device=device, dtype=dtype).contiguous()


def to_device_vector(t: torch.Tensor, dtype: torch.dtype, device) -> torch.Tensor:
    """Small vectors (norm weights, biases) keep 32-bit storage when they have it; in float32 mode
    bfloat16 ones are widened."""
    if dtype == torch.float32 or t.dtype == torch.float32:
        return t.to(device=device, dtype=torch.float32).contiguous()
    return t.to(device=device, dtype=torch.bfloat16).contiguous()


@dataclass
class StepPlan:
    """A part's host-side preparation of one step. `arrays`: int32 numpy arrays on the host, replaced by device
    tensors of the same shapes before the parts run. `host`: plain values for the part's own use. `shape`: a
    hashable value that, together with the batch's padded sizes, determines every launch the part will make (two
    steps with equal shapes can replay one captured graph)."""
    arrays: dict = field(default_factory=dict)
    host: dict = field(default_factory=dict)
    shape: tuple = ()


def takes_pending_norm(part, rows: int) -> bool:
    """Whether `part` finishes an RMS norm that the product before it has begun, in a step of `rows` rows: its
    `takes_pending_norm_at(rows)` if it has one, else its flag `takes_pending_norm`. The product before begins the
    norm only then (beginning it costs its epilogue a little; a reader that norms the stream itself gains nothing)."""
    at = getattr(part, "takes_pending_norm_at", None)
    return bool(at(rows)) if at is not None else bool(getattr(part, "takes_pending_norm", False))


class PendingNormRows:
    """Rows whose RMS norm has been begun by the product that wrote the residual stream and is finished by the product
    that reads them: `rows` = bfloat16(stream * norm weight), `sums` [T, parts] = sums of squares of each row of the
    stream (in parts, added in a fixed order), `eps` and the norm it is. A part that cannot take them asks for
    `normed(ctx)`, which runs the norm's own kernel on the stream."""

    def __init__(self, rows, sums, norm, stream):
        self.rows, self.sums, self.norm, self.stream = rows, sums, norm, stream
        self.eps = norm.eps
        self.shape = rows.shape

    def normed(self, ctx):
        return self.norm.forward(ctx, self.stream)


@dataclass
class StepContext:
    """Everything a part may look at while one step runs. Device tensors are int32.

    The batch is flat: `T` tokens of `R` requests, request r owning tokens cu_q[r] .. cu_q[r+1] - 1
    at positions ctx_len[r] - q_len[r] .. ctx_len[r] - 1.
    """
    dtype: torch.dtype
    device: torch.device
    T: int
    R: int
    token_ids: torch.Tensor            # [T]
    positions: torch.Tensor            # [T] absolute position of each token
    tok_req: torch.Tensor              # [T] index (in this batch) of the token's request
    cu_q: torch.Tensor                 # [R + 1]
    ctx_len: torch.Tensor              # [R] tokens the request holds after this step
    slots: torch.Tensor                # [R] the request's state slot
    logit_rows: torch.Tensor           # [N] flat token indices whose logits are wanted
    block_tables: List[torch.Tensor]   # per paged group: [R, width]
    q_lens: List[int]                  # host copies, for parts that choose a kernel or loop on the host
    ctx_lens: List[int]
    slot_list: List[int]
    storage: object                    # cache.CacheStorage
    fast: bool = True                  # False: plain kernels only (the twins)
    plans: dict = field(default_factory=dict)      # key -> StepPlan: what parts worked out on the host for this step
    memo: dict = field(default_factory=dict)       # what a part works out once per step and its other layers reuse
    next_norm: object = None                       # the norm that reads the residual stream after the part that runs now (or None)
    norm_after_block: object = None                # ... after the block that runs now

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    def kv(self, cache_layer: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(keys, values, block table) of a cache layer: pages `[pages, kv heads, page size, head size]`."""
        kind, gi, li = self.storage.manager.layer_location[cache_layer]
        if kind != "paged":
            raise TypeError(f"cache layer {cache_layer} holds fixed-size state, not pages")
        return self.storage.kv[gi][li, 0], self.storage.kv[gi][li, 1], self.block_tables[gi]

    def state(self, cache_layer: int) -> torch.Tensor:
        """`[request slots, *shape]` of a cache layer with fixed-size state; index it with `slots`."""
        return self.storage.layer_state(cache_layer)

    def empty(self, shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)
