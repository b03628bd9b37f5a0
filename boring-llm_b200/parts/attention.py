"""Mixers: the parts of a block that let tokens see one another."""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from ..cache import PagedKVSpec
from ..kernels import ops
from ..weights import TensorSpec, MATRIX, BIAS
from .base import PendingNormRows, Part, StepPlan, to_device_matrix, to_device_vector
from .linear import linear, EPI_BIAS, EPI_NONE, EPI_RESIDUAL
from .norm import RMSNorm
from .rotary import RotaryTable

FUSED_MAX_ROWS = 64       # steps with at most this many rows take the fused norm + product kernels

QKV_EPILOGUE_MIN_ROWS = ops.PAIR_MIN_ROWS  # from here the joined product runs on pairs of SMs, whose epilogue can rotate and write the cache
PREFILL_TC_MIN_TOKENS = 256          # steps with fewer prompt tokens keep the 64-row tiles of the mma.sync kernel (measured: 512-token portions gain 8%)
DECODE_MAX_SPLITS = ops.DECODE_CLUSTER_SPLITS   # the slices of a request are one cluster of blocks that merge in shared memory
PLAN_KEY = "paged attention"         # one plan per step for all attention layers: its lists do not depend on head sizes


def tc_attention_tiles(q_lens, ctx_lens):
    """The launch list of the tcgen05 prefill attention: (request, first token) of every tile of 128 new tokens of
    the requests with more than one, the tile with the fewest keys first (the kernel starts from the end of the
    list, so that the long tiles run first and the short ones fill the tail). Key blocks are counted without the
    window (an upper bound)."""
    tiles = []                                           # [key blocks, request, first token]
    for r, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        if n <= 1:
            continue
        for t0 in range(0, n, 128):
            tiles.append([-(-(c - n + min(t0 + 128, n)) // 128), r, t0])
    tiles.sort()
    return [[r, t0] for _, r, t0 in tiles]


def attention_plan(q_lens, ctx_lens, filler=None) -> StepPlan:
    """What the attention kernels walk in one step: the 64-token tiles (and, for steps with many prompt tokens, the
    128-token tiles in launch order) of the requests with several new tokens, and the list of requests with a
    single one, with the longest context among those. For a step that will be replayed (`filler` given) the lists
    are padded to multiples of 8 with entries of the request without tokens, and the longest context is rounded up
    to a power of two: launches then depend on these sizes only."""
    tiles64 = [[r, t0] for r, n in enumerate(q_lens) if n > 1 for t0 in range(0, n, 64)]
    singles = [r for r, n in enumerate(q_lens) if n == 1]
    use_tc = sum(n for n in q_lens if n > 1) >= PREFILL_TC_MIN_TOKENS
    tiles128 = tc_attention_tiles(q_lens, ctx_lens) if use_tc else []
    longest = max((ctx_lens[r] for r in singles), default=0)
    if filler is not None:
        pad = lambda n: -(-n // 8) * 8 - n
        tiles64 = tiles64 + [[filler, 0]] * pad(len(tiles64))
        tiles128 = [[filler, 0]] * pad(len(tiles128)) + tiles128          # the front of this list is launched last
        singles = singles + [filler] * pad(len(singles))
        bucket = 256
        while bucket < longest:
            bucket *= 2
        longest = bucket if singles else 0
    return StepPlan(
        arrays={"tiles64": np.asarray(tiles64, dtype=np.int32).reshape(-1, 2),
                "tiles128": np.asarray(tiles128, dtype=np.int32).reshape(-1, 2),
                "singles": np.asarray(singles, dtype=np.int32)},
        host={"longest_single": longest},
        shape=(len(tiles64), len(tiles128), len(singles), longest))


class Mixer(Part):
    """Interface of a mixer.

    `cache_spec()` says what one cache layer of this mixer needs (`PagedKVSpec`, `StateSpec` or
    None). `forward(ctx, h, residual, cache_layer, write_cache)` reads the normed rows `h` [T, dim],
    adds its result into the 32-bit `residual` [T, dim] in place, and may read and write the cache
    layer it is given through `ctx.kv(cache_layer)` / `ctx.state(cache_layer)`. With `write_cache`
    false it reads a layer that another call has written in this step.
    """

    # True when forward() only launches work on the current stream from device-side inputs (no host loops
    # over the batch, no host reads): such a mixer may be captured in a CUDA graph and replayed.
    graph_safe = False

    def cache_spec(self):
        return None

    def forward(self, ctx, h, residual, cache_layer: Optional[int], write_cache: bool = True) -> None:
        raise NotImplementedError

    def forward_fused_norm(self, ctx, x, norm, cache_layer: Optional[int], write_cache: bool = True) -> bool:
        """Optional: run `norm` and this mixer on the residual stream `x` in fused kernels and return True,
        or return False to be called with the normed rows as usual."""
        return False


class GQAAttention(Mixer):
    """Causal grouped-query attention over the paged cache.

    q, k, v = h.Wq^T + bq, h.Wk^T + bk, h.Wv^T + bv as ONE joined product (src/model.br:765-768,
    864-869, 1113-1115); q and k rotated by position; k cached after rotation, v as projected
    (:1814-1820); softmax(q.k^T * scale) over the keys a token may see (src/math.br:304-359);
    out.Wo^T added to the residual stream (src/model.br:1328-1334).
    """
    graph_safe = True
    takes_pending_norm = True            # its first product can finish an RMS norm that the product before has begun

    def takes_pending_norm_at(self, rows: int) -> bool:
        """... in steps with enough rows for the product on pairs of SMs (with few rows the norm is part of the q/k/v
        kernel, which reads the stream itself: measured, a norm begun by the layer before's down projection made a
        batch-8 decode step 4 % slower)."""
        return rows >= QKV_EPILOGUE_MIN_ROWS

    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, head_dim: int, rotary: Optional[RotaryTable],
                 names: Dict[str, str], qkv_bias: bool = True, out_bias: bool = False, window: int = 0,
                 scale: Optional[float] = None):
        super().__init__(names)
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"{n_heads} query heads cannot share {n_kv_heads} key/value heads")
        self.out_bias = bool(out_bias)
        self.dim, self.H, self.KV, self.dh = dim, n_heads, n_kv_heads, head_dim
        self.rotary = rotary if rotary is not None else RotaryTable(head_dim, 10000.0, n_rot=0)
        self.qkv_bias, self.window = qkv_bias, int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.w_qkv = self.b_qkv = self.wo = self.bo = None

    def local_specs(self):
        s = {"wq": TensorSpec((self.H * self.dh, self.dim), MATRIX),
             "wk": TensorSpec((self.KV * self.dh, self.dim), MATRIX),
             "wv": TensorSpec((self.KV * self.dh, self.dim), MATRIX),
             "wo": TensorSpec((self.dim, self.H * self.dh), MATRIX)}
        if self.qkv_bias:
            s.update({"bq": TensorSpec((self.H * self.dh,), BIAS), "bk": TensorSpec((self.KV * self.dh,), BIAS),
                      "bv": TensorSpec((self.KV * self.dh,), BIAS)})
        if self.out_bias:                       # read per file in the reference (src/model.br:500, 1328)
            s["bo"] = TensorSpec((self.dim,), BIAS)
        return s

    def place(self, local, dtype, device):
        self.w_qkv = to_device_matrix(torch.cat([local["wq"], local["wk"], local["wv"]], dim=0), dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        if self.qkv_bias:
            b = [local["bq"], local["bk"], local["bv"]]
            if any(t.dtype == torch.float32 for t in b):
                b = [t.to(torch.float32) for t in b]
            self.b_qkv = to_device_vector(torch.cat(b, dim=0), dtype, device)
        if self.out_bias:
            self.bo = to_device_vector(local["bo"], dtype, device)
        self.rotary.to(device)

    def cache_spec(self):
        return PagedKVSpec(self.KV, self.dh, self.window)

    def forward(self, ctx, h, residual, cache_layer, write_cache=True):
        T = h.shape[0]
        width = (self.H + 2 * self.KV) * self.dh
        k_cache, v_cache, table = ctx.kv(cache_layer)
        q = ctx.empty((T, self.H * self.dh))
        pending = h if isinstance(h, PendingNormRows) else None
        rows = pending.rows if pending is not None else h
        if (ctx.fast and T >= QKV_EPILOGUE_MIN_ROWS and self.rotary.pair_layout == 0 and self.rotary.rot_half * 2 == self.dh
                and ops.qkv_rope_tc_supported(rows, self.w_qkv, self.H, self.KV, self.dh, k_cache.shape[2])):
            # many rows: bias, rotation and the writes of q, k and v are the epilogue of the joined product (and the
            # scale of a norm that the product before has begun)
            cs, sn = self.rotary.step_table(ctx)
            ops.qkv_rope_tc(rows, self.w_qkv, self.b_qkv if self.qkv_bias else None, ctx.positions, ctx.tok_req, table, cs, sn,
                            q, k_cache if write_cache else None, v_cache if write_cache else None, self.H, self.KV, self.dh,
                            row_sums=pending.sums if pending is not None else None, eps=pending.eps if pending is not None else 0.0)
        else:
            if pending is not None:
                h = pending.normed(ctx)
            qkv = ctx.empty((T, width), torch.float32)
            linear(ctx, h, self.w_qkv, qkv, self.b_qkv, EPI_BIAS if self.qkv_bias else EPI_NONE)
            ops.rope_kv_write(qkv, ctx.positions, ctx.tok_req, table, self.rotary.inv_freq, self.rotary.rot_half,
                              self.rotary.mscale, q, k_cache if write_cache else None,
                              v_cache if write_cache else None, self.H, self.KV, self.dh, self.rotary.pair_layout)
        attn = ctx.empty((T, self.H * self.dh))
        self.attend(ctx, q, k_cache, v_cache, table, attn)
        self.project_out(ctx, attn, residual)

    def project_out(self, ctx, attn, residual):
        """residual += attn . Wo^T (+ bo)."""
        if self.out_bias:
            ops.add_row_vector(residual, self.bo)
        linear(ctx, attn, self.wo, residual, None, EPI_RESIDUAL)

    def forward_fused_norm(self, ctx, x, norm, cache_layer, write_cache=True) -> bool:
        """Few rows in bfloat16: norm, joined product, bias, rotation and cache write are ONE kernel."""
        T = x.shape[0]
        if not (ctx.fast and ctx.dtype == torch.bfloat16 and T <= FUSED_MAX_ROWS and isinstance(norm, RMSNorm)
                and self.rotary.rot_half * 2 == self.dh and self.dh % 16 == 0
                and ops.norm_gemm_supported(x, self.w_qkv)):
            return False
        k_cache, v_cache, table = ctx.kv(cache_layer)
        q = ctx.empty((T, self.H * self.dh))
        ops.norm_qkv_rope(x, norm.weight, norm.eps, self.w_qkv, self.b_qkv if self.qkv_bias else None,
                          ctx.positions, ctx.tok_req, table, self.rotary.inv_freq, self.rotary.mscale, q,
                          k_cache if write_cache else None, v_cache if write_cache else None, self.H, self.KV, self.dh,
                          self.rotary.pair_layout)
        attn = ctx.empty((T, self.H * self.dh))
        self.attend(ctx, q, k_cache, v_cache, table, attn)
        self.project_out(ctx, attn, x)
        return True

    def plan_step(self, q_lens, ctx_lens, filler=None):
        return PLAN_KEY, attention_plan(q_lens, ctx_lens, filler)

    def attend(self, ctx, q, k_cache, v_cache, table, out):
        """Tensor-core kernels for bfloat16 where they are built (pages of 16, common head sizes): one launch for
        the requests with several new tokens (the tcgen05 kernel for head sizes 64 and 128 when the step has many of them),
        one for those with a single token. Otherwise, and always in float32, the plain kernel. Which requests those
        are comes from the step's plan (`attention_plan`)."""
        if not (ctx.fast and ops.attention_mma_supported(q.dtype, self.dh, k_cache.shape[2])):
            ops.attention_plain(q, k_cache, v_cache, ctx.tok_req, ctx.cu_q, ctx.ctx_len, table, out,
                                self.H, self.window, self.scale)
            return
        plan = ctx.plans.get(PLAN_KEY)
        if plan is None:                                 # a step put together without asking the parts: plan it now
            plan = attention_plan(ctx.q_lens, ctx.ctx_lens)
            plan.arrays = {k: torch.from_numpy(v).to(ctx.device) for k, v in plan.arrays.items()}
            ctx.plans[PLAN_KEY] = plan
        tiles64, tiles128, singles = plan.arrays["tiles64"], plan.arrays["tiles128"], plan.arrays["singles"]
        if tiles64.shape[0]:
            if tiles128.shape[0] and ops.attention_prefill_tc_supported(q.dtype, self.dh, k_cache.shape[2]):
                ops.attention_prefill_tc(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, tiles128, out,
                                         self.H, self.window, self.scale)
            else:
                ops.attention_prefill(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, tiles64, out,
                                      self.H, self.window, self.scale)
        n = singles.shape[0]
        if n:
            # as many slices of the keys as fill the device once (the kernel knows how many of its blocks fit)
            longest = plan.host["longest_single"]
            if self.window > 0:
                longest = min(longest, self.window + 64)
            G = self.H // self.KV
            if ops.attention_decode_tma_supported(q.dtype, self.dh, k_cache.shape[2]):
                # head sizes 64 and 128: the TMA-fed kernel, which knows how many slices pay for this many requests
                n_splits = ops.attention_decode_tma_splits(n, self.KV, G, self.dh, longest)
                ops.attention_decode_tma(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, singles, n_splits, out,
                                         self.H, self.window, self.scale)
                return
            groups = self.KV * (-(-G // 16))
            resident = ops.attention_decode_resident_blocks(self.dh)
            n_splits = max(1, min(-(-longest // 64), resident // (n * groups), DECODE_MAX_SPLITS))
            ops.attention_decode(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, singles, n_splits, out,
                                 self.H, self.window, self.scale)
