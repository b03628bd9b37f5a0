"""Typed Python front of the kernel library: every function takes torch CUDA tensors, checks what
the C side cannot see (devices, dtypes, shapes, contiguity) and launches on torch's current stream.
Nothing here computes on the CPU or through a library model: without the built library and an
sm_100a device these functions raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import library

F32, BF16 = 0, 1
EPI_NONE, EPI_BIAS, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
PAIRS_HALVES, PAIRS_INTERLEAVED = 0, 1

_checked_device = False


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported tensor dtype {t.dtype}: kernels take float32 or bfloat16")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """torch's current stream as a pointer. The two C entry points cost a fraction of a microsecond; a step of
    the engine asks hundreds of times, and `torch.cuda.current_stream()` builds a Python object each time."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_ready = None             # the library, once the device has been checked


def _lib():
    global _checked_device, _ready
    if _ready is not None:
        return _ready
    lib = library.load()
    if not _checked_device:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine runs on an sm_100a GPU only (there is no CPU path)")
        if lib.bl_device_check() != 0:
            raise KernelError(lib.bl_last_error().decode())
        _checked_device = True
    _ready = lib
    return lib


launch_count = 0          # kernels launched through this module since import (the benchmark reads it)


_trace = None             # a StepTrace while one is recording


def _call(fn, *args):
    global launch_count
    launch_count += 1
    if fn(*args) != 0:
        raise KernelError(library.load().bl_last_error().decode())
    if _trace is not None and fn.__name__ != "bl_stamp":
        _trace.after(fn.__name__)


class StepTrace:
    """Time line of the kernels launched while it records: a time stamp kernel goes between every two of them
    (also inside a CUDA graph that is being captured), and `durations()` turns the stamps of the last run or
    replay into (kernel, microseconds) pairs. Stamps serialise the kernels, so overlap between neighbours
    (programmatic dependent launch) is not in these figures: they are each kernel's own time in place."""

    def __init__(self, device, capacity: int = 4096):
        self.buf = torch.zeros(capacity, dtype=torch.int64, device=device)
        self.names = []

    def __enter__(self):
        global _trace
        _trace = self
        self.names = []
        _call(_lib().bl_stamp, ctypes.c_void_p(self.buf.data_ptr()), 0, _stream())
        return self

    def __exit__(self, *exc):
        global _trace
        _trace = None

    def after(self, name: str) -> None:
        self.names.append(name)
        if len(self.names) < self.buf.numel():
            library.load().bl_stamp(ctypes.c_void_p(self.buf.data_ptr()), len(self.names), _stream())

    def durations(self):
        torch.cuda.synchronize()
        t = self.buf[:len(self.names) + 1].cpu().tolist()
        return [(n, (t[i + 1] - t[i]) / 1000.0) for i, n in enumerate(self.names)]


def _need(t: torch.Tensor, name: str, dtype=None, shape=None):
    if not t.is_cuda:
        raise KernelError(f"{name}: must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name}: must have shape {tuple(shape)}, got {tuple(t.shape)}")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] widened to 32-bit. The caller has checked that ids lie inside the table."""
    T = ids.shape[0]
    V, d = table.shape
    _need(table, "table"); _need(ids, "ids", torch.int32, (T,)); _need(out, "out", torch.float32, (T, d))
    _call(_lib().bl_embed, _p(table), _dt(table), _p(ids), _p(out), T, d, V, _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            row_idx: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[row_idx[r]] if row_idx is given else x[r]) * weight."""
    d = x.shape[1]
    rows = out.shape[0]
    _need(x, "x", torch.float32); _need(weight, "weight", None, (d,)); _need(out, "out", None, (rows, d))
    if row_idx is not None:
        _need(row_idx, "row_idx", torch.int32, (rows,))
    elif x.shape[0] != rows:
        raise KernelError("rmsnorm: x and out differ in rows")
    _call(_lib().bl_rmsnorm, _p(x), _p(row_idx), _p(weight), _dt(weight), _p(out), _dt(out),
          rows, d, ctypes.c_float(eps), _stream())


def add_row_vector(x: torch.Tensor, v: torch.Tensor) -> None:
    """x[r] += v for every row of the 32-bit residual stream."""
    rows, d = x.shape
    _need(x, "x", torch.float32); _need(v, "v", None, (d,))
    _call(_lib().bl_add_row_vector, _p(x), _p(v), _dt(v), rows, d, _stream())


def gemm_plain(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
               epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T) on CUDA cores with 32-bit accumulation."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x"); _need(w, "w", None, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_plain, _p(x), _dt(x), _p(w), _dt(w), _p(bias), _dt(bias) if bias is not None else 0,
          _p(out), _dt(out), M, N, K, epilogue, _stream())


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                  block_table: torch.Tensor, inv_freq: torch.Tensor, rot_half: int, mscale: float,
                  q_out: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  H: int, KV: int, dh: int, pair_layout: int = 0) -> None:
    """Rotates q and k of joined [q | k | v] rows and writes k, v into the request's pages. `pair_layout`: which
    dimensions turn together, PAIRS_HALVES (j, j + rot_half) or PAIRS_INTERLEAVED (2j, 2j + 1)."""
    T = qkv.shape[0]
    _need(qkv, "qkv", torch.float32, (T, (H + 2 * KV) * dh))
    _need(positions, "positions", torch.int32, (T,)); _need(tok_req, "tok_req", torch.int32, (T,))
    _need(block_table, "block_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32, (dh // 2,))
    _need(q_out, "q_out", None, (T, H * dh))
    page_size = 1
    if k_cache is not None:
        _need(k_cache, "k_cache", q_out.dtype); _need(v_cache, "v_cache", q_out.dtype, k_cache.shape)
        if k_cache.shape[1] != KV or k_cache.shape[3] != dh:
            raise KernelError(f"k_cache: shape {tuple(k_cache.shape)} does not hold {KV} heads of {dh}")
        page_size = k_cache.shape[2]
    _call(_lib().bl_rope_kv_write, _p(qkv), _p(positions), _p(tok_req), _p(block_table),
          block_table.shape[1], _p(inv_freq), rot_half, ctypes.c_float(mscale), _p(q_out), _p(k_cache),
          _p(v_cache), _dt(q_out), T, H, KV, dh, page_size, pair_layout, _stream())


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, rot_half: int, mscale: float):
    """(cos, sin) of every token's rotation, float32 [T, rot_half] each, scaled by `mscale`: worked out once per step
    for the kernels that take the rotation from a table."""
    T = positions.shape[0]
    _need(positions, "positions", torch.int32, (T,)); _need(inv_freq, "inv_freq", torch.float32)
    both = torch.empty((2, T, rot_half), dtype=torch.float32, device=positions.device)
    _call(_lib().bl_rope_table, _p(positions), _p(inv_freq), rot_half, ctypes.c_float(mscale), _p(both[0]), _p(both[1]), T, _stream())
    return both[0], both[1]


def qkv_rope_tc_supported(x: torch.Tensor, w: torch.Tensor, H: int, KV: int, dh: int, page_size: int) -> bool:
    """Whether `qkv_rope_tc` takes this layer's joined product: bfloat16 operands, 16-byte aligned, head size 64 or
    128 with every pair of a head rotated, pages of 16."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(library.load().bl_gemm_tc_pair_qkv_rope_supported(H, KV, dh, page_size, x.shape[1])))


def qkv_rope_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                tok_req: torch.Tensor, block_table: torch.Tensor, cs: torch.Tensor, sn: torch.Tensor, q_out: torch.Tensor,
                k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], H: int, KV: int, dh: int,
                row_sums: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """The joined q/k/v product of many rows on pairs of SMs (tcgen05) with bias, rotation (pairs j, j + dh / 2, from
    the step's table `rope_table`) and the writes of q and of k and v into the requests' pages in its epilogue.
    `row_sums` (with `eps`): x holds rows whose RMS norm is pending (`gemm_residual_norm`); the product's rows are
    scaled by 1 / sqrt(row_sums[m].sum() / K + eps) before the bias."""
    M, K = x.shape
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, ((H + 2 * KV) * dh, K))
    _need(positions, "positions", torch.int32, (M,)); _need(tok_req, "tok_req", torch.int32, (M,))
    _need(block_table, "block_table", torch.int32)
    _need(cs, "cs", torch.float32, (M, dh // 2)); _need(sn, "sn", torch.float32, (M, dh // 2))
    _need(q_out, "q_out", torch.bfloat16, (M, H * dh))
    if bias is not None:
        _need(bias, "bias", None, ((H + 2 * KV) * dh,))
    page_size = 16
    if k_cache is not None:
        _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
        if k_cache.shape[1] != KV or k_cache.shape[3] != dh:
            raise KernelError(f"k_cache: shape {tuple(k_cache.shape)} does not hold {KV} heads of {dh}")
        page_size = k_cache.shape[2]
    _call(_lib().bl_gemm_tc_pair_qkv_rope, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, M, K, _p(tok_req),
          _p(positions), _p(block_table), block_table.shape[1], _p(cs), _p(sn), _p(q_out), _p(k_cache), _p(v_cache),
          H, KV, dh, page_size, _p(row_sums), 0 if row_sums is None else row_sums.shape[1], ctypes.c_float(1.0 / K),
          ctypes.c_float(eps), _stream())


def attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tok_req: torch.Tensor,
                    cu_q: torch.Tensor, ctx_len: torch.Tensor, block_table: torch.Tensor,
                    out: torch.Tensor, H: int, window: int, scale: float) -> None:
    """Paged causal grouped-query attention, one warp per (token, head)."""
    T = q.shape[0]
    _, KV, page_size, dh = k_cache.shape
    _need(q, "q", k_cache.dtype, (T, H * dh)); _need(k_cache, "k_cache"); _need(v_cache, "v_cache", k_cache.dtype, k_cache.shape)
    _need(tok_req, "tok_req", torch.int32, (T,)); _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32)
    _need(block_table, "block_table", torch.int32); _need(out, "out", q.dtype, (T, H * dh))
    _call(_lib().bl_attention_plain, _p(q), _p(k_cache), _p(v_cache), _dt(q), _p(tok_req), _p(cu_q),
          _p(ctx_len), _p(block_table), block_table.shape[1], _p(out), T, H, KV, dh, page_size, window,
          ctypes.c_float(scale), _stream())


def argmax(logits: torch.Tensor, out_ids: torch.Tensor) -> None:
    rows, V = logits.shape
    _need(logits, "logits", torch.float32); _need(out_ids, "out_ids", torch.int32, (rows,))
    _call(_lib().bl_argmax, _p(logits), _p(out_ids), rows, V, _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, out_ids: torch.Tensor) -> None:
    """One token per row: greedy where temperature <= 0, else temperature sampling after the top-k,
    top-p and min-p cuts, with the row's uniform random number."""
    rows, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(temperature, "temperature", torch.float32, (rows,)); _need(top_k, "top_k", torch.int32, (rows,))
    _need(top_p, "top_p", torch.float32, (rows,)); _need(min_p, "min_p", torch.float32, (rows,))
    _need(uniform, "uniform", torch.float32, (rows,)); _need(out_ids, "out_ids", torch.int32, (rows,))
    _call(_lib().bl_sample, _p(logits), rows, V, _p(temperature), _p(top_k), _p(top_p), _p(min_p),
          _p(uniform), _p(out_ids), _stream())


def repeat_penalty(logits: torch.Tensor, tokens: torch.Tensor, offsets: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: logits[r, t] /= penalty[r] if positive else *= penalty[r], for the listed tokens of row r."""
    rows, V = logits.shape
    _need(logits, "logits", torch.float32); _need(tokens, "tokens", torch.int32)
    _need(offsets, "offsets", torch.int32, (rows + 1,)); _need(penalty, "penalty", torch.float32, (rows,))
    _call(_lib().bl_repeat_penalty, _p(logits), rows, V, _p(tokens), _p(offsets), _p(penalty), _stream())


def gemm_skinny_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T) for few rows: W streams once from HBM into tensor-core registers."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_skinny, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _stream())


def attention_mma_supported(dtype: torch.dtype, dh: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(library.load().bl_attention_mma_supported(dh, page_size))


def attention_prefill(q, k_cache, v_cache, cu_q, ctx_len, block_table, tiles, out, H: int, window: int,
                      scale: float) -> None:
    """Tensor-core attention for requests with several new tokens. tiles: int32 [n, 2] = (request, first token
    of a 64-token tile among the request's new tokens)."""
    T = q.shape[0]
    _, KV, page_size, dh = k_cache.shape
    _need(q, "q", torch.bfloat16, (T, H * dh)); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape); _need(out, "out", torch.bfloat16, (T, H * dh))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(tiles, "tiles", torch.int32)
    _call(_lib().bl_attention_prefill, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(tiles), tiles.shape[0], _p(out), H, KV, dh, page_size, window,
          ctypes.c_float(scale), _stream())


def attention_prefill_tc_supported(dtype: torch.dtype, dh: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(library.load().bl_attention_prefill_tc_supported(dh, page_size))


def attention_prefill_tc(q, k_cache, v_cache, cu_q, ctx_len, block_table, tiles, out, H: int, window: int,
                         scale: float) -> None:
    """The tcgen05 form of `attention_prefill` (head size 64, pages of 16). tiles: int32 [n, 2] = (request,
    first token of a tile of 128 among the request's new tokens); the last entries are launched first."""
    T = q.shape[0]
    n_pages, KV, page_size, dh = k_cache.shape
    _need(q, "q", torch.bfloat16, (T, H * dh)); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape); _need(out, "out", torch.bfloat16, (T, H * dh))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(tiles, "tiles", torch.int32, (tiles.shape[0], 2))
    _call(_lib().bl_attention_prefill_tc, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(tiles), tiles.shape[0], _p(out), T, n_pages, H, KV, dh, page_size, window,
          ctypes.c_float(scale), _stream())


DECODE_CLUSTER_SPLITS = 16     # up to this many slices merge through distributed shared memory (one cluster a request and head group)


def attention_decode(q, k_cache, v_cache, cu_q, ctx_len, block_table, reqs, n_splits: int, out, H: int, window: int,
                     scale: float, scratch: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention for requests with one new token; `reqs` int32 [n] lists them. The keys of each are
    cut into `n_splits` slices. Up to `DECODE_CLUSTER_SPLITS` slices without `scratch`: the slices of a request are
    the blocks of a cluster and merge in shared memory. More slices, or a `scratch` tensor (float32,
    `attention_decode_scratch(...)` elements): the partial results go through scratch and the last block merges."""
    T = q.shape[0]
    _, KV, page_size, dh = k_cache.shape
    n = reqs.shape[0]
    _need(q, "q", torch.bfloat16, (T, H * dh)); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape); _need(out, "out", torch.bfloat16, (T, H * dh))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(reqs, "reqs", torch.int32, (n,))
    need = attention_decode_scratch(n, H, dh, n_splits)
    if scratch is None and n_splits <= DECODE_CLUSTER_SPLITS:
        need = 0                               # the slices of a request form a cluster and merge in shared memory: no scratch
    if need:
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError(f"scratch: {scratch.numel()} floats, {need} needed")
    counters = None
    if need:
        n_counters = n * KV * (-(-(H // KV) // 16))
        counters = _decode_counters.get(q.device)
        if counters is None or counters.numel() < n_counters:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("attention_decode: its counters must exist before a capture (run the step once first)")
            # zero once; every launch leaves them at zero again
            counters = _decode_counters[q.device] = torch.zeros(max(n_counters, 4096), dtype=torch.int32, device=q.device)
    _call(_lib().bl_attention_decode, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(reqs), n, n_splits, _p(scratch if need else None), _p(counters), _p(out), H, KV, dh,
          page_size, window, ctypes.c_float(scale), _stream())


def attention_decode_tma_supported(dtype: torch.dtype, dh: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(library.load().bl_attention_decode_tma_supported(dh, page_size))


def attention_decode_tma(q, k_cache, v_cache, cu_q, ctx_len, block_table, reqs, n_splits: int, out, H: int, window: int,
                         scale: float) -> None:
    """`attention_decode` for head sizes 64 and 128 with keys and values streamed by TMA into per-warp rings and the
    query heads of a key/value head as the columns of the MMAs; 1 to `DECODE_CLUSTER_SPLITS` slices, which are the
    blocks of one cluster and send their partial rows to the blocks that finish them."""
    T = q.shape[0]
    n_pages, KV, page_size, dh = k_cache.shape
    n = reqs.shape[0]
    _need(q, "q", torch.bfloat16, (T, H * dh)); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape); _need(out, "out", torch.bfloat16, (T, H * dh))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(reqs, "reqs", torch.int32, (n,))
    # Large clusters of a launch with more blocks than SMs start only when the kernel before has finished: placed while
    # its blocks still hold SMs they pile up two to an SM beside empty SMs (measured at batch 8: 54 -> 44 us a layer at
    # 32,000 tokens, 81 -> 62 at 64,000; small launches gain 2.5 us a layer from the early start)
    G = H // KV
    blocks = n * KV * (-(-G // (8 if G <= 8 else 16))) * n_splits
    early = not (n_splits >= DECODE_TMA_LATE_CLUSTER and blocks > _sms())
    _call(_lib().bl_attention_decode_tma, _p(q), _p(k_cache), _p(v_cache), n_pages, _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(reqs), n, n_splits, _p(out), H, KV, dh, page_size, window, ctypes.c_float(scale),
          1 if early else 0, _stream())


def attention_decode_tma_resident_blocks(dh: int, heads_per_kv: int) -> int:
    """Blocks of `attention_decode_tma` that the device holds at once (the kernel's own occupancy, asked once)."""
    key = (torch.cuda.current_device(), dh, heads_per_kv > 8)
    if key not in _decode_tma_resident:
        _decode_tma_resident[key] = max(1, int(_lib().bl_attention_decode_tma_resident_blocks(dh, heads_per_kv)))
    return _decode_tma_resident[key]


_decode_tma_resident = {}
_decode_tma_clusters = {}
_sm_count = {}
DECODE_TMA_LATE_CLUSTER = 8           # clusters from this size on, in launches of more blocks than SMs, are launched late


def _sms() -> int:
    dev = torch.cuda.current_device()
    if dev not in _sm_count:
        _sm_count[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_count[dev]

DECODE_TMA_UNIT = 32                  # keys a warp of `attention_decode_tma` takes at a time
DECODE_TMA_MIN_UNITS = 4              # a slice is worth a block from four units on (one for each warp)
DECODE_TMA_FEW_UNITS = 12             # up to this many units a warp, one block an SM is best: it may start under its predecessor (measured inside a layer's chain of kernels: 8 requests of 8,000 tokens 27.1 us a layer against 29.5, of 16,000 33.0 against 34.7; 32 requests of 3,900 want four slices)


def attention_decode_tma_splits(n: int, KV: int, heads_per_kv: int, dh: int, longest: int) -> int:
    """Slices for `attention_decode_tma` with n requests whose longest context (or window) has `longest` keys.
    Measured on a B200: a launch should run in one round (more clusters than the device holds at once cost a second
    round), slices below 128 keys cost more than they save, and while a warp has only a few units to walk, one block
    per SM beats two (the step is a chain of latencies); with long walks two blocks per SM keep more bytes in
    flight. Among the slice counts that qualify, the smallest that gives a warp the fewest units."""
    dev = torch.cuda.current_device()
    sms = _sms()
    groups = KV * (-(-heads_per_kv // (8 if heads_per_kv <= 8 else 16)))
    clusters = n * groups
    units = -(-max(1, longest) // DECODE_TMA_UNIT)
    most = max(1, min(DECODE_CLUSTER_SPLITS, units // DECODE_TMA_MIN_UNITS))

    def per_warp(s):
        return -(-(-(-units // s)) // 4)

    def fits(s):
        key = (dev, dh, heads_per_kv > 8)
        if key not in _decode_tma_clusters:                # asked once, for every cluster size (never inside a later capture)
            _decode_tma_clusters[key] = [0] + [int(_lib().bl_attention_decode_tma_max_clusters(dh, heads_per_kv, c))
                                               for c in range(1, DECODE_CLUSTER_SPLITS + 1)]
        return clusters <= _decode_tma_clusters[key][s]

    one_per_sm = max(1, min(most, sms // clusters))
    if per_warp(one_per_sm) <= DECODE_TMA_FEW_UNITS:
        top = one_per_sm
    else:
        top = next((s for s in range(most, 0, -1) if fits(s)), 1)
    return min(range(1, top + 1), key=lambda s: (per_warp(s), s))
_decode_counters = {}
_decode_resident = {}


def attention_decode_resident_blocks(dh: int) -> int:
    """Blocks of `attention_decode` that the device holds at once for this head size (asked of the kernel's own
    occupancy on the current device, once per head size)."""
    key = (torch.cuda.current_device(), dh)
    if key not in _decode_resident:
        _decode_resident[key] = max(1, int(_lib().bl_attention_decode_resident_blocks(dh)))
    return _decode_resident[key]


def attention_decode_scratch(n: int, H: int, dh: int, n_splits: int) -> int:
    return 0 if n_splits <= 1 else n * H * n_splits * (dh + 2)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T) for many rows: tcgen05 tensor cores, TMA-fed tiles, accumulator in tensor memory.
    Same operand rules as `gemm_skinny` (`gemm_skinny_supported`)."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_tc, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _stream())


def gemm_tc_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 epilogue: int = EPI_NONE) -> None:
    """`gemm_tc` on pairs of SMs (tcgen05 cta_group::2): 256 x 256 tiles, for a few hundred rows and more."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_tc_pair, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _stream())


def gemm_tc_splitk(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   epilogue: int = EPI_NONE) -> None:
    """`gemm_tc` for shapes with few output tiles: clusters of up to eight blocks share a tile and cut K among them,
    their partial tiles added in block order through distributed shared memory."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_tc_splitk, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _stream())


_splitk_split = {}


def gemm_tc_splitk_split(M: int, N: int, K: int, epilogue: int) -> int:
    """Blocks that would share a tile of this product in `gemm_tc_splitk` (1: it has nothing over `gemm_tc`)."""
    key = (-(-M // 128), N, K, epilogue == EPI_SWIGLU)
    if key not in _splitk_split:
        _splitk_split[key] = int(_lib().bl_gemm_tc_splitk_split(M, N, K, epilogue))
    return _splitk_split[key]


def gemm_tc_cols_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `gemm_tc_cols` takes these operands: bfloat16, up to 64 rows, 16-byte aligned, x fits shared memory."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(library.load().bl_gemm_tc_cols_supported(x.shape[0], w.shape[0], x.shape[1])))


def gemm_tc_cols(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = x @ w.T for few rows and very many columns (an output head): the tcgen05 kernel that streams W once
    through a deep TMA ring with W as the M side of the product."""
    M, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16, (M, K)); _need(w, "w", torch.bfloat16, (N, K)); _need(out, "out", None, (M, N))
    _call(_lib().bl_gemm_tc_cols, _p(x), _p(w), _p(out), _dt(out), M, N, K, _stream())


# Which matrix-product kernel takes a bfloat16 product of M rows by N columns. The thresholds were measured on a
# B200 (148 SMs) and live here, beside the kernels they choose between, not in the parts that call them.
SKINNY_MAX_ROWS = 64                  # up to here W streams through registers (faster than 128-row tcgen05 tiles at 64 rows)
TC_MIN_COLUMNS_FEW_ROWS = 4096        # 17..64 rows: wide products have enough 128-column tiles for TMA to stream W at full rate
TC_MIN_COLUMNS_VERY_FEW_ROWS = 32768  # an output head: up to 64 rows take the kernel made for it; without it 128-row tiles win from 9 rows
PAIR_MIN_ROWS = 256                   # from here on pairs of SMs share 256 x 256 tiles (tcgen05 cta_group::2)
SPLITK_MIN_ROWS, SPLITK_MAX_ROWS = 32, 640   # products with few tiles in this range of rows are cut along K over clusters ...
SPLITK_VERY_LONG_K = 16384            # ... or, below 32 rows, very long (K 18,944 by N 3,584 at 8 rows: 43 us against 72 us through registers)
STREAM_MIN_BYTES = 128 << 20          # matrices from this size on stream faster through TMA and tcgen05 than through registers, at any number of rows
SPLITK_LONG_K = 2048                  # ... when K is long (measured: K 4,864 by N 896 gains 2x at 128 rows, 1.25x at 512; K 896 gains only up to 128 rows)


def gemm_streams_better(w: torch.Tensor) -> bool:
    """Whether a matrix is so large that few rows of x are better served by the TMA-fed tcgen05 kernels than by the
    kernels that stream W through registers (measured on 272 MB at 8 rows: 4.3 TB/s against 2.6 TB/s)."""
    return w.numel() * w.element_size() >= STREAM_MIN_BYTES


def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
         epilogue: int = EPI_NONE, fast: bool = True) -> None:
    """out = epilogue(x @ w.T) by the kernel that suits the operands: float32 operands, operands the tensor-core
    kernels cannot take, and `fast=False` run the plain CUDA-core kernel; bfloat16 operands a tensor-core kernel
    chosen by the number of rows (and, for few rows, of columns)."""
    kind = gemm_kernel(x, w, out.shape[1], bias, epilogue, fast)
    if kind == "plain":
        gemm_plain(x, w, out, bias, epilogue)
    elif kind == "cols":
        gemm_tc_cols(x, w, out)
    elif kind == "splitk":
        gemm_tc_splitk(x, w, out, bias, epilogue)
    elif kind == "skinny":
        gemm_skinny(x, w, out, bias, epilogue)
    elif kind == "tc":
        gemm_tc(x, w, out, bias, epilogue)
    else:
        gemm_tc_pair(x, w, out, bias, epilogue)


def gemm_kernel(x: torch.Tensor, w: torch.Tensor, N: int, bias: Optional[torch.Tensor], epilogue: int, fast: bool = True) -> str:
    """Which kernel `gemm` runs this product on: "plain", "cols" (an output head at decode time: W streams once, as the
    M side of the product), "splitk" (few tiles and a long K, a down projection: clusters cut K among their blocks),
    "skinny" (few rows: W streams through registers), "tc" or "pair" (tcgen05 tiles on one SM, on pairs of SMs)."""
    if not (fast and gemm_skinny_supported(x, w)):
        return "plain"
    M, K = x.shape
    few_rows_tc = ((M > 16 and N >= TC_MIN_COLUMNS_FEW_ROWS) or (M > 8 and N >= TC_MIN_COLUMNS_VERY_FEW_ROWS)
                   or gemm_streams_better(w))
    if (N >= TC_MIN_COLUMNS_VERY_FEW_ROWS and bias is None and epilogue == EPI_NONE and M <= 64
            and gemm_tc_cols_supported(x, w)):
        return "cols"
    if (epilogue != EPI_SWIGLU and M <= SPLITK_MAX_ROWS and (M >= SPLITK_MIN_ROWS or K >= SPLITK_VERY_LONG_K)
            and (K >= SPLITK_LONG_K or 64 < M <= 128) and gemm_tc_splitk_split(M, N, K, epilogue) >= 2):
        return "splitk"
    if M <= SKINNY_MAX_ROWS and not few_rows_tc:
        return "skinny"
    return "tc" if M < PAIR_MIN_ROWS else "pair"


def gemm_on_pairs(x: torch.Tensor, w: torch.Tensor, N: int, epilogue: int, fast: bool = True) -> bool:
    """Whether `gemm` would run this product on pairs of SMs (`gemm_tc_pair`): the kernel whose epilogues can leave an
    RMS norm pending (`gemm_residual_norm`) and apply a pending one (`gemm_swiglu_scaled`, `qkv_rope_tc`)."""
    return gemm_kernel(x, w, N, None, epilogue, fast) == "pair"


SKINNY_LINK_MIN_ROWS = 2       # steps of this many rows ...
SKINNY_LINK_MAX_ROWS = 16      # ... to this many share a norm between two register-streaming products (measured at the 0.5B
                               # sizes: a decode step 2 % faster at 2 rows, 6 % at 4, 4 % at 8, 1 % at 16; 2 % slower at 1 row)
SKINNY_LINK_MAX_BLOCKS = 592   # column blocks of 16 up to which the linked kernel keeps two batches of loads in flight (with more it
                               # runs its lighter form, and the fused norm + product kernel is the faster: 3B sizes, 688 blocks, +5 %)


def gemm_skinny_links_norm(x: torch.Tensor, w: torch.Tensor, N: int, epilogue: int, fast: bool = True) -> bool:
    """Whether `gemm` would run this product on the register-streaming kernel at a row count where that kernel's
    epilogues begin an RMS norm (`gemm_skinny_residual_norm`) and finish one (`gemm_skinny_scaled`)."""
    return (SKINNY_LINK_MIN_ROWS <= x.shape[0] <= SKINNY_LINK_MAX_ROWS and -(-N // 16) <= SKINNY_LINK_MAX_BLOCKS
            and gemm_kernel(x, w, N, None, epilogue, fast) == "skinny")


def gemm_skinny_residual_norm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, norm_w: torch.Tensor):
    """out += x @ w.T (32-bit residual stream, in place) on the register-streaming kernel, and, for the RMS norm with
    weight `norm_w` that reads `out` next, (hw, ss): hw = bfloat16(out * norm_w), ss[m, :] = sums of squares of row m
    by block of 16 columns (what `gemm_residual_norm` gives on pairs of SMs, for decode steps)."""
    M, K = x.shape
    N = out.shape[1]
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (N, K)); _need(out, "out", torch.float32, (M, N))
    _need(norm_w, "norm_w", None, (N,))
    parts = int(_lib().bl_gemm_skinny_norm_parts(N))
    hw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ss = torch.empty((M, parts), dtype=torch.float32, device=x.device)
    _call(_lib().bl_gemm_skinny_residual_norm, _p(x), _p(w), _p(out), M, N, K, _p(norm_w), _dt(norm_w), _p(hw), _p(ss), _stream())
    return hw, ss


def gemm_skinny_scaled(hw: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ss: torch.Tensor, eps: float,
                       bias: Optional[torch.Tensor] = None, epilogue: int = EPI_NONE) -> None:
    """out = epilogue(r * (hw @ w.T)), r[m] = 1 / sqrt(ss[m].sum() / K + eps): the product of rows whose RMS norm
    `gemm_skinny_residual_norm` (or `gemm_residual_norm`) left pending. Epilogues: none, bias, SwiGLU."""
    M, K = hw.shape
    N = out.shape[1]
    _need(hw, "hw", torch.bfloat16); _need(w, "w", torch.bfloat16, ((2 * N if epilogue == EPI_SWIGLU else N), K))
    _need(out, "out", None, (M, N)); _need(ss, "ss", torch.float32)
    if ss.shape[0] != M:
        raise KernelError("gemm_skinny_scaled: ss and hw differ in rows")
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_skinny_scaled, _p(hw), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _p(ss), ss.shape[1], ctypes.c_float(eps), _stream())


def gemm_residual_norm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, norm_w: torch.Tensor):
    """out += x @ w.T (32-bit residual stream, in place) on pairs of SMs, and, for the RMS norm with weight `norm_w`
    that reads `out` next, (hw, ss): hw = bfloat16(out * norm_w) and ss[m, :] = sums of squares of row m's columns by
    tile. A product that takes hw as its x and scales its rows by 1 / sqrt(ss[m].sum() / N + eps) computes what it would
    from the normed rows (`gemm_swiglu_scaled`, `qkv_rope_tc` with `row_sums`)."""
    M, K = x.shape
    N = out.shape[1]
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (N, K)); _need(out, "out", torch.float32, (M, N))
    _need(norm_w, "norm_w", None, (N,))
    parts = int(_lib().bl_gemm_tc_pair_norm_parts(M, N))
    hw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ss = torch.empty((M, parts), dtype=torch.float32, device=x.device)
    _call(_lib().bl_gemm_tc_pair_residual_norm, _p(x), _p(w), _p(out), M, N, K, _p(norm_w), _dt(norm_w), _p(hw), _p(ss), _stream())
    return hw, ss


def gemm_swiglu_scaled(hw: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ss: torch.Tensor, eps: float) -> None:
    """out = silu(r g) * (r u), g and u the two halves of hw @ w.T, r[m] = 1 / sqrt(ss[m].sum() / K + eps): the SwiGLU
    product of rows whose RMS norm `gemm_residual_norm` left pending."""
    M, K = hw.shape
    N = out.shape[1]
    _need(hw, "hw", torch.bfloat16); _need(w, "w", torch.bfloat16, (2 * N, K)); _need(out, "out", torch.bfloat16, (M, N))
    _need(ss, "ss", torch.float32)
    if ss.shape[0] != M:
        raise KernelError("gemm_swiglu_scaled: ss and hw differ in rows")
    _call(_lib().bl_gemm_tc_pair_swiglu_scaled, _p(hw), _p(w), _p(out), M, N, K, _p(ss), ss.shape[1], ctypes.c_float(1.0 / K),
          ctypes.c_float(eps), _stream())


def check_status() -> None:
    """Raises if a tensor-core block gave up on one of its bounded waits since the last check. Synchronises."""
    for name, fn in (("bl_gemm_tc", _lib().bl_gemm_tc_status), ("bl_gemm_tc_pair", _lib().bl_gemm_tc_pair_status),
                     ("bl_attention_prefill_tc", _lib().bl_attention_prefill_tc_status),
                     ("bl_gemm_tc_cols", _lib().bl_gemm_tc_cols_status),
                     ("bl_gemm_tc_splitk", _lib().bl_gemm_tc_splitk_status),
                     ("bl_attention_decode_tma", _lib().bl_attention_decode_tma_status)):
        v = ctypes.c_int(0)
        _call(fn, ctypes.byref(v))
        if v.value != 0:
            who = {1: "the TMA loader", 2: "the MMA issuer", 3: "the epilogue"}.get(v.value, "a thread")
            raise KernelError(f"{name}: {who} gave up on a bounded wait (code {v.value}); results of that launch are invalid")


def norm_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the fused norm + product kernels take these operands (float32 rows, bfloat16 matrix)."""
    return (x.dtype == torch.float32 and w.dtype == torch.bfloat16 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and bool(library.load().bl_norm_gemm_supported(x.shape[1])))


def norm_gemm(x: torch.Tensor, norm_w: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor,
              bias: Optional[torch.Tensor] = None, epilogue: int = EPI_NONE,
              row_idx: Optional[torch.Tensor] = None) -> None:
    """out = epilogue(rmsnorm(x[row_idx]) @ w.T) in one launch, for few rows. EPI_NONE / EPI_BIAS write float32,
    EPI_SWIGLU (w with twice the rows) writes bfloat16."""
    K = x.shape[1]
    M, N = out.shape
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.float32); _need(norm_w, "norm_w", None, (K,)); _need(w, "w", torch.bfloat16, (rows_w, K))
    _need(out, "out", torch.bfloat16 if epilogue == EPI_SWIGLU else torch.float32)
    if row_idx is not None:
        _need(row_idx, "row_idx", torch.int32, (M,))
    elif x.shape[0] != M:
        raise KernelError("norm_gemm: x and out differ in rows")
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_norm_gemm, _p(x), _p(row_idx), _p(norm_w), _dt(norm_w), ctypes.c_float(eps), _p(w), _p(bias),
          _dt(bias) if bias is not None else 0, _p(out), M, N, K, epilogue, _stream())


def norm_qkv_rope(x: torch.Tensor, norm_w: torch.Tensor, eps: float, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                  positions: torch.Tensor, tok_req: torch.Tensor, block_table: torch.Tensor, inv_freq: torch.Tensor,
                  mscale: float, q_out: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  H: int, KV: int, dh: int, pair_layout: int = 0) -> None:
    """rmsnorm -> joined q/k/v product (+ bias) -> rotation of q and k -> k, v into the pages, q out, in one launch."""
    M, K = x.shape
    _need(x, "x", torch.float32); _need(norm_w, "norm_w", None, (K,)); _need(w_qkv, "w_qkv", torch.bfloat16, ((H + 2 * KV) * dh, K))
    _need(positions, "positions", torch.int32, (M,)); _need(tok_req, "tok_req", torch.int32, (M,))
    _need(block_table, "block_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32, (dh // 2,))
    _need(q_out, "q_out", torch.bfloat16, (M, H * dh))
    if bias is not None:
        _need(bias, "bias", None, ((H + 2 * KV) * dh,))
    page_size = 1
    if k_cache is not None:
        _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
        if k_cache.shape[1] != KV or k_cache.shape[3] != dh:
            raise KernelError(f"k_cache: shape {tuple(k_cache.shape)} does not hold {KV} heads of {dh}")
        page_size = k_cache.shape[2]
    _call(_lib().bl_norm_qkv_rope, _p(x), _p(norm_w), _dt(norm_w), ctypes.c_float(eps), _p(w_qkv), _p(bias),
          _dt(bias) if bias is not None else 0, _p(positions), _p(tok_req), _p(block_table), block_table.shape[1],
          _p(inv_freq), ctypes.c_float(mscale), _p(q_out), _p(k_cache), _p(v_cache), M, K, H, KV, dh, page_size,
          pair_layout, _stream())
