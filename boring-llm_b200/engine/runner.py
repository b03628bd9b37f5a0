"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

The reference has four single-sequence functions in this role: `prefill_gpu_quantized`,
`prefill_step_gpu_quantized` (append n tokens after `cache.pos`, last-row logits),
`forward_batch_gpu_quantized` (same, every row's logits) and `forward_step` (one token)
(src/model.br:1747, 1852, 1935, 2043). Here one function runs any mix of them as one flat batch:
portions of prompts beside single decoded tokens, cut anywhere. It runs only the tokens it is given,
against the cache that earlier steps left, and is free of policy: which tokens to run is the
scheduler's (or the trace's) business.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage
from ..config import EngineOptions
from ..models.loading import torch_dtype
from ..parts import StepContext, StepPlan


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


class OutOfPages(RuntimeError):
    """The step needs more cache pages than are free. Nothing was changed."""


class StepError(ValueError):
    """A step that cannot run: an unknown token id, a request past its context size, ..."""


GRAPH_MAX_BATCH = 64          # decode steps of up to this many requests replay a captured CUDA graph
STEP_GRAPH_MAX_WANTED = 64    # general steps that want more rows of logits than this are launched kernel by kernel
STEP_GRAPH_CACHE = 48         # captured general steps kept (least recently used goes first)


def _fill_batch(f: dict, entries, rcs, q_lens, ctx_lens) -> list:
    """Writes the batch's index arrays into the host views `f` (token_ids, positions, tok_req, cu_q, ctx_len,
    slots, logit_rows, tables [groups, requests, width]); returns the requests' slots. Rows past the batch's own
    are the caller's."""
    t0 = 0
    n_want = 0
    slot_list = []
    token_ids, positions, tok_req, cu_q = f["token_ids"], f["positions"], f["tok_req"], f["cu_q"]
    ctx_len, slots, logit_rows, tables = f["ctx_len"], f["slots"], f["logit_rows"], f["tables"]
    fresh = tables.shape[1] == len(entries)
    if fresh:
        tables[...] = -1
    for r, (e, rc) in enumerate(zip(entries, rcs)):
        n = q_lens[r]
        token_ids[t0:t0 + n] = np.asarray(e.tokens, dtype=np.int32)
        positions[t0:t0 + n] = np.arange(rc.num_tokens, rc.num_tokens + n, dtype=np.int32)
        tok_req[t0:t0 + n] = r
        cu_q[r] = t0
        ctx_len[r] = ctx_lens[r]
        slots[r] = rc.slot
        for w in e.want:
            logit_rows[n_want] = t0 + int(w)
            n_want += 1
        for gi, tab in enumerate(rc.tables):
            tables[gi, r, :len(tab)] = tab
        slot_list.append(rc.slot)
        t0 += n
    cu_q[len(entries)] = t0
    return slot_list


class _StepGraph:
    """A captured general step for one padded shape (tokens, requests, wanted rows, the parts' plan shapes)."""

    def __init__(self, runner: "ModelRunner", T_b: int, R_b: int, N_b: int, plans: dict):
        G = len(runner.cache.paged_groups)
        W = runner._table_width
        plan_items = [((key, name), arr) for key, plan in plans.items() for name, arr in plan.arrays.items()]
        sizes = [("token_ids", T_b), ("positions", T_b), ("tok_req", T_b), ("cu_q", R_b + 1), ("ctx_len", R_b),
                 ("slots", R_b), ("logit_rows", N_b), ("tables", G * R_b * W)]
        sizes += [(k, int(arr.size)) for k, arr in plan_items]
        total = sum(n for _, n in sizes)
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(total, dtype=torch.int32, device=runner.device)
        hn = self.host.numpy()
        self.fields: Dict[object, np.ndarray] = {}
        d: Dict[object, torch.Tensor] = {}
        o = 0
        for name, n in sizes:
            self.fields[name] = hn[o:o + n]
            d[name] = self.dev[o:o + n]
            o += n
        self.fields["tables"] = self.fields["tables"].reshape(G, R_b, W)
        self.plan_host = {k: self.fields[k].reshape(arr.shape) for k, arr in plan_items}
        # until the first batch is written, every row is a padding request on the spare page
        f = self.fields
        f["tok_req"][:] = 0
        f["ctx_len"][:] = 1
        f["slots"][:] = runner.storage.trash_slot
        f["tables"][...] = -1
        f["tables"][:, :, 0] = runner.storage.trash_page
        f["cu_q"][:] = 0
        f["cu_q"][1:] = T_b
        for (k, name), dst in self.plan_host.items():
            dst[...] = plans[k].arrays[name]
        self.dev.copy_(self.host)
        self.ctx = StepContext(
            dtype=runner.dtype, device=runner.device, T=T_b, R=R_b, token_ids=d["token_ids"], positions=d["positions"],
            tok_req=d["tok_req"], cu_q=d["cu_q"], ctx_len=d["ctx_len"], slots=d["slots"], logit_rows=d["logit_rows"],
            block_tables=[d["tables"][g * R_b * W:(g + 1) * R_b * W].view(R_b, W) for g in range(G)],
            q_lens=[], ctx_lens=[], slot_list=[], storage=runner.storage, fast=True,
            plans=_plans_on_device(plans, {k: d[k].view(arr.shape) for k, arr in plan_items}))
        self.copied = torch.cuda.Event()
        self.graph = None
        self.logits = None
        self.kernels = 0

    def capture(self, runner: "ModelRunner") -> None:
        """Captures the step. The same kernels have just run once through this context outside a capture, so whatever
        they set up at their first launch is done."""
        from ..kernels import ops
        torch.cuda.synchronize()
        before = ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=runner._step_graph_pool()):
            self.logits = runner.model.forward(self.ctx)
        self.kernels = ops.launch_count - before


class PendingDecode:
    """A decode step that has been launched and whose sampled tokens have not been read yet."""
    __slots__ = ("graph", "buffer", "rows")

    def __init__(self, graph: "_DecodeGraph", buffer: int, rows: List[int]):
        self.graph, self.buffer, self.rows = graph, buffer, rows


def _plans_on_device(plans: dict, views: dict) -> dict:
    """The parts' plans with their host arrays replaced by the device views that hold them."""
    return {key: StepPlan(arrays={name: views[(key, name)] for name in plan.arrays}, host=dict(plan.host), shape=plan.shape)
            for key, plan in plans.items()}


class _DecodeRows:
    """What the captured decode steps of one row count share: the rows' sampled tokens on the device (a step may take
    its input tokens from them) and the two pinned buffers that bring them to the host."""

    def __init__(self, rows: int, device):
        self.sampled = torch.zeros(rows, dtype=torch.int32, device=device)
        # two steps may be in flight (the next is launched before this one's tokens are read): two buffers take turns
        self.sampled_host = [torch.zeros(rows, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.sampled_ready = [torch.cuda.Event() for _ in range(2)]
        self.next_buffer = 0
        self.last_live = 0                             # live rows of the last replay (whose tokens `sampled` holds)


class _DecodeGraph:
    """A captured decode step for a fixed number of rows and an upper bound of their contexts. All per-step inputs
    live in one int32 device buffer that a single copy refreshes before each replay; rows beyond the live requests
    point at the storage's spare page and slot."""

    def __init__(self, runner: "ModelRunner", rows: int, ctx_bound: int, shared: _DecodeRows):
        self.rows, self.shared = rows, shared
        G = len(runner.cache.paged_groups)
        W = runner._table_width
        B = rows
        collect = getattr(runner.model, "collect_plans", None)
        plans = collect([1] * B, [ctx_bound] * B, None) if collect is not None else {}
        sizes = [("token_ids", B), ("positions", B), ("ctx_len", B), ("slots", B),
                 ("temperature", B), ("top_k", B), ("top_p", B), ("min_p", B), ("uniform", B),
                 ("tables", G * B * W),
                 ("tok_req", B), ("cu_q", B + 1), ("logit_rows", B)]
        sizes += [((key, name), int(arr.size)) for key, plan in plans.items() for name, arr in plan.arrays.items()]
        total = sum(n for _, n in sizes)
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(total, dtype=torch.int32, device=runner.device)
        self.h: Dict[object, np.ndarray] = {}
        self.d: Dict[object, torch.Tensor] = {}
        o = 0
        hn = self.host.numpy()
        for name, n in sizes:
            self.h[name] = hn[o:o + n]
            self.d[name] = self.dev[o:o + n]
            o += n
        self.dynamic_ints = 9 * B + G * B * W          # the leading fields change every step
        self.small_ints = 9 * B                        # ... and the tables only when a request gets a new page
        self.h["tables"] = self.h["tables"].reshape(G, B, W)
        for name in ("temperature", "top_p", "min_p", "uniform"):      # 32-bit floats in the same buffer
            self.h[name] = self.h[name].view(np.float32)
            self.d[name] = self.d[name].view(torch.float32)
        self.h["top_p"][:] = 1.0
        self.row_owner = [None] * B                    # (request uid, table version) whose table a row holds
        self.tables_dirty = True
        ar = np.arange(B, dtype=np.int32)
        self.h["tok_req"][:] = ar; self.h["logit_rows"][:] = ar
        self.h["cu_q"][:] = np.arange(B + 1, dtype=np.int32)
        for key, plan in plans.items():                # the same for every replay: all rows are single tokens
            for name, arr in plan.arrays.items():
                self.h[(key, name)][:] = arr.reshape(-1)
                self.d[(key, name)] = self.d[(key, name)].view(arr.shape)
        self.trash_page, self.trash_slot = runner.storage.trash_page, runner.storage.trash_slot
        self.fill_padding(0)
        self.dev.copy_(self.host)
        self.ctx = StepContext(
            dtype=runner.dtype, device=runner.device, T=B, R=B, token_ids=self.d["token_ids"],
            positions=self.d["positions"], tok_req=self.d["tok_req"], cu_q=self.d["cu_q"], ctx_len=self.d["ctx_len"],
            slots=self.d["slots"], logit_rows=self.d["logit_rows"],
            block_tables=[self.d["tables"][g * B * W:(g + 1) * B * W].view(B, W) for g in range(G)],
            q_lens=[1] * B, ctx_lens=[ctx_bound] * B, slot_list=[runner.storage.trash_slot] * B,
            storage=runner.storage, fast=True, plans=_plans_on_device(plans, self.d))
        # run once outside a capture (first-use set-up inside the kernels), then capture
        side = torch.cuda.Stream(device=runner.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            runner.model.forward(self.ctx)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..kernels import ops
        before = ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = runner.model.forward(self.ctx)
            # one token per row from the step's own logits: greedy rows (temperature 0) cost one pass
            ops.sample(self.logits, self.d["temperature"], self.d["top_k"], self.d["top_p"], self.d["min_p"],
                       self.d["uniform"], shared.sampled)
        self.kernels = ops.launch_count - before       # kernels of this library that one replay launches
        self.copied = torch.cuda.Event()

    def fill_padding(self, live: int) -> None:
        h = self.h
        h["token_ids"][live:] = 0
        h["positions"][live:] = 0
        h["ctx_len"][live:] = 1
        h["slots"][live:] = self.trash_slot
        for r in range(live, self.rows):
            if self.row_owner[r] != "padding":
                h["tables"][:, r, :] = -1
                h["tables"][:, r, 0] = self.trash_page
                self.row_owner[r] = "padding"
                self.tables_dirty = True
        h["temperature"][live:] = 0.0


class ModelRunner:
    def __init__(self, model, options: EngineOptions, vocab_size: Optional[int] = None):
        self.model = model
        self.options = options
        self.device = torch.device(options.device)
        self.dtype = torch_dtype(options.dtype)
        self.vocab_size = vocab_size if vocab_size is not None else model.vocab_size
        self.cache = CacheManager(model.cache_specs(), options.page_size, options.capacity_tokens,
                                  options.max_num_seqs)
        self.storage = CacheStorage(self.cache, self.dtype, self.device)
        self.fast = True            # False: plain kernels only
        self._pinned: List[torch.Tensor] = []
        self._pinned_events: List[Optional[torch.cuda.Event]] = []
        self._pinned_next = 0
        self.steps = 0
        self.tokens_run = 0
        self.graph_steps = 0
        self.last_step_graph_kernels = 0               # kernels launched by the last step through a graph replay
        self.last_h2d_bytes = self.last_d2h_bytes = 0  # bytes the last step copied to and from the device
        self._graphs: Dict[tuple, "_DecodeGraph"] = {}      # (rows, bound of the contexts) -> captured decode step
        self._decode_rows: Dict[int, "_DecodeRows"] = {}
        self._step_graphs: Dict[tuple, "_StepGraph"] = {}    # padded shape -> captured general step, least recently used first
        self._step_shapes_seen: Dict[tuple, int] = {}
        self._graph_pool = None
        self._graph_safe: Optional[bool] = None
        self._waits_unchecked = False                  # a step ran kernels with bounded waits since the last check
        self._table_width = -(-(-(-options.ctx_size // options.page_size)) // 8) * 8

    # ---- requests --------------------------------------------------------------------------------
    def add_request(self, request_id) -> None:
        self.cache.add_request(request_id)

    def free_request(self, request_id) -> None:
        self.cache.free(request_id)

    def has_request(self, request_id) -> bool:
        return request_id in self.cache

    def truncate(self, request_id, n_keep: int) -> None:
        """Keeps the first `n_keep` tokens of a request's cache and gives the pages behind them back; the next step's
        tokens of that request continue at position `n_keep` (the reference truncates by setting the cache's length,
        src/model.br:2313-2314, 2330-2342). Refused for a request whose mixer keeps state that cannot be rolled back
        (anything but pages), or whose window has already given pages of the kept prefix back."""
        if self.cache.state_groups:
            raise StepError(f"request {request_id!r}: state of fixed size cannot be truncated; recompute from the start")
        self.cache.truncate(request_id, n_keep)

    # ---- the step ----------------------------------------------------------------------------------
    def _host_buffer(self, n_ints: int) -> torch.Tensor:
        """One of two pinned staging buffers, reused once the copy that last read it is done."""
        if len(self._pinned) < 2:
            self._pinned.append(torch.empty(max(n_ints, 1 << 14), dtype=torch.int32).pin_memory())
            self._pinned_events.append(None)
            i = len(self._pinned) - 1
        else:
            i = self._pinned_next
            self._pinned_next = (i + 1) % 2
            if self._pinned_events[i] is not None:
                self._pinned_events[i].synchronize()
            if self._pinned[i].numel() < n_ints:
                self._pinned[i] = torch.empty(n_ints * 2, dtype=torch.int32).pin_memory()
        self._slot_index = i
        return self._pinned[i]

    def _graphed_decode(self, entries: Sequence[StepEntry], sampling=None, from_device: bool = False, wait: bool = True):
        """A step in which every request has exactly one token: replays the captured graph of the next
        larger row count. Reservation, commit and the returned logits are those of the general path.
        With `sampling` (one (params, generator, history) per entry) the graph's own sampler picks the
        tokens and they are returned as a list instead of the logits; with `wait` false a `PendingDecode`
        is returned instead, for `collect_decode`. With `from_device` the rows' tokens are the ones the
        replay before this one sampled (same requests in the same rows): they are taken on the device,
        so the step can be launched before the host has seen them."""
        R = len(entries)
        rows = 1
        while rows < R:
            rows *= 2
        get = self.cache.get
        rcs = [get(e.request_id) for e in entries]
        # one graph per row count and power-of-two bound of the contexts: the slices of the decode attention are
        # cut for the bound, so short contexts do not pay for the longest one the engine allows
        longest = max(rc.num_tokens for rc in rcs) + 1
        bound = 256
        while bound < longest:
            bound *= 2
        bound = min(bound, self.options.ctx_size)
        gr = self._graphs.get((rows, bound))
        if gr is None:
            shared = self._decode_rows.get(rows)
            if shared is None:
                shared = self._decode_rows[rows] = _DecodeRows(rows, self.device)
            gr = self._graphs[(rows, bound)] = _DecodeGraph(self, rows, bound, shared)
        sh = gr.shared
        gr.copied.synchronize()                        # the previous copy out of the pinned buffer is done
        h = gr.h
        slot_list = [rc.slot for rc in rcs]
        if from_device:
            if sampling is None or sh.last_live != R:
                raise StepError("tokens can be taken on the device only from the sampled rows of the replay before")
        else:
            h["token_ids"][:R] = [e.tokens[0] for e in entries]
        h["positions"][:R] = [rc.num_tokens for rc in rcs]
        np.add(h["positions"][:R], 1, out=h["ctx_len"][:R])
        h["slots"][:R] = slot_list
        owners = gr.row_owner
        for r, rc in enumerate(rcs):
            owner = (rc.uid, rc.version)
            if owners[r] != owner:                     # a new request in this row, a new page, or a page a window freed
                for gi, tab in enumerate(rc.tables):
                    row = h["tables"][gi, r]
                    row[:len(tab)] = tab
                    row[len(tab):] = -1
                owners[r] = owner
                gr.tables_dirty = True
        if sampling is not None:
            h["temperature"][:R] = [s[0].temperature for s in sampling]
            h["top_k"][:R] = [s[0].top_k for s in sampling]
            h["top_p"][:R] = [s[0].top_p for s in sampling]
            h["min_p"][:R] = [s[0].min_p for s in sampling]
            for r, (prm, rng, _) in enumerate(sampling):
                if prm.temperature > 0:
                    h["uniform"][r] = rng.next_f32()
        else:
            h["temperature"][:R] = 0.0
        gr.fill_padding(R)
        gr.ctx.slot_list = slot_list + [gr.trash_slot] * (rows - R)
        n_copy = gr.dynamic_ints if gr.tables_dirty else gr.small_ints
        gr.tables_dirty = False
        gr.dev[:n_copy].copy_(gr.host[:n_copy], non_blocking=True)
        gr.copied.record()
        if from_device:                                # after the copy, which brought stale ids along
            gr.d["token_ids"][:R].copy_(sh.sampled[:R])
        self.last_h2d_bytes, self.last_d2h_bytes = 4 * n_copy, (4 * rows if sampling is not None else 0)
        gr.graph.replay()
        sh.last_live = R if sampling is not None else 0
        self.last_step_graph_kernels = gr.kernels
        for e in entries:
            self.cache.commit(e.request_id, 1)
        self.steps += 1
        self.graph_steps += 1
        if self.graph_steps % 256 == 0:                # graphs of more than a few rows hold tcgen05 products: look at their
            self._waits_unchecked = True               # status word now and then (a look costs a device synchronisation)
        self.tokens_run += R
        if sampling is not None:
            k = sh.next_buffer
            sh.next_buffer = k ^ 1
            sh.sampled_host[k].copy_(sh.sampled, non_blocking=True)
            sh.sampled_ready[k].record()
            pending = PendingDecode(gr, k, [r for r, e in enumerate(entries) if len(e.want)])
            return self.collect_decode(pending) if wait else pending
        wanted = [r for r, e in enumerate(entries) if len(e.want)]
        if len(wanted) == R:
            return gr.logits[:R]
        return gr.logits[torch.tensor(wanted, dtype=torch.long, device=self.device)] if wanted else gr.logits[:0]

    def collect_decode(self, pending: PendingDecode) -> List[int]:
        """Waits for a launched decode step's tokens (not for whatever was launched after it)."""
        sh = pending.graph.shared
        sh.sampled_ready[pending.buffer].synchronize()
        toks = sh.sampled_host[pending.buffer].numpy()
        return [int(toks[r]) for r in pending.rows]

    def launch_decode(self, entries: Sequence[StepEntry], rows, from_device: bool = False) -> Optional[PendingDecode]:
        """Launches a decode-only step with its sampler and returns without waiting for it, or returns None if
        the step is not one that the captured graphs take (then nothing has been done). At most two such
        steps may be uncollected at a time. See `_graphed_decode` for `from_device`."""
        if not (len(rows) == len(entries) and all(len(e.tokens) == 1 for e in entries) and self._graphs_usable(entries)
                and all(r[0].repeat_penalty == 1.0 for r in rows)):
            return None
        self._prepare(entries)
        return self._graphed_decode(entries, rows, from_device=from_device, wait=False)

    def step_and_sample(self, entries: Sequence[StepEntry], rows, sampler) -> List[int]:
        """A step followed by sampling: `rows` holds one (params, generator, history) per entry that wants
        logits (each such entry wants exactly its last token). Decode-only steps without a repeat penalty
        run the sampler inside the captured graph and bring back only the token ids."""
        pending = self.launch_decode(entries, rows)
        if pending is not None:
            return self.collect_decode(pending)
        logits = self.step(entries)
        return sampler.sample(logits, rows) if rows else []

    def _step_graph_pool(self):
        """One memory pool for all captured general steps: they never run at the same time, and a step's results are
        the caller's only until the next step."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    def _graphs_usable(self, entries) -> bool:
        if self._graph_safe is None:                   # the model's parts do not change after it is built
            self._graph_safe = bool(getattr(self.model, "graph_safe", False))
        return (self.options.cuda_graphs and self.fast and self.dtype == torch.bfloat16
                and self._graph_safe and len(entries) <= GRAPH_MAX_BATCH)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the entries' tokens as one batch; returns float32 logits `[wanted, vocab]` on the
        device, in the order of the entries and of each entry's `want`. Requests not seen before
        are admitted; pages are reserved here, and an `OutOfPages` leaves everything as it was.
        The returned tensor may be a view of a buffer that the next step overwrites: use or copy it
        before stepping again."""
        self._prepare(entries)
        if self._graphs_usable(entries) and all(len(e.tokens) == 1 for e in entries):
            return self._graphed_decode(entries)
        return self._general_step(entries)

    def _prepare(self, entries: Sequence[StepEntry]) -> None:
        """Checks the entries, admits new requests and reserves pages for the whole batch or not at all."""
        page = self.options.page_size
        if not entries:
            raise StepError("a step needs at least one entry")
        if self.options.debug_poison:
            self.storage.poison_freed_pages()
        if self._prepare_decode(entries):
            return
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request_id!r}: no tokens in its entry")
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise StepError(f"request {e.request_id!r}: token id {t} is outside the vocabulary (0..{self.vocab_size - 1})")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
        new_ids = [e.request_id for e in entries if e.request_id not in self.cache]
        free_slots = self.cache.max_requests - len(self.cache.live_requests())
        if len(new_ids) > free_slots:
            raise StepError(f"{len(new_ids)} new requests but only {free_slots} free request slots")
        # all-or-nothing reservation across the whole batch
        need = [0] * len(self.cache.paged_groups)
        for e in entries:
            held = self.cache.get(e.request_id) if e.request_id in self.cache else None
            n_have = held.num_tokens if held else 0
            if n_have + len(e.tokens) > self.options.ctx_size:
                raise StepError(f"request {e.request_id!r}: {n_have + len(e.tokens)} tokens exceed the context size {self.options.ctx_size}")
            total = -(-(n_have + len(e.tokens)) // page)
            for gi in range(len(need)):
                need[gi] += max(0, total - (len(held.tables[gi]) if held else 0))
        free = self.cache.free_pages()
        if any(n > f for n, f in zip(need, free)):
            raise OutOfPages(f"the step needs {need} pages per group, {free} are free")
        for rid in new_ids:
            self.cache.add_request(rid)
        for e in entries:
            ok = self.cache.reserve(e.request_id, len(e.tokens))
            assert ok, "reservation was checked for the whole batch"

    def _prepare_decode(self, entries: Sequence[StepEntry]) -> bool:
        """The common case in one pass: every entry is one token of a different live request that still has
        room on its last page. True: nothing is left to check or reserve. False: nothing was changed."""
        find = self.cache.find
        page, limit, vocab = self.options.page_size, self.options.ctx_size, self.vocab_size
        seen = set()
        for e in entries:
            rc = find(e.request_id)
            if rc is None or len(e.tokens) != 1 or rc.num_tokens >= limit:
                return False
            t = e.tokens[0]
            if type(t) is not int or not 0 <= t < vocab:
                return False
            for w in e.want:
                if w != 0:
                    return False
            room = rc.num_tokens < page * len(rc.tables[0]) if rc.tables else True
            for tab in rc.tables[1:]:
                room = room and rc.num_tokens < page * len(tab)
            if not room:
                return False
            seen.add(e.request_id)
        return len(seen) == len(entries)

    def _general_step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Any mix of portions and single tokens. The batch's index arrays and the parts' plans go to the device
        in one pinned copy. A batch whose padded shape has been seen before replays a captured graph (`_StepGraph`);
        otherwise the kernels are launched one by one."""
        self.last_step_graph_kernels = 0
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        N = sum(len(e.want) for e in entries)
        rcs = [self.cache.get(e.request_id) for e in entries]
        q_lens = [len(e.tokens) for e in entries]
        ctx_lens = [rc.num_tokens + n for rc, n in zip(rcs, q_lens)]
        logits = None
        if self._step_graphs_usable(T, N):
            logits = self._graphed_step(entries, rcs, q_lens, ctx_lens, T, N)
        if logits is None:
            logits = self._eager_step(entries, rcs, q_lens, ctx_lens, T, N)
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps += 1
        self.tokens_run += T
        return logits

    def _eager_step(self, entries, rcs, q_lens, ctx_lens, T: int, N: int) -> torch.Tensor:
        R = len(entries)
        G = len(self.cache.paged_groups)
        width = max(1, max(len(t) for rc in rcs for t in (rc.tables or [[0]])))
        width = -(-width // 8) * 8
        collect = getattr(self.model, "collect_plans", None)
        plans = collect(q_lens, ctx_lens, None) if collect is not None else {}
        plan_items = [((key, name), arr) for key, plan in plans.items() for name, arr in plan.arrays.items()]
        n_ints = 3 * T + (R + 1) + 2 * R + N + G * R * width + sum(int(a.size) for _, a in plan_items)
        host = self._host_buffer(n_ints)
        h = host.numpy()
        o = 0

        def take_host(n):
            nonlocal o
            v = h[o:o + n]; o += n
            return v
        fields = dict(token_ids=take_host(T), positions=take_host(T), tok_req=take_host(T), cu_q=take_host(R + 1),
                      ctx_len=take_host(R), slots=take_host(R), logit_rows=take_host(N),
                      tables=take_host(G * R * width).reshape(G, R, width))
        for _, arr in plan_items:
            take_host(int(arr.size))[:] = arr.reshape(-1)
        slot_list = _fill_batch(fields, entries, rcs, q_lens, ctx_lens)
        dev = torch.empty(n_ints, dtype=torch.int32, device=self.device)
        dev.copy_(host[:n_ints], non_blocking=True)
        self.last_h2d_bytes, self.last_d2h_bytes = 4 * n_ints, 0
        ev = torch.cuda.Event()
        ev.record()
        self._pinned_events[self._slot_index] = ev
        o = 0

        def take(n):
            nonlocal o
            v = dev[o:o + n]; o += n
            return v
        ctx = StepContext(
            dtype=self.dtype, device=self.device, T=T, R=R,
            token_ids=take(T), positions=take(T), tok_req=take(T), cu_q=take(R + 1), ctx_len=take(R),
            slots=take(R), logit_rows=take(N),
            block_tables=[take(R * width).view(R, width) for _ in range(G)],
            q_lens=q_lens, ctx_lens=ctx_lens, slot_list=slot_list, storage=self.storage, fast=self.fast)
        ctx.plans = _plans_on_device(plans, {k: take(int(arr.size)).view(arr.shape) for k, arr in plan_items})
        logits = self.model.forward(ctx)
        self._waits_unchecked = self.fast and self.dtype == torch.bfloat16
        return logits

    # ---- captured general steps ------------------------------------------------------------------------
    def _step_graphs_usable(self, T: int, N: int) -> bool:
        if self._graph_safe is None:
            self._graph_safe = bool(getattr(self.model, "graph_safe", False))
        return (self.options.cuda_graphs and self.options.step_graph_after > 0 and self.fast
                and self.dtype == torch.bfloat16 and self._graph_safe and N <= STEP_GRAPH_MAX_WANTED
                and T <= self.options.max_num_batched_tokens + GRAPH_MAX_BATCH)

    def _graphed_step(self, entries, rcs, q_lens, ctx_lens, T: int, N: int) -> Optional[torch.Tensor]:
        """The batch padded to a shape that other batches share: tokens up to a multiple of 16, each padding token a
        single-token request of its own on the spare page (a legitimate batch for every kernel), then requests
        without tokens up to a multiple of 8 (at least one: the parts' padded work lists point at it), wanted rows
        up to a multiple of 8. A shape replays its captured graph; it is captured when it comes for the
        `step_graph_after`-th time, and the least recently used graph makes room when there are too many. Returns
        None when the step should be launched kernel by kernel."""
        R = len(entries)
        T_b = -(-T // 16) * 16
        pads = T_b - T
        R_b = -(-(R + pads + 1) // 8) * 8
        N_b = max(8, -(-N // 8) * 8)
        q_ext = q_lens + [1] * pads + [0] * (R_b - R - pads)
        c_ext = ctx_lens + [1] * (R_b - R)
        plans = self.model.collect_plans(q_ext, c_ext, R_b - 1)
        key = (T_b, R_b, N_b, tuple(sorted((k, p.shape) for k, p in plans.items())))
        gr = self._step_graphs.get(key)
        if gr is None:
            seen = self._step_shapes_seen.get(key, 0) + 1
            self._step_shapes_seen[key] = seen
            if len(self._step_shapes_seen) > 4096:
                self._step_shapes_seen.clear()
            if seen < self.options.step_graph_after:
                return None
            if len(self._step_graphs) >= STEP_GRAPH_CACHE:
                del self._step_graphs[next(iter(self._step_graphs))]
            gr = _StepGraph(self, T_b, R_b, N_b, plans)
        else:
            del self._step_graphs[key]
        self._step_graphs[key] = gr                    # most recently used last
        gr.copied.synchronize()
        f = gr.fields
        f["token_ids"][T:] = 0
        f["positions"][T:] = 0
        f["tok_req"][T:] = np.arange(R, R + pads, dtype=np.int32)
        f["cu_q"][R:R + pads + 1] = np.arange(T, T_b + 1, dtype=np.int32)
        f["cu_q"][R + pads + 1:] = T_b
        f["ctx_len"][R:] = 1
        f["slots"][R:] = self.storage.trash_slot
        f["logit_rows"][N:] = 0
        f["tables"][...] = -1
        f["tables"][:, R:, 0] = self.storage.trash_page
        for (k, name), dst in gr.plan_host.items():
            dst[...] = plans[k].arrays[name]
        gr.ctx.slot_list = _fill_batch(f, entries, rcs, q_lens, ctx_lens) + [self.storage.trash_slot] * (R_b - R)
        gr.dev.copy_(gr.host, non_blocking=True)
        gr.copied.record()
        self.last_h2d_bytes, self.last_d2h_bytes = 4 * gr.host.numel(), 0
        self._waits_unchecked = True
        if gr.graph is None:                           # the first time: run it kernel by kernel, then capture it
            logits = self.model.forward(gr.ctx)[:N]
            gr.capture(self)
            return logits
        gr.graph.replay()
        self.last_step_graph_kernels = gr.kernels
        self.graph_steps += 1
        return gr.logits[:N]

    def check_kernels(self) -> None:
        """The tcgen05 kernels bound every wait on a barrier and record it when a bound runs out instead of
        hanging; the results of such a launch are invalid. Raises then. Call after the step's results have been
        read (it synchronises); costs nothing when no such kernel ran since the last call."""
        if self._waits_unchecked:
            self._waits_unchecked = False
            from ..kernels import ops
            ops.check_status()
