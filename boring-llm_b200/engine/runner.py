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
from ..parts import StepContext


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


class PendingDecode:
    """A decode step that has been launched and whose sampled tokens have not been read yet."""
    __slots__ = ("graph", "buffer", "rows")

    def __init__(self, graph: "_DecodeGraph", buffer: int, rows: List[int]):
        self.graph, self.buffer, self.rows = graph, buffer, rows


class _DecodeGraph:
    """A captured decode step for a fixed number of rows. All per-step inputs live in one int32 device
    buffer that a single copy refreshes before each replay; rows beyond the live requests point at the
    storage's spare page and slot."""

    def __init__(self, runner: "ModelRunner", rows: int):
        self.rows = rows
        G = len(runner.cache.paged_groups)
        W = runner._table_width
        B = rows
        sizes = [("token_ids", B), ("positions", B), ("ctx_len", B), ("slots", B),
                 ("temperature", B), ("top_k", B), ("top_p", B), ("min_p", B), ("uniform", B),
                 ("tables", G * B * W),
                 ("tok_req", B), ("cu_q", B + 1), ("logit_rows", B), ("decode_reqs", B)]
        total = sum(n for _, n in sizes)
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(total, dtype=torch.int32, device=runner.device)
        self.h: Dict[str, np.ndarray] = {}
        self.d: Dict[str, torch.Tensor] = {}
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
        self.h["tok_req"][:] = ar; self.h["logit_rows"][:] = ar; self.h["decode_reqs"][:] = ar
        self.h["cu_q"][:] = np.arange(B + 1, dtype=np.int32)
        self.trash_page, self.trash_slot = runner.storage.trash_page, runner.storage.trash_slot
        self.fill_padding(0)
        self.dev.copy_(self.host)
        self.ctx = StepContext(
            dtype=runner.dtype, device=runner.device, T=B, R=B, token_ids=self.d["token_ids"],
            positions=self.d["positions"], tok_req=self.d["tok_req"], cu_q=self.d["cu_q"], ctx_len=self.d["ctx_len"],
            slots=self.d["slots"], logit_rows=self.d["logit_rows"],
            block_tables=[self.d["tables"][g * B * W:(g + 1) * B * W].view(B, W) for g in range(G)],
            q_lens=[1] * B, ctx_lens=[runner.options.ctx_size] * B, slot_list=[runner.storage.trash_slot] * B,
            storage=runner.storage, fast=True, decode_reqs=self.d["decode_reqs"],
            max_decode_ctx=runner.options.ctx_size)
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
        self.sampled = torch.zeros(B, dtype=torch.int32, device=runner.device)
        with torch.cuda.graph(self.graph):
            self.logits = runner.model.forward(self.ctx)
            # one token per row from the step's own logits: greedy rows (temperature 0) cost one pass
            ops.sample(self.logits, self.d["temperature"], self.d["top_k"], self.d["top_p"], self.d["min_p"],
                       self.d["uniform"], self.sampled)
        self.kernels = ops.launch_count - before       # kernels of this library that one replay launches
        self.copied = torch.cuda.Event()
        # two steps may be in flight (the next is launched before this one's tokens are read): two buffers take turns
        self.sampled_host = [torch.zeros(B, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.sampled_ready = [torch.cuda.Event() for _ in range(2)]
        self.next_buffer = 0
        self.last_live = 0                             # live rows of the last replay (whose tokens `sampled` holds)

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
        self._graphs: Dict[int, "_DecodeGraph"] = {}
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
        gr = self._graphs.get(rows)
        if gr is None:
            gr = self._graphs[rows] = _DecodeGraph(self, rows)
        gr.copied.synchronize()                        # the previous copy out of the pinned buffer is done
        h = gr.h
        get = self.cache.get
        rcs = [get(e.request_id) for e in entries]
        slot_list = [rc.slot for rc in rcs]
        if from_device:
            if sampling is None or gr.last_live != R:
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
            gr.d["token_ids"][:R].copy_(gr.sampled[:R])
        self.last_h2d_bytes, self.last_d2h_bytes = 4 * n_copy, (4 * rows if sampling is not None else 0)
        gr.graph.replay()
        gr.last_live = R if sampling is not None else 0
        self.last_step_graph_kernels = gr.kernels
        for e in entries:
            self.cache.commit(e.request_id, 1)
        self.steps += 1
        self.graph_steps += 1
        if self.graph_steps % 256 == 0:                # graphs of more than a few rows hold tcgen05 products: look at their
            self._waits_unchecked = True               # status word now and then (a look costs a device synchronisation)
        self.tokens_run += R
        if sampling is not None:
            k = gr.next_buffer
            gr.next_buffer = k ^ 1
            gr.sampled_host[k].copy_(gr.sampled, non_blocking=True)
            gr.sampled_ready[k].record()
            pending = PendingDecode(gr, k, [r for r, e in enumerate(entries) if len(e.want)])
            return self.collect_decode(pending) if wait else pending
        wanted = [r for r, e in enumerate(entries) if len(e.want)]
        if len(wanted) == R:
            return gr.logits[:R]
        return gr.logits[torch.tensor(wanted, dtype=torch.long, device=self.device)] if wanted else gr.logits[:0]

    def collect_decode(self, pending: PendingDecode) -> List[int]:
        """Waits for a launched decode step's tokens (not for whatever was launched after it)."""
        gr = pending.graph
        gr.sampled_ready[pending.buffer].synchronize()
        toks = gr.sampled_host[pending.buffer].numpy()
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
        """Any mix of portions and single tokens: metadata built for this batch, kernels launched one by one."""
        self.last_step_graph_kernels = 0
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        N = sum(len(e.want) for e in entries)
        G = len(self.cache.paged_groups)
        rcs = [self.cache.get(e.request_id) for e in entries]
        width = max(1, max(len(t) for rc in rcs for t in (rc.tables or [[0]])))
        width = -(-width // 8) * 8
        tiles = [(r, t0) for r, e in enumerate(entries) if len(e.tokens) > 1 for t0 in range(0, len(e.tokens), 64)]
        singles = [r for r, e in enumerate(entries) if len(e.tokens) == 1]
        n_ints = 3 * T + (R + 1) + 2 * R + N + G * R * width + 2 * len(tiles) + len(singles)
        host = self._host_buffer(n_ints)
        h = host.numpy()
        o = 0
        token_ids = h[o:o + T]; o += T
        positions = h[o:o + T]; o += T
        tok_req = h[o:o + T]; o += T
        cu_q = h[o:o + R + 1]; o += R + 1
        ctx_len = h[o:o + R]; o += R
        slots = h[o:o + R]; o += R
        logit_rows = h[o:o + N]; o += N
        tables = h[o:o + G * R * width].reshape(G, R, width); o += G * R * width
        tables[...] = -1
        tile_arr = h[o:o + 2 * len(tiles)]; o += 2 * len(tiles)
        single_arr = h[o:o + len(singles)]; o += len(singles)
        if tiles:
            tile_arr[:] = np.asarray(tiles, dtype=np.int32).reshape(-1)
        if singles:
            single_arr[:] = np.asarray(singles, dtype=np.int32)
        t0 = 0
        n_want = 0
        q_lens, ctx_lens, slot_list = [], [], []
        for r, (e, rc) in enumerate(zip(entries, rcs)):
            n = len(e.tokens)
            token_ids[t0:t0 + n] = np.asarray(e.tokens, dtype=np.int32)
            positions[t0:t0 + n] = np.arange(rc.num_tokens, rc.num_tokens + n, dtype=np.int32)
            tok_req[t0:t0 + n] = r
            cu_q[r] = t0
            ctx_len[r] = rc.num_tokens + n
            slots[r] = rc.slot
            for w in e.want:
                logit_rows[n_want] = t0 + int(w)
                n_want += 1
            for gi in range(G):
                tab = rc.tables[gi]
                tables[gi, r, :len(tab)] = tab
            q_lens.append(n); ctx_lens.append(rc.num_tokens + n); slot_list.append(rc.slot)
            t0 += n
        cu_q[R] = T
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
        if tiles:
            ctx.prefill_tiles = take(2 * len(tiles)).view(len(tiles), 2)
            ctx.prefill_tokens = sum(n for n in q_lens if n > 1)
        if singles:
            ctx.decode_reqs = take(len(singles))
            ctx.max_decode_ctx = max(ctx_lens[r] for r in singles)
        logits = self.model.forward(ctx)
        self._waits_unchecked = self.fast and self.dtype == torch.bfloat16
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps += 1
        self.tokens_run += T
        return logits

    def check_kernels(self) -> None:
        """The tcgen05 kernels bound every wait on a barrier and record it when a bound runs out instead of
        hanging; the results of such a launch are invalid. Raises then. Call after the step's results have been
        read (it synchronises); costs nothing when no such kernel ran since the last call."""
        if self._waits_unchecked:
            self._waits_unchecked = False
            from ..kernels import ops
            ops.check_status()
