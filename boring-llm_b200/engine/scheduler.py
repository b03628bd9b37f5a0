"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees, and decides what happens when pages run out.

The reference serves one request at a time (README.md:235, src/server.br:2030-2054); what it has in
this role is the admission check against the context size (src/server.br:646-649, 660-663), prompt
portions of `min(batch, ubatch)` tokens (src/cli_config.br:24-25, src/model.br:2264-2278) and the
generation loop that samples, stops on an end-of-generation token WITHOUT feeding it, and otherwise
feeds the token back (src/model.br:2293-2304). Continuous batching, the page-based admission and
preemption are this engine's own.

Policy of one step, in order, under `max_num_batched_tokens`:
  1. every running request that is decoding gets its one token;
  2. running requests still inside their prompt get `min(remaining, prefill_chunk, budget left)`;
  3. waiting requests are admitted in arrival order while a slot is free and the pages of their
     first portion can be reserved (never while a preempted request waits for pages).
When a running request cannot get the pages for its tokens, the most recently admitted running
request is preempted: its pages and slot are freed and it goes back to the FRONT of the queue with
its generated tokens kept as part of what has to be recomputed. The oldest running request is never
the victim unless it is the only one; if it alone cannot fit, it ends with the reason "out_of_cache".
This module never touches the GPU: it decides, `apply()` records what the step produced.
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

from ..cache import CacheManager
from ..config import EngineOptions
from ..sampling.params import SamplingParams, XorShift64
from .runner import StepEntry

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class AdmissionError(ValueError):
    """A request that can never run: empty prompt, or no room for even one new token."""


@dataclass(eq=False)          # a request is itself: lists of requests are searched by identity, not by comparing fields
class Request:
    request_id: object
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    num_computed: int = 0                 # tokens whose keys and values are in the cache
    state: str = WAITING
    finish_reason: Optional[str] = None   # "stop" (end token), "length", "out_of_cache", "aborted"
    max_new: int = 0
    arrival: int = 0
    preemptions: int = 0
    rng: Optional[XorShift64] = None

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def token_slice(self, a: int, b: int) -> List[int]:
        """tokens[a:b] without building the whole list (a decode step wants one token of thousands)."""
        n = len(self.prompt)
        if b <= n:
            return self.prompt[a:b]
        if a >= n:
            return self.output[a - n:b - n]
        return self.prompt[a:] + self.output[:b - n]

    @property
    def remaining(self) -> int:
        """Tokens known but not yet in the cache."""
        return len(self.prompt) + len(self.output) - self.num_computed


@dataclass
class ScheduledStep:
    entries: List[StepEntry]
    requests: List[Request]               # same order as entries
    samples: List[bool]                   # whether the entry's last token yields a sampled token


class Scheduler:
    def __init__(self, cache: CacheManager, options: EngineOptions):
        self.cache = cache
        self.options = options
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in admission order: oldest first
        self.finished: Dict[object, Request] = {}
        self._arrivals = itertools.count()
        self.num_preemptions = 0

    # ---- admission ---------------------------------------------------------------------------------
    def add(self, request_id, prompt: Sequence[int], params: SamplingParams) -> Request:
        """Queues a request. Refused like the reference's server (src/server.br:642-649): an empty
        prompt, or a prompt that leaves no room in the context; `n_predict` is clamped to the room
        (negative: all the room, :660-663)."""
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise AdmissionError("empty prompt")
        room = self.options.ctx_size - len(prompt)
        if room <= 0:
            raise AdmissionError(
                f"context_length_exceeded: the prompt has {len(prompt)} tokens, the context size is {self.options.ctx_size}")
        if -(-(len(prompt) + 1) // self.cache.page_size) > self.cache.num_pages:
            raise AdmissionError(
                f"out_of_cache: the prompt has {len(prompt)} tokens, the cache holds {self.cache.num_pages * self.cache.page_size}")
        max_new = room if params.n_predict < 0 else min(params.n_predict, room)
        req = Request(request_id, prompt, params, max_new=max_new, arrival=next(self._arrivals),
                      rng=XorShift64(params.seed))
        if max_new == 0:
            self._finish(req, "length", live=False)
            return req
        self.waiting.append(req)
        return req

    def abort(self, request_id, reason: str = "aborted") -> None:
        """Ends a request wherever it is; its pages and slot go back at once."""
        for req in list(self.running):
            if req.request_id == request_id:
                self.running.remove(req)
                self._finish(req, reason, live=True)
                return
        for req in list(self.waiting):
            if req.request_id == request_id:
                self.waiting.remove(req)
                self._finish(req, reason, live=False)
                return

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step ----------------------------------------------------------------------------------
    def schedule(self) -> Optional[ScheduledStep]:
        budget = self.options.max_num_batched_tokens
        chunk = self.options.effective_prefill_chunk
        picked: Dict[int, tuple] = {}             # id(request) -> (request, n tokens), in pick order
        preempted = False

        def drop(victim: Request) -> None:
            nonlocal budget, preempted
            if id(victim) in picked:
                budget += picked.pop(id(victim))[1]
            self._preempt(victim)
            preempted = True

        def try_take(req: Request, n: int) -> None:
            """Pages for n more tokens of a running request; younger requests yield theirs if needed."""
            nonlocal budget
            while not self.cache.reserve(req.request_id, n):
                younger = [r for r in self.running if r.arrival > req.arrival]
                if younger:
                    drop(max(younger, key=lambda r: r.arrival))
                elif len(self.running) > 1:
                    drop(req)                      # its elders hold the pages: wait for them
                    return
                else:
                    self.running.remove(req)       # alone and still too large for the cache
                    self._finish(req, "out_of_cache", live=True)
                    return
            picked[id(req)] = (req, n)
            budget -= n

        # 1. decoding requests, oldest first
        for req in list(self.running):
            if budget <= 0:
                break
            if req.state == RUNNING and req.output and req.remaining == 1:
                try_take(req, 1)
        # 2. running requests inside their prompt (or re-computing after a preemption)
        for req in list(self.running):
            if budget <= 0:
                break
            if req.state == RUNNING and id(req) not in picked and req.remaining > 0:
                try_take(req, min(req.remaining, chunk, budget))
        # 3. admissions in arrival order; none in a step that had to preempt
        while self.waiting and budget > 0 and not preempted and self.cache.has_free_slot():
            req = self.waiting[0]
            n = min(req.remaining, chunk, budget)
            self.cache.add_request(req.request_id)
            if not self.cache.reserve(req.request_id, n):
                self.cache.free(req.request_id)
                if not self.running:               # nobody holds pages, so it can never fit
                    self.waiting.popleft()
                    self._finish(req, "out_of_cache", live=False)
                    continue
                break
            self.waiting.popleft()
            req.state = RUNNING
            self.running.append(req)
            picked[id(req)] = (req, n)
            budget -= n
        if not picked:
            return None
        entries, reqs, samples = [], [], []
        for req, n in picked.values():
            toks = req.token_slice(req.num_computed, req.num_computed + n)
            last = req.num_computed + n == len(req.prompt) + len(req.output)
            entries.append(StepEntry(req.request_id, toks, [n - 1] if last else []))
            reqs.append(req)
            samples.append(last)
        return ScheduledStep(entries, reqs, samples)

    def lookahead(self, prev: ScheduledStep) -> Optional[ScheduledStep]:
        """The decode step that follows `prev`, put together BEFORE `prev`'s tokens are known, so that it can be
        launched while `prev` still runs (its input tokens are then taken on the device; the entries carry
        token 0 in their place). Only when that step is certain but for end-of-generation tokens: `prev` was a
        decode step of all running requests in their order, nobody waits, none of them ends by length with
        `prev`'s token, and the pages for one more token each are there. Otherwise None, and nothing is changed
        but pages that the requests' next tokens need anyway. A request that `prev` ends with an end token still
        has its row in the step: `apply` skips it."""
        if self.waiting or len(prev.requests) != len(self.running):
            return None
        for req, run, e, samp in zip(prev.requests, self.running, prev.entries, prev.samples):
            if req is not run or req.state != RUNNING or not samp or len(e.tokens) != 1:
                return None
            n_out = len(req.output) + 1                       # once prev's token is there
            if n_out >= req.max_new or len(req.prompt) + n_out >= self.options.ctx_size:
                return None
        if len(prev.requests) > self.options.max_num_batched_tokens:
            return None
        for req in prev.requests:
            if not self.cache.reserve(req.request_id, 1):
                return None
        return ScheduledStep([StepEntry(req.request_id, [0], [0]) for req in prev.requests], list(prev.requests),
                             [True] * len(prev.requests))

    def apply(self, step: ScheduledStep, sampled: Sequence[int]) -> List[Request]:
        """Records a finished step: `sampled` holds one token for every entry with `samples` true, in
        order. Returns the requests that finished. An end-of-generation token is returned but not
        fed (src/model.br:2299-2300); `n_predict` tokens or a full context end with "length"."""
        done = []
        it = iter(sampled)
        for e, req, samp in zip(step.entries, step.requests, step.samples):
            if req.state != RUNNING:                          # ended or preempted since the step was put together
                if samp:
                    next(it, None)                            # its row's token belongs to nobody
                continue
            req.num_computed += len(e.tokens)
            if not samp:
                continue
            tok = int(next(it))
            req.output.append(tok)
            p = req.params
            if not p.ignore_eos and tok in p.eos_token_ids:
                reason = "stop"
            elif len(req.output) >= req.max_new:
                reason = "length"
            elif len(req.prompt) + len(req.output) >= self.options.ctx_size:
                reason = "length"
            else:
                continue
            self.running.remove(req)
            self._finish(req, reason, live=True)
            done.append(req)
        return done

    # ---- inner workings ----------------------------------------------------------------------------
    def _preempt(self, victim: Request) -> None:
        """Preemption by recomputation: everything the victim holds is freed, and it waits at the
        FRONT of the queue with its generated tokens kept as part of what is to be recomputed."""
        self.running.remove(victim)
        self.cache.free(victim.request_id)
        victim.num_computed = 0
        victim.state = WAITING
        victim.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)

    def _finish(self, req: Request, reason: str, live: bool) -> None:
        req.state = FINISHED
        req.finish_reason = reason
        if live and req.request_id in self.cache:
            self.cache.free(req.request_id)
        self.finished[req.request_id] = req
