"""The Python entry point: token ids in, token ids out.

`Engine.generate` plays the reference's `generate_kv` (src/model.br:2280-2306: chunked prefill,
then sample, stop on an end token, else feed the token back), for many requests at once: the
scheduler builds each step's batch, the runner computes logits, the device sampler picks tokens.
"""
from __future__ import annotations

import itertools
import time
from typing import Dict, List, Optional, Sequence

import torch

from ..config import EngineOptions
from ..models.loading import load_model, load_random_model
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .runner import ModelRunner, StepEntry
from .scheduler import RUNNING, Request, Scheduler


class Engine:
    def __init__(self, model_dir: str, options: Optional[EngineOptions] = None, **overrides):
        """Loads the model folder (config.json chooses the model class) onto the device.
        `overrides` set fields of `EngineOptions` (dtype, ctx_size, max_tokens, ...)."""
        if options is None:
            options = EngineOptions(**overrides)
        elif overrides:
            raise TypeError("give either options or keyword overrides, not both")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this engine runs on an sm_100a GPU only (there is no CPU path)")
        self.options = options
        if isinstance(model_dir, tuple):
            self.config, self.model = model_dir          # (configuration, model already on the device)
        else:
            self.config, self.model = load_model(model_dir, options.dtype, options.device)
        max_pos = getattr(self.config, "max_position_embeddings", None)
        if max_pos is not None and options.ctx_size > max_pos:
            raise ValueError(f"ctx_size {options.ctx_size} exceeds the model's max_position_embeddings {max_pos}")
        self.runner = ModelRunner(self.model, options)
        self.scheduler = Scheduler(self.runner.cache, options)
        self.sampler = Sampler(options.device)
        self._ids = itertools.count()
        self._inflight = None                 # (scheduled step, PendingDecode): launched, tokens not read yet
        self.stats_time = {"engine_steps": 0, "step_seconds": 0.0}

    @classmethod
    def from_model(cls, config, model, options: EngineOptions) -> "Engine":
        """An engine around a model that is already built and loaded on the device."""
        return cls((config, model), options)

    @classmethod
    def from_random(cls, config, seed: int, options: Optional[EngineOptions] = None, std: float = 0.02,
                    weight_dtype=None) -> "Engine":
        """An engine around a model with seeded random weights, made on the device without a file (the same
        tensors as `write_random_model` writes for this configuration, seed and standard deviation)."""
        options = options if options is not None else EngineOptions()
        return cls(load_random_model(config, seed, options.dtype, options.device, std, weight_dtype), options)

    # ---- requests ----------------------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, request_id=None) -> Request:
        if params is None:
            params = SamplingParams()
        if not params.eos_token_ids and not params.ignore_eos:
            params.eos_token_ids = tuple(getattr(self.config, "eos_token_ids", ()))
        for t in prompt:
            if not 0 <= int(t) < self.runner.vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary (0..{self.runner.vocab_size - 1})")
        rid = request_id if request_id is not None else next(self._ids)
        return self.scheduler.add(rid, prompt, params)

    def step(self) -> List[Request]:
        """One scheduler step. Returns the requests that finished in it.

        While the running requests only decode, the step after this one is launched before this one's tokens are
        read (`EngineOptions.lookahead`): the device feeds the sampled tokens back itself, the host reads them one
        step behind, and the GPU does not wait for the host between steps. A request that ends with an end token
        has then already got a row in the step after; that row's result is dropped (the reference's loop,
        src/model.br:2293-2304, feeds no token after the end token either: nothing of the row is kept)."""
        t0 = time.perf_counter()
        if self._inflight is None:
            sched = self.scheduler.schedule()
            if sched is None:
                return []
            # the third item is the request itself: its token history is only put together if a penalty asks for it
            rows = [(r.params, r.rng, r) for r, s in zip(sched.requests, sched.samples) if s]
            pending = self.runner.launch_decode(sched.entries, rows) if self.options.lookahead else None
            if pending is None:
                sampled = self.runner.step_and_sample(sched.entries, rows, self.sampler)
                return self._finish_step(sched, sampled, t0)
            self._inflight = (sched, pending)
        sched, pending = self._inflight
        ahead = self.scheduler.lookahead(sched)
        nxt = None
        if ahead is not None:
            rows = [(r.params, r.rng, r) for r in ahead.requests]
            p2 = self.runner.launch_decode(ahead.entries, rows, from_device=True)
            if p2 is not None:
                nxt = (ahead, p2)
        try:
            sampled = self.runner.collect_decode(pending)
            done = self._finish_step(sched, sampled, t0)
        except BaseException:
            # The step in flight failed (a kernel gave up on a bounded wait, the read of its tokens failed). The step
            # ahead has already been launched: it has taken cache positions and random numbers for every row. Nothing of
            # either step can be kept: forget both and end their requests, so that the scheduler and the cache agree
            # again before the error reaches the caller.
            self._inflight = None
            self._abort_rows(sched.requests + (nxt[0].requests if nxt is not None else []))
            raise
        if nxt is not None and not any(r.state == RUNNING for r in nxt[0].requests):
            nxt = None                            # every row of the step ahead has ended: nobody reads it
        self._inflight = nxt
        return done

    def _abort_rows(self, requests) -> None:
        seen = set()
        for r in requests:
            if r.request_id in seen:
                continue
            seen.add(r.request_id)
            self.scheduler.abort(r.request_id, "error")

    def drain(self) -> List[Request]:
        """Reads the step that was launched ahead, if there is one, so that the host's view is complete.
        Returns the requests that finished in it."""
        if self._inflight is None:
            return []
        (sched, pending), self._inflight = self._inflight, None
        return self._finish_step(sched, self.runner.collect_decode(pending), time.perf_counter())

    def _finish_step(self, sched, sampled, t0) -> List[Request]:
        self.runner.check_kernels()
        self.stats_time["engine_steps"] += 1
        self.stats_time["step_seconds"] += time.perf_counter() - t0
        return self.scheduler.apply(sched, sampled)

    def run_until_done(self) -> None:
        while self.scheduler.has_work():
            before = (len(self.scheduler.waiting), len(self.scheduler.running), len(self.scheduler.finished))
            self.step()
            after = (len(self.scheduler.waiting), len(self.scheduler.running), len(self.scheduler.finished))
            if before == after and not self.scheduler.running:
                raise RuntimeError("the scheduler made no progress with requests still waiting")

    def generate(self, prompts: Sequence[Sequence[int]], n_predict: int = 40, temperature: float = 0.0,
                 seed: int = 0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
                 repeat_penalty: float = 1.0, repeat_last_n: int = 64,
                 eos_token_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False) -> List[List[int]]:
        """Generated token ids for each prompt (lists of token ids), in the prompts' order. Request i
        draws from a generator seeded with `seed + i`, so a batch and the same prompts one by one
        give the same tokens."""
        reqs = []
        for i, prompt in enumerate(prompts):
            params = SamplingParams(n_predict=n_predict, temperature=temperature, seed=seed + i, top_k=top_k,
                                    top_p=top_p, min_p=min_p, repeat_penalty=repeat_penalty,
                                    repeat_last_n=repeat_last_n,
                                    eos_token_ids=tuple(eos_token_ids) if eos_token_ids is not None else (),
                                    ignore_eos=ignore_eos)
            reqs.append(self.add_request(prompt, params))
        self.run_until_done()
        return [list(r.output) for r in reqs]

    def stats(self) -> dict:
        s = dict(self.runner.cache.stats())
        s.update(steps=self.runner.steps, tokens_run=self.runner.tokens_run,
                 preemptions=self.scheduler.num_preemptions, **self.stats_time)
        return s


def generate(model_dir: str, prompts: Sequence[Sequence[int]], n_predict: int = 40, temperature: float = 0.0,
             seed: int = 0, dtype: str = "bfloat16", ctx_size: int = 4096, **sampling) -> List[List[int]]:
    """One call from a model folder and prompts (token ids) to generated token ids."""
    eng = Engine(model_dir, dtype=dtype, ctx_size=ctx_size, max_num_seqs=max(1, min(64, len(prompts))))
    return eng.generate(prompts, n_predict=n_predict, temperature=temperature, seed=seed, **sampling)
