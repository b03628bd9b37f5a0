"""Runs ONE part through the engine's real step machinery (runner, cache manager, pages, metadata)
without a model around it: token ids select rows of a prepared input, and the step returns whatever
the part produced for the batch's tokens."""
import torch

from boring_llm_b200.config import EngineOptions
from boring_llm_b200.engine.runner import ModelRunner, StepEntry


class Probe:
    def __init__(self, inputs, body, cache_specs=()):
        self.inputs, self.body, self._specs = inputs, body, list(cache_specs)
        self.vocab_size = inputs.shape[0]

    def cache_specs(self):
        return self._specs

    def forward(self, ctx):
        x = self.inputs[ctx.token_ids.long()].contiguous()
        return self.body(ctx, x)


def runner_for(inputs, body, cache_specs=(), dtype="float32", max_tokens=256, fast=True):
    opts = EngineOptions(dtype=dtype, max_tokens=max_tokens, ctx_size=max_tokens, max_num_seqs=4, cuda_graphs=False)
    r = ModelRunner(Probe(inputs, body, cache_specs), opts)
    r.fast = fast
    return r


def run_portions(runner, rid, n_tokens, sizes):
    """Feeds token ids 0..n-1 of one request in the given portions; returns the concatenated outputs."""
    outs, at = [], 0
    for n in sizes:
        outs.append(runner.step([StepEntry(rid, list(range(at, at + n)), [])]).clone())
        at += n
    assert at == n_tokens
    runner.free_request(rid)
    return torch.cat(outs)
