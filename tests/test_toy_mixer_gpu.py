"""A toy architecture defined HERE, outside the framework: a mixer with per-request state of fixed size
(an exponential running mean of its inputs) beside an ordinary attention layer. It is registered,
written as a random model folder, loaded through config.json, and stepped in portions and mixed
batches, without a change to the framework's files. It is a test fixture, not a model of anyone's."""
import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_model as plain

pytestmark = pytest.mark.gpu


def define_toy():
    from boring_llm_b200.cache import StateSpec
    from boring_llm_b200.config import register_architecture
    from boring_llm_b200.parts import (DecoderModel, Embedding, GQAAttention, Mixer, OutputHead, PreNormBlock, RMSNorm,
                                       RotaryTable, SwiGLU)
    from boring_llm_b200.weights import TensorSpec, MATRIX

    @dataclass(frozen=True)
    class ToyConfig:
        architecture: str
        vocab_size: int
        dim: int
        decay: float
        max_position_embeddings: int = 512

        @classmethod
        def from_dict(cls, d):
            return cls(d["architectures"][0], d["vocab_size"], d["dim"], d["decay"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "dim": self.dim, "decay": self.decay}

    class RunningMean(Mixer):
        """state <- decay * state + (1 - decay) * h_t, token by token; adds W . state_t to the residual."""

        def __init__(self, dim, decay, names):
            super().__init__(names)
            self.dim, self.decay = dim, decay

        def local_specs(self):
            return {"w": TensorSpec((self.dim, self.dim), MATRIX)}

        def cache_spec(self):
            return StateSpec((self.dim,), "float32")

        def forward(self, ctx, h, residual, cache_layer, write_cache=True):
            state = ctx.state(cache_layer)                   # [slots, dim]
            at = 0
            for n, slot in zip(ctx.q_lens, ctx.slot_list):
                s = state[slot].clone()
                for t in range(at, at + n):
                    s = self.decay * s + (1 - self.decay) * h[t].float()
                    residual[t] += (self.w.float() @ s)
                state[slot] = s
                at += n

    def build(cfg):
        d = cfg.dim
        emb = Embedding(cfg.vocab_size, d, {"table": "emb"})
        toy = PreNormBlock(RMSNorm(d, 1e-6, {"weight": "b0.n1"}), RunningMean(d, cfg.decay, {"w": "b0.mix"}),
                           RMSNorm(d, 1e-6, {"weight": "b0.n2"}), SwiGLU(d, 2 * d, {"w_gate": "b0.g", "w_up": "b0.u", "w_down": "b0.d"}))
        att = PreNormBlock(RMSNorm(d, 1e-6, {"weight": "b1.n1"}),
                           GQAAttention(d, 2, 1, d // 2, RotaryTable(d // 2, 10000.0),
                                        {k: "b1." + k for k in ("wq", "wk", "wv", "wo", "bq", "bk", "bv")}),
                           RMSNorm(d, 1e-6, {"weight": "b1.n2"}), SwiGLU(d, 2 * d, {"w_gate": "b1.g", "w_up": "b1.u", "w_down": "b1.d"}))
        return DecoderModel(emb, [toy, att], RMSNorm(d, 1e-6, {"weight": "fn"}), OutputHead(cfg.vocab_size, d, {}, tied_to=emb))

    register_architecture(["ToyStateForCausalLM"], ToyConfig, build)
    return ToyConfig


def toy_plain(W, tokens, d, decay):
    W = {k: v.double() for k, v in W.items()}
    x = W["emb"][tokens]
    h = plain.rms_norm(x, W["b0.n1"], 1e-6)
    s = torch.zeros(d, dtype=torch.float64)
    for t in range(len(tokens)):
        s = decay * s + (1 - decay) * h[t]
        x[t] = x[t] + W["b0.mix"] @ s
    x = x + plain.swiglu_ffn(plain.rms_norm(x, W["b0.n2"], 1e-6), W["b0.g"], W["b0.u"], W["b0.d"])
    h = plain.rms_norm(x, W["b1.n1"], 1e-6)
    dh = d // 2
    q = plain.linear(h, W["b1.wq"], W["b1.bq"]).reshape(-1, 2, dh)
    k = plain.linear(h, W["b1.wk"], W["b1.bk"]).reshape(-1, 1, dh)
    v = plain.linear(h, W["b1.wv"], W["b1.bv"]).reshape(-1, 1, dh)
    f = plain.rope_inv_freq(dh, 10000.0)
    pos = np.arange(len(tokens))
    a = plain.gqa_attention(plain.rope_neox(q, pos, f), plain.rope_neox(k, pos, f), v, dh ** -0.5)
    x = x + plain.linear(a.reshape(-1, 2 * dh), W["b1.wo"])
    x = x + plain.swiglu_ffn(plain.rms_norm(x, W["b1.n2"], 1e-6), W["b1.g"], W["b1.u"], W["b1.d"])
    return plain.linear(plain.rms_norm(x, W["fn"], 1e-6), W["emb"]).numpy()


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from boring_llm_b200 import load_config, registered_architectures, write_random_model
    from boring_llm_b200.config import unregister_architecture
    ToyConfig = define_toy()
    try:
        assert "ToyStateForCausalLM" in registered_architectures()
        cfg = ToyConfig("ToyStateForCausalLM", 61, 32, 0.75)
        d = str(tmp_path / "toy")
        write_random_model(d, cfg, 4, "float32", 0.25)
        assert load_config(d) == cfg                               # the model class is chosen by config.json
        W = plain.read_safetensors(d + "/model.safetensors")
        reqs = {f"t{i}": helpers.random_tokens(61, n, 40 + i) for i, n in enumerate([9, 30, 47, 21])}
        want = {rid: toy_plain(W, toks, 32, 0.75) for rid, toks in reqs.items()}
        # each request in changing portions, then all of them mixed with so few pages and slots that both are used again
        steps, n0 = [], 0
        for i, (rid, toks) in enumerate(reqs.items()):
            s = helpers.solo_trace(rid, toks, helpers.cut_varying(toks, i), n0)
            steps += s; n0 += len(s)
        outputs, runner = helpers.run_inprocess(d, "float32", steps, max_tokens=64)
        assert len(runner.cache.state_groups) == 1 and len(runner.cache.paged_groups) == 1
        rows = helpers.collect_rows(steps, outputs)
        for rid, w in want.items():
            helpers.assert_close(np.stack([rows[(rid, p)] for p in range(len(w))]), w, "float32", f"toy {rid} portions")
        steps, peak = helpers.mixed_trace(reqs, seed=2, max_live=3)
        outputs, runner = helpers.run_inprocess(d, "float32", steps, max_tokens=peak)
        rows = helpers.collect_rows(steps, outputs)
        for rid, w in want.items():
            helpers.assert_close(np.stack([rows[(rid, p)] for p in range(len(w))]), w, "float32", f"toy {rid} mixed")
    finally:
        unregister_architecture(["ToyStateForCausalLM"])
