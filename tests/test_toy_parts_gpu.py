"""More toy parts defined HERE, outside the framework, to show what the part interfaces carry: a feed-forward
with routing (top-2 of four small experts), another position encoding (learned absolute positions added by a
custom embedding part, with attention that rotates nothing), and a run order that names a block twice (the second
visit reads the cache the first one wrote). Registered, written as a random model folder, loaded through
config.json and stepped in portions and mixed batches without a change to the framework's files. Test fixtures,
not models of anyone's."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_model as plain

pytestmark = pytest.mark.gpu

ARCH = "ToyRoutedForCausalLM"
EXPERTS, TOP = 4, 2


def define_toy():
    from boring_llm_b200.config import register_architecture
    from boring_llm_b200.parts import (DecoderModel, Embedding, FeedForward, GQAAttention, LayerCall, OutputHead,
                                       PreNormBlock, RMSNorm, RotaryTable, SwiGLU)
    from boring_llm_b200.weights import TensorSpec, MATRIX

    @dataclass(frozen=True)
    class ToyConfig:
        architecture: str
        vocab_size: int
        dim: int
        max_position_embeddings: int = 128

        @classmethod
        def from_dict(cls, d):
            return cls(d["architectures"][0], d["vocab_size"], d["dim"], d["max_position_embeddings"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "dim": self.dim,
                    "max_position_embeddings": self.max_position_embeddings}

    class LearnedPositions(Embedding):
        """x[t] = table[token[t]] + pos[position[t]]: a position encoding that lives in the embedding part."""

        def __init__(self, vocab, dim, max_pos, names):
            super().__init__(vocab, dim, names)
            self.max_pos = max_pos

        def local_specs(self):
            return dict(super().local_specs(), pos=TensorSpec((self.max_pos, self.dim), MATRIX))

        def place(self, local, dtype, device):
            super().place(local, dtype, device)
            self.pos = local["pos"].to(device=device, dtype=torch.float32)

        def forward(self, ctx):
            x = super().forward(ctx)
            x += self.pos[ctx.positions.long()]
            return x

    class RoutedFF(FeedForward):
        """Each token goes to its TOP experts by router logit (32-bit), weighted by the softmax over those logits;
        an expert is down(relu(up(h)))."""

        def __init__(self, dim, hidden, names):
            super().__init__(names)
            self.dim, self.hidden = dim, hidden

        def local_specs(self):
            return {"router": TensorSpec((EXPERTS, self.dim), MATRIX),
                    "up": TensorSpec((EXPERTS, self.hidden, self.dim), MATRIX),
                    "down": TensorSpec((EXPERTS, self.dim, self.hidden), MATRIX)}

        def forward(self, ctx, h, residual):
            hf = h.float()
            logits = hf @ self.router.float().T                                  # [T, E]
            top_v, top_i = torch.topk(logits, TOP, dim=-1)
            gate = torch.softmax(top_v, dim=-1)
            for e in range(EXPERTS):
                w = (gate * (top_i == e)).sum(-1, keepdim=True)                  # 0 for tokens that skip this expert
                residual += w * (torch.relu(hf @ self.up[e].float().T) @ self.down[e].float().T)

    def build(cfg):
        d = cfg.dim
        emb = LearnedPositions(cfg.vocab_size, d, cfg.max_position_embeddings, {"table": "emb", "pos": "pos"})

        def attention(prefix):
            return GQAAttention(d, 2, 2, d // 2, RotaryTable(d // 2, 10000.0, n_rot=0),       # rotates nothing
                                {k: prefix + k for k in ("wq", "wk", "wv", "wo", "bq", "bk", "bv")})
        routed = PreNormBlock(RMSNorm(d, 1e-6, {"weight": "b0.n1"}), attention("b0."),
                              RMSNorm(d, 1e-6, {"weight": "b0.n2"}), RoutedFF(d, 2 * d, {"router": "b0.r", "up": "b0.u", "down": "b0.d"}))
        dense = PreNormBlock(RMSNorm(d, 1e-6, {"weight": "b1.n1"}), attention("b1."),
                             RMSNorm(d, 1e-6, {"weight": "b1.n2"}), SwiGLU(d, 2 * d, {"w_gate": "b1.g", "w_up": "b1.u", "w_down": "b1.d"}))
        # block 0 runs twice: its second visit attends over the keys and values its first visit cached
        order = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 0, write_cache=False)]
        return DecoderModel(emb, [routed, dense], RMSNorm(d, 1e-6, {"weight": "fn"}),
                            OutputHead(cfg.vocab_size, d, {}, tied_to=emb), schedule=order)

    register_architecture([ARCH], ToyConfig, build)
    return ToyConfig


def toy_plain(W, tokens, d):
    W = {k: v.double() for k, v in W.items()}
    n, dh = len(tokens), d // 2
    x = W["emb"][tokens] + W["pos"][:n]

    def project(h, p):
        q = plain.linear(h, W[p + "wq"], W[p + "bq"]).reshape(n, 2, dh)
        k = plain.linear(h, W[p + "wk"], W[p + "bk"]).reshape(n, 2, dh)
        v = plain.linear(h, W[p + "wv"], W[p + "bv"]).reshape(n, 2, dh)
        return q, k, v

    def routed_ff(h):
        logits = h @ W["b0.r"].T
        top_v, top_i = torch.topk(logits, TOP, dim=-1)
        gate = torch.softmax(top_v, dim=-1)
        out = torch.zeros_like(h)
        for e in range(EXPERTS):
            w = (gate * (top_i == e)).sum(-1, keepdim=True)
            out += w * (torch.relu(h @ W["b0.u"][e].T) @ W["b0.d"][e].T)
        return out

    # first visit of block 0: its keys and values are the cache of layer 0
    q, k0, v0 = project(plain.rms_norm(x, W["b0.n1"], 1e-6), "b0.")
    x = x + plain.linear(plain.gqa_attention(q, k0, v0, dh ** -0.5).reshape(n, d), W["b0.wo"])
    x = x + routed_ff(plain.rms_norm(x, W["b0.n2"], 1e-6))
    q, k, v = project(plain.rms_norm(x, W["b1.n1"], 1e-6), "b1.")
    x = x + plain.linear(plain.gqa_attention(q, k, v, dh ** -0.5).reshape(n, d), W["b1.wo"])
    x = x + plain.swiglu_ffn(plain.rms_norm(x, W["b1.n2"], 1e-6), W["b1.g"], W["b1.u"], W["b1.d"])
    # second visit of block 0: new queries over the cached keys and values of the first visit
    q, _, _ = project(plain.rms_norm(x, W["b0.n1"], 1e-6), "b0.")
    x = x + plain.linear(plain.gqa_attention(q, k0, v0, dh ** -0.5).reshape(n, d), W["b0.wo"])
    x = x + routed_ff(plain.rms_norm(x, W["b0.n2"], 1e-6))
    return plain.linear(plain.rms_norm(x, W["fn"], 1e-6), W["emb"]).numpy()


def test_routing_learned_positions_and_a_block_visited_twice(tmp_path):
    from boring_llm_b200 import load_config, write_random_model
    from boring_llm_b200.config import unregister_architecture
    ToyConfig = define_toy()
    try:
        cfg = ToyConfig(ARCH, 53, 32, 128)
        d = str(tmp_path / "toy")
        write_random_model(d, cfg, 6, "float32", 0.25)
        assert load_config(d) == cfg
        W = plain.read_safetensors(d + "/model.safetensors")
        reqs = {f"r{i}": helpers.random_tokens(53, n, 70 + i) for i, n in enumerate([5, 26, 40, 17])}
        want = {rid: toy_plain(W, toks, 32) for rid, toks in reqs.items()}
        steps, n0 = [], 0
        for i, (rid, toks) in enumerate(reqs.items()):
            s = helpers.solo_trace(rid, toks, helpers.cut_varying(toks, 3 + i), n0)
            steps += s; n0 += len(s)
        outputs, runner = helpers.run_inprocess(d, "float32", steps, max_tokens=64)
        assert len(runner.cache.paged_groups) == 1 and len(runner.cache.paged_groups[0].cache_layers) == 2
        rows = helpers.collect_rows(steps, outputs)
        for rid, w in want.items():
            helpers.assert_close(np.stack([rows[(rid, p)] for p in range(len(w))]), w, "float32", f"toy {rid} portions")
        steps, peak = helpers.mixed_trace(reqs, seed=4, max_live=3)
        outputs, runner = helpers.run_inprocess(d, "float32", steps, max_tokens=peak)
        rows = helpers.collect_rows(steps, outputs)
        for rid, w in want.items():
            helpers.assert_close(np.stack([rows[(rid, p)] for p in range(len(w))]), w, "float32", f"toy {rid} mixed")
    finally:
        unregister_architecture([ARCH])


# ---- a rotary encoding that turns neighbouring dimensions (2j, 2j + 1) together, on part of each head ------------
ARCH_PAIRS = "ToyInterleavedForCausalLM"


def rope_interleaved(x, positions, inv_freq, n_rot):
    """src/math.br:128-157 with neox == 0: pair j = (2j, 2j + 1) for the first n_rot dimensions of each head."""
    ang = torch.from_numpy((positions.astype(np.float32)[:, None] * inv_freq[None, :n_rot // 2]).astype(np.float64))
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
    out[..., 0:n_rot:2] = a * c - b * s
    out[..., 1:n_rot:2] = a * s + b * c
    return out


@pytest.mark.parametrize("dtype,n_rot", [("float32", 16), ("float32", 32), ("bfloat16", 32), ("bfloat16", 16)])
def test_rotary_positions_on_interleaved_pairs(tmp_path, dtype, n_rot):
    """The same attention part with another pair layout (and, for n_rot 16, only half of each head rotated): nothing
    but the `RotaryTable` differs. With full rotation the bfloat16 engine takes the fused q/k/v kernel for steps
    of few rows, so both kernels that rotate are covered."""
    from dataclasses import dataclass as dc
    from boring_llm_b200 import write_random_model
    from boring_llm_b200.config import register_architecture, unregister_architecture
    from boring_llm_b200.parts import (DecoderModel, Embedding, GQAAttention, OutputHead, PreNormBlock, RMSNorm,
                                       RotaryTable, SwiGLU)
    d, H, KV, dh, F, V, theta = 64, 4, 2, 32, 96, 61, 10000.0

    @dc(frozen=True)
    class Cfg:
        architecture: str
        vocab_size: int
        max_position_embeddings: int = 256

        @classmethod
        def from_dict(cls, c):
            return cls(c["architectures"][0], c["vocab_size"], c["max_position_embeddings"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "max_position_embeddings": self.max_position_embeddings}

    def build(cfg):
        emb = Embedding(cfg.vocab_size, d, {"table": "emb"})
        blocks = [PreNormBlock(
            RMSNorm(d, 1e-6, {"weight": f"b{i}.n1"}),
            GQAAttention(d, H, KV, dh, RotaryTable(dh, theta, n_rot=n_rot, pairs="interleaved"),
                         {k: f"b{i}." + k for k in ("wq", "wk", "wv", "wo", "bq", "bk", "bv")}),
            RMSNorm(d, 1e-6, {"weight": f"b{i}.n2"}),
            SwiGLU(d, F, {"w_gate": f"b{i}.g", "w_up": f"b{i}.u", "w_down": f"b{i}.d"})) for i in range(2)]
        return DecoderModel(emb, blocks, RMSNorm(d, 1e-6, {"weight": "fn"}), OutputHead(cfg.vocab_size, d, {}, tied_to=emb))

    def toy_forward(W, tokens):
        st = plain.round_bf16 if dtype == "bfloat16" else (lambda t: t)
        W = {k: v.double() for k, v in W.items()}
        n = len(tokens)
        pos = np.arange(n)
        j = np.arange(n_rot // 2, dtype=np.float32)
        inv = np.float32(1.0) / np.power(np.float32(theta), (np.float32(2.0) * j) / np.float32(n_rot), dtype=np.float32)
        x = W["emb"][tokens]
        for i in range(2):
            p = f"b{i}."
            h = st(plain.rms_norm(x, W[p + "n1"], 1e-6))
            q = st(rope_interleaved(plain.linear(h, W[p + "wq"], W[p + "bq"]).reshape(n, H, dh), pos, inv, n_rot))
            k = st(rope_interleaved(plain.linear(h, W[p + "wk"], W[p + "bk"]).reshape(n, KV, dh), pos, inv, n_rot))
            v = st(plain.linear(h, W[p + "wv"], W[p + "bv"]).reshape(n, KV, dh))
            a = st(plain.gqa_attention(q, k, v, dh ** -0.5, 0, st if dtype == "bfloat16" else None))
            x = x + plain.linear(a.reshape(n, H * dh), W[p + "wo"])
            h = st(plain.rms_norm(x, W[p + "n2"], 1e-6))
            x = x + plain.linear(st(plain.silu(plain.linear(h, W[p + "g"])) * plain.linear(h, W[p + "u"])), W[p + "d"])
        return plain.linear(st(plain.rms_norm(x, W["fn"], 1e-6)), W["emb"]).numpy()

    register_architecture([ARCH_PAIRS], Cfg, build)
    try:
        folder = str(tmp_path / "toy")
        write_random_model(folder, Cfg(ARCH_PAIRS, V), 8, dtype, 0.25)
        W = plain.read_safetensors(folder + "/model.safetensors")
        reqs = {f"r{i}": helpers.random_tokens(V, n, 90 + i) for i, n in enumerate([9, 70, 33])}
        want = {rid: toy_forward(W, toks) for rid, toks in reqs.items()}
        steps, peak = helpers.mixed_trace(reqs, seed=6, max_live=3)
        outputs, _ = helpers.run_inprocess(folder, dtype, steps, max_tokens=peak, step_graph_after=1)
        rows = helpers.collect_rows(steps, outputs)
        for rid, w in want.items():
            helpers.assert_close(np.stack([rows[(rid, p)] for p in range(len(w))]), w, dtype, f"interleaved pairs {rid}")
        # the other layout must NOT fit: the comparison can tell the layouts apart
        other = plain.forward  # noqa: F841  (the halves layout is what plain_model implements; a direct check follows)
        x = torch.randn(5, 2, dh, dtype=torch.float64)
        inv_full = plain.rope_inv_freq(dh, theta)
        assert not torch.allclose(rope_interleaved(x, np.arange(5), inv_full, dh), plain.rope_neox(x, np.arange(5), inv_full))
    finally:
        unregister_architecture([ARCH_PAIRS])
