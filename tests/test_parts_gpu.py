"""Each part alone, through the real step machinery, against the plain implementation's function for it."""
import math

import numpy as np
import pytest
import torch

import plain_model as plain
from part_harness import run_portions, runner_for

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 2e-2}


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    scale = max(want.abs().max().item(), 1e-6)
    err = (got - want).abs().max().item()
    assert err <= TOL[dtype] * scale, f"{what}: max |diff| {err:.3e} > {TOL[dtype]:.0e} * {scale:.3f}"


def rand(shape, seed, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from boring_llm_b200.parts import RMSNorm
    d = 70
    part = RMSNorm(d, 3e-5, {"weight": "n.w"})
    w = rand((d,), 1, 0.2, DT[dtype]) + 1
    part.load({"n.w": w}, DT[dtype], DEV)
    x = rand((11, d), 2, 2.0).to(DEV)
    r = runner_for(x, lambda ctx, h: part.forward(ctx, h), dtype=dtype)
    got = run_portions(r, "a", 11, [11])
    close(got, plain.rms_norm(x.double().cpu(), w.double(), 3e-5), dtype)
    assert got.dtype == DT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_output_head_parts(dtype):
    from boring_llm_b200.parts import Embedding, OutputHead
    V, d = 37, 24
    emb = Embedding(V, d, {"table": "e"})
    table = rand((V, d), 3, 0.5, DT[dtype])
    emb.load({"e": table}, DT[dtype], DEV)
    tied = OutputHead(V, d, {}, tied_to=emb)
    tied.load({}, DT[dtype], DEV)
    sep = OutputHead(V, d, {"weight": "h"})
    hw = rand((V, d), 4, 0.5, DT[dtype])
    sep.load({"h": hw}, DT[dtype], DEV)
    assert tied.tensor_specs() == {} and list(sep.tensor_specs()) == ["h"]
    assert tied.matrix().data_ptr() == emb.table.data_ptr()        # shared, not copied

    def body(ctx, x):
        e = emb.forward(ctx)
        y = e.to(DT[dtype])
        return torch.cat([e, tied.forward(ctx, y), sep.forward(ctx, y)], dim=1)

    r = runner_for(torch.zeros(V, 1, device=DEV), body, dtype=dtype)
    out = run_portions(r, "a", V, [V])          # token ids 0..V-1
    e_ref = table.double()
    assert torch.equal(out[:, :d].cpu(), table.float())
    close(out[:, d:d + V], e_ref @ e_ref.T, dtype, "tied head")
    close(out[:, d + V:], e_ref @ hw.double().T, dtype, "separate head")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_part(dtype):
    from boring_llm_b200.parts import SwiGLU
    d, F = 48, 100
    part = SwiGLU(d, F, {"w_gate": "g", "w_up": "u", "w_down": "d"})
    W = {"g": rand((F, d), 5, 0.3, DT[dtype]), "u": rand((F, d), 6, 0.3, DT[dtype]), "d": rand((d, F), 7, 0.3, DT[dtype])}
    part.load(W, DT[dtype], DEV)
    x = rand((9, d), 8).to(DEV)

    def body(ctx, h):
        res = h.clone()
        part.forward(ctx, h.to(DT[dtype]), res)
        return res

    r = runner_for(x, body, dtype=dtype)
    got = run_portions(r, "a", 9, [4, 5])
    xin = x.to(DT[dtype]).double().cpu()
    want = x.double().cpu() + plain.swiglu_ffn(xin, W["g"].double(), W["u"].double(), W["d"].double())
    close(got, want, dtype)


def attention_reference(x, W, H, KV, dh, theta, window, scale=None):
    seq = x.shape[0]
    q = plain.linear(x, W["q"], W.get("bq")).reshape(seq, H, dh)
    k = plain.linear(x, W["k"], W.get("bk")).reshape(seq, KV, dh)
    v = plain.linear(x, W["v"], W.get("bv")).reshape(seq, KV, dh)
    f = plain.rope_inv_freq(dh, theta)
    pos = np.arange(seq)
    q, k = plain.rope_neox(q, pos, f), plain.rope_neox(k, pos, f)
    a = plain.gqa_attention(q, k, v, scale if scale is not None else 1 / math.sqrt(dh), window)
    return plain.linear(a.reshape(seq, H * dh), W["o"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,dh,bias,window", [(4, 2, 16, True, 0), (3, 1, 32, True, 0), (5, 5, 48, False, 20),
                                                  (7, 1, 64, True, 0), (2, 2, 128, True, 33)])
def test_attention_part_whole_and_in_portions(dtype, H, KV, dh, bias, window):
    from boring_llm_b200.parts import GQAAttention, RotaryTable
    d, theta, n = 40, 50000.0, 75
    names = {k: k for k in ("wq", "wk", "wv", "wo", "bq", "bk", "bv")}
    part = GQAAttention(d, H, KV, dh, RotaryTable(dh, theta), names, qkv_bias=bias, window=window)
    std = 0.6 / math.sqrt(dh) * 2
    W = {"wq": rand((H * dh, d), 1, std, DT[dtype]), "wk": rand((KV * dh, d), 2, std, DT[dtype]),
         "wv": rand((KV * dh, d), 3, 0.2, DT[dtype]), "wo": rand((d, H * dh), 4, 0.2, DT[dtype])}
    if bias:
        W.update({"bq": rand((H * dh,), 5, 0.1, DT[dtype]), "bk": rand((KV * dh,), 6, 0.1, DT[dtype]),
                  "bv": rand((KV * dh,), 7, 0.1, DT[dtype])})
    part.load(W, DT[dtype], DEV)
    x = rand((n, d), 9).to(DEV)

    def body(ctx, h):
        res = torch.zeros_like(h)
        part.forward(ctx, h.to(DT[dtype]), res, 0, True)
        return res

    Wd = {k[1:] if k[0] == "w" else k: v.double() for k, v in W.items()}
    want = attention_reference(x.to(DT[dtype]).double().cpu(), Wd, H, KV, dh, theta, window)
    r = runner_for(x, body, [part.cache_spec()], dtype=dtype, max_tokens=96)
    whole = run_portions(r, "a", n, [n])
    close(whole, want, dtype, "whole")
    cut = run_portions(r, "b", n, [2, 31, 1, 17, 2, 1, 1, 20])        # pages of request a are used again
    close(cut, want, dtype, "portions")
    if dtype == "float32":
        assert torch.equal(whole, cut)                   # the 32-bit path computes a position the same way however the work is cut
    r.cache.check()
    # the same part with a bias on its output projection (read per file in the reference, src/model.br:500, 1328):
    # the residual stream gets the product plus the bias
    with_bias = GQAAttention(d, H, KV, dh, RotaryTable(dh, theta), dict(names, bo="bo"), qkv_bias=bias, out_bias=True, window=window)
    assert "bo" in with_bias.local_specs() and "bo" not in part.local_specs()
    bo = rand((d,), 11, 0.3, DT[dtype])
    with_bias.load(dict(W, bo=bo), DT[dtype], DEV)

    def body_bias(ctx, h):
        res = torch.zeros_like(h)
        with_bias.forward(ctx, h.to(DT[dtype]), res, 0, True)
        return res
    r2 = runner_for(x, body_bias, [with_bias.cache_spec()], dtype=dtype, max_tokens=96)
    close(run_portions(r2, "c", n, [40, 1, 34]), want + bo.double().cpu(), dtype, "with an output bias")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part_and_a_run_order_that_repeats_and_shares(dtype):
    """A pre-norm block equals norm -> attention -> add -> norm -> SwiGLU -> add; a run order may name a
    block twice and let an entry read the cache another entry wrote."""
    from boring_llm_b200.parts import (DecoderModel, Embedding, GQAAttention, LayerCall, OutputHead, PreNormBlock,
                                       RMSNorm, RotaryTable, SwiGLU)
    from boring_llm_b200.weights import random_tensors
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine.runner import ModelRunner, StepEntry
    d, H, KV, dh, F, V = 32, 2, 1, 16, 56, 50

    def block(i):
        p = f"l{i}."
        return PreNormBlock(
            RMSNorm(d, 1e-6, {"weight": p + "n1"}),
            GQAAttention(d, H, KV, dh, RotaryTable(dh, 10000.0),
                         {k: p + k for k in ("wq", "wk", "wv", "wo", "bq", "bk", "bv")}),
            RMSNorm(d, 1e-6, {"weight": p + "n2"}),
            SwiGLU(d, F, {"w_gate": p + "g", "w_up": p + "u", "w_down": p + "dn"}))

    emb = Embedding(V, d, {"table": "emb"})
    # block 0 runs twice (second time on its own cache layer), block 1 reads block 0's first cache
    order = [LayerCall(0, 0), LayerCall(1, 0, write_cache=False), LayerCall(0, 1)]
    model = DecoderModel(emb, [block(0), block(1)], RMSNorm(d, 1e-6, {"weight": "fn"}), OutputHead(V, d, {}, tied_to=emb),
                         schedule=order)
    assert len(model.cache_specs()) == 2
    T = random_tensors(model.tensor_specs(), 3, DT[dtype], 0.25)
    model.load(T, DT[dtype], DEV)
    tokens = list(np.random.default_rng(0).integers(0, V, 40))

    # plain restatement of the same run order
    Wd = {k: v.double() for k, v in T.items()}
    x = Wd["emb"][tokens]
    pos = np.arange(len(tokens)); f = plain.rope_inv_freq(dh, 10000.0)

    def qkv(p, h):
        q = plain.linear(h, Wd[p + "wq"], Wd[p + "bq"]).reshape(-1, H, dh)
        k = plain.linear(h, Wd[p + "wk"], Wd[p + "bk"]).reshape(-1, KV, dh)
        v = plain.linear(h, Wd[p + "wv"], Wd[p + "bv"]).reshape(-1, KV, dh)
        return plain.rope_neox(q, pos, f), plain.rope_neox(k, pos, f), v

    st = plain.round_bf16 if dtype == "bfloat16" else (lambda t: t)     # what a bfloat16 engine stores between kernels
    caches = {}
    for call in order:
        p = f"l{call.block}."
        h = st(plain.rms_norm(x, Wd[p + "n1"], 1e-6))
        q, k, v = (st(t) for t in qkv(p, h))
        if call.write_cache:
            caches[call.cache] = (k, v)
        k, v = caches[call.cache]
        a = st(plain.gqa_attention(q, k, v, 1 / math.sqrt(dh)))
        x = x + plain.linear(a.reshape(-1, H * dh), Wd[p + "wo"])
        h = st(plain.rms_norm(x, Wd[p + "n2"], 1e-6))
        act = st(plain.silu(plain.linear(h, Wd[p + "g"])) * plain.linear(h, Wd[p + "u"]))
        x = x + plain.linear(act, Wd[p + "dn"])
    want = plain.linear(st(plain.rms_norm(x, Wd["fn"], 1e-6)), Wd["emb"])

    opts = EngineOptions(dtype=dtype, max_tokens=64, ctx_size=64, max_num_seqs=2, cuda_graphs=False)
    runner = ModelRunner(model, opts)
    got = runner.step([StepEntry("a", tokens, list(range(len(tokens))))])
    close(got, want, dtype, "whole")
    runner.free_request("a")
    parts = [runner.step([StepEntry("b", tokens[:23], list(range(23)))]),
             runner.step([StepEntry("b", tokens[23:], list(range(17)))])]
    close(torch.cat(parts), want, dtype, "two portions")

    with pytest.raises(ValueError, match="before any entry writes"):
        DecoderModel(emb, [block(0)], RMSNorm(d, 1e-6, {"weight": "fn"}), OutputHead(V, d, {}, tied_to=emb),
                     schedule=[LayerCall(0, 0, write_cache=False)])
    with pytest.raises(ValueError, match="written by two"):
        DecoderModel(emb, [block(0)], RMSNorm(d, 1e-6, {"weight": "fn"}), OutputHead(V, d, {}, tied_to=emb),
                     schedule=[LayerCall(0, 0), LayerCall(0, 0)])
