"""The path that the benchmark times, at the benchmark's layer sizes, against the plain implementation.

A model with the layer sizes of Qwen2.5-0.5B (hidden 896, 14 query heads on 2 key/value heads of 64, feed-forward
4,864, vocabulary 151,936; two layers instead of 24) is built by the random-weights mode in device memory. At these
sizes the engine takes the kernels that the tiny test models never reach: the output head on tcgen05 with W as the
M side, gate/up on pairs of SMs at N = 9,728, the tcgen05 prefill attention above its token threshold, decode
attention cut into 16 slices (one cluster of blocks a request and head group) inside a captured graph, tokens fed back on the device one step ahead.

Random weights N(0, 0.02) give almost uniform attention, which would hide a lost key among two thousand. So two
tokens are planted in every prompt, one in the first page and one in the middle, and layer 0 is edited so that
every later query of key/value group 0 scores the first and every later query of group 1 scores the second about 14
above all other keys (a bias on one low-frequency dimension of q, a matching weight on k, an embedding row that
is one-hot): the attention output of every later token is then 99 % the value vector of a single far key. A kernel that
skips that key, reads a neighbour, merges the slices wrongly or takes the wrong page changes the logits wholesale; the
test measures that in the plain model itself (the same prompt without the planted token) and requires it to exceed
the tolerance it compares with by a factor of ten.
"""
import math

import numpy as np
import pytest
import torch

import helpers
import plain_model as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=896,
             num_attention_heads=14, num_key_value_heads=2, head_dim=64, intermediate_size=4864, vocab_size=151936,
             rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=32768)
X1, X2 = 11, 23                 # the planted tokens; prompts draw their other tokens from [100, vocab)
C1, C2 = 5, 6                   # the embedding columns that carry them
D1, D2 = 31, 30                 # dimensions of a head whose rotation pairs (31, 63), (30, 62) turn slowest
ALPHA, BETA = 0.5, 7.5          # score of a planted key: BETA * ALPHA * sqrt(896) / sqrt(64) = 14.0


def planted_tensors(cfg, seed, dtype):
    """The random model's tensors (made on the device by the product's random mode) with layer 0 edited."""
    from boring_llm_b200 import build_model
    from boring_llm_b200.weights import random_tensors
    specs = build_model(cfg).tensor_specs()
    lazy = random_tensors(specs, seed, dtype, 0.02, device=DEV)
    T = {n: lazy[n] for n in lazy}
    emb = T["model.embed_tokens.weight"]
    for tok, col in ((X1, C1), (X2, C2)):
        emb[tok] = 0
        emb[tok, col] = 1.0
    p = "model.layers.0."
    T[p + "input_layernorm.weight"][[C1, C2]] = 1.0
    T[p + "self_attn.k_proj.weight"][0 * 64 + D1, C1] = ALPHA       # key/value head 0 answers to X1
    T[p + "self_attn.k_proj.weight"][1 * 64 + D2, C2] = ALPHA       # key/value head 1 answers to X2
    bq = T[p + "self_attn.q_proj.bias"]
    for h in range(14):
        bq[h * 64 + (D1 if h < 7 else D2)] = BETA
    return T


def make_prompt(n, seed, at2):
    toks = (100 + np.random.default_rng(seed).integers(0, 151936 - 100, n)).tolist()
    toks[3], toks[at2] = X1, X2
    return toks


def plain_rows(cfg, T, tokens, rows, dtype):
    Wd = {k: v.double() for k, v in T.items()}                    # 64-bit, on the GPU: the oracle is plain, not slow
    stored = plain.round_bf16 if dtype == "bfloat16" else None
    return plain.forward(cfg.to_dict(), Wd, tokens, stored=stored, rows=rows).cpu().numpy()


def test_random_mode_makes_the_same_bits_on_the_device_as_in_a_folder(tmp_path):
    from boring_llm_b200 import Qwen2Config, build_model, write_random_model
    from boring_llm_b200.weights import random_tensors
    cfg = Qwen2Config.from_dict(helpers.TINY["B"])
    d = str(tmp_path / "m")
    write_random_model(d, cfg, 3, "bfloat16", 0.02)               # made on the CPU
    _, W = plain.read_model_folder(d)
    mem = random_tensors(build_model(cfg).tensor_specs(), 3, torch.bfloat16, 0.02, device=DEV)
    assert sorted(mem) == sorted(W)
    for n in mem:
        assert mem[n].is_cuda and torch.equal(mem[n].cpu().float(), W[n].float()), n
    from boring_llm_b200.weights import TensorSpec
    spec = {"w": TensorSpec((3000, 3001))}                        # several chunks of the generator
    big = random_tensors(spec, 1, torch.float32, 1.0, device=DEV)["w"]
    cpu = random_tensors(spec, 1, torch.float32, 1.0)["w"]
    assert torch.equal(big.cpu(), cpu)


def test_bfloat16_benchmarked_path_equals_the_plain_implementation():
    from boring_llm_b200 import EngineOptions, Qwen2Config, build_model
    from boring_llm_b200.engine import Engine, StepEntry
    from boring_llm_b200.kernels import ops
    cfg = Qwen2Config.from_dict(SIZES)
    T = planted_tensors(cfg, 0, torch.bfloat16)
    model = build_model(cfg)
    model.load(T, torch.bfloat16, torch.device(DEV))
    opts = EngineOptions(dtype="bfloat16", ctx_size=4096, max_num_seqs=4, max_tokens=4 * 4096,
                         max_num_batched_tokens=2304, prefill_chunk=2304)
    eng = Engine.from_model(cfg, model, opts)
    used = set()
    real_call = ops._call
    ops._call = lambda fn, *a: (used.add(fn.__name__), real_call(fn, *a))[1]
    try:
        # (a) one prefill step of 2,100 tokens: logits of 32 rows, the last among them
        prompt = make_prompt(2100, 1, 1037)
        rows = sorted(set(np.linspace(4, 2099, 31).astype(int).tolist() + [1038, 2099]))
        got = eng.runner.step([StepEntry("whole", prompt, rows)]).float().cpu().numpy()
        eng.runner.check_kernels()
        eng.runner.free_request("whole")
        want = plain_rows(cfg, T, prompt, rows, "bfloat16")
        scale = np.abs(want).max()
        err = np.abs(got - want)
        print(f"prefill: scale {scale:.3f} max err {err.max():.4f} ({err.max() / scale:.2e}) mean {err.mean() / scale:.2e}")
        helpers.assert_close(got, want, "bfloat16", "prefill of 2,100 tokens", tol=1.5e-2, mean_tol=1.5e-3)
        # what a lost key costs: the same prompt without the planted tokens, in the plain model
        for tok_at in (3, 1037):
            other = list(prompt)
            other[tok_at] = 99
            lost = plain_rows(cfg, T, other, rows[-1:], "bfloat16")
            effect = np.abs(lost - want[-1:]).max() / scale
            print(f"without the planted token at {tok_at}: the last row moves by {effect:.2f} of the scale")
            assert effect > 10 * 1.5e-2, f"the planted key at {tok_at} does not show in the logits ({effect:.3f})"
        # (b) three requests through the engine: chunked and mixed prefill, then 40 decode steps in captured graphs,
        # launched one ahead, the decode attention in 16 slices
        prompts = [make_prompt(2100, 2, 1500), make_prompt(1500, 3, 700), make_prompt(700, 4, 350)]
        outs = eng.generate(prompts, n_predict=40, ignore_eos=True)
    finally:
        ops._call = real_call
    assert eng.runner.graph_steps >= 30
    for name in ("bl_gemm_tc_cols", "bl_gemm_tc_pair", "bl_attention_prefill_tc", "bl_attention_decode_tma",
                 "bl_norm_qkv_rope", "bl_gemm_skinny_residual_norm", "bl_gemm_skinny_scaled", "bl_gemm_skinny"):
        assert name in used, f"{name} was not on the path"
    check_tokens(cfg, T, prompts, outs)
    # the same with every step in turn and no captured graph (other slice counts in the decode attention)
    slow = Engine.from_model(cfg, model, EngineOptions(dtype="bfloat16", ctx_size=4096, max_num_seqs=4, max_tokens=4 * 4096,
                                                       max_num_batched_tokens=2304, prefill_chunk=2304,
                                                       cuda_graphs=False, lookahead=False))
    check_tokens(cfg, T, prompts, slow.generate(prompts, n_predict=40, ignore_eos=True))


def check_tokens(cfg, T, prompts, outs, tol=1.5e-2):
    """Every generated token is the plain implementation's arg-max given the engine's own prefix, or within the
    logits' tolerance of it."""
    for p, o in zip(prompts, outs):
        assert len(o) == 40
        logits = plain_rows(cfg, T, p + o, list(range(len(p) - 1, len(p) + 39)), "bfloat16")
        scale = np.abs(logits).max()
        for i, tok in enumerate(o):
            best = int(np.argmax(logits[i]))
            if tok != best:
                gap = logits[i][best] - logits[i][tok]
                assert gap <= 2 * tol * scale, f"token {i}: engine chose {tok}, plain {best} (gap {gap:.3e}, scale {scale:.3f})"


def test_float32_path_at_the_benchmark_sizes():
    from boring_llm_b200 import EngineOptions, Qwen2Config, build_model
    from boring_llm_b200.engine import Engine, StepEntry
    cfg = Qwen2Config.from_dict(SIZES)
    T = planted_tensors(cfg, 0, torch.float32)
    model = build_model(cfg)
    model.load(T, torch.float32, torch.device(DEV))
    eng = Engine.from_model(cfg, model, EngineOptions(dtype="float32", ctx_size=1024, max_num_seqs=2, max_tokens=2048,
                                                      max_num_batched_tokens=512, prefill_chunk=512))
    prompt = make_prompt(300, 5, 150)
    rows = sorted(set(np.linspace(4, 299, 15).astype(int).tolist() + [299]))
    got = eng.runner.step([StepEntry("whole", prompt, rows)]).float().cpu().numpy()
    eng.runner.free_request("whole")
    want = plain_rows(cfg, T, prompt, rows, "float32")
    helpers.assert_close(got, want, "float32", "float32 prefill of 300 tokens")
    out = eng.generate([prompt], n_predict=12, ignore_eos=True)[0]
    logits = plain_rows(cfg, T, prompt + out, list(range(299, 299 + 12)), "float32")
    assert out == [int(np.argmax(r)) for r in logits]
