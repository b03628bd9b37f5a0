"""Shared by the tests: the tiny configurations, trace builders, the replay driver and tolerances."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Tiny configurations of the architecture that differ in every size and option. A and B have the layer sizes of the
# benchmark description's two tiny configurations (2 layers / hidden 64 / 4:2 heads of 16 / feed-forward 128 / vocabulary
# 256 / theta 1e4 / eps 1e-6 / tied; 3 layers / 96 / 3:1 heads of 32 / 200 / 320 / theta 1e6 / eps 1e-5 / separate head);
# they differ from it in two things, on purpose: max_position_embeddings is 512 instead of 128 / 256, so that the
# replay traces can hold prompts of several pages plus 300 decoded tokens, and the replay tests draw weights with
# std 0.25 instead of 0.02, which makes attention sharp enough for a lost key to show (the generation tests and the
# tests against the pure 64-bit implementation use the description's 0.02; its workloads, prompts of 7 / 16 / 33 tokens
# with 8 greedy tokens and prompts of 1 / 5 / 19 / 64 tokens in portions of 8 with 12 tokens at temperature 0 and 0.8,
# are those of tests/test_generate_gpu.py).
TINY = {
    # 2 layers, 4 heads in 2 groups, head 16, tied output head, theta 1e4, eps 1e-6, no window
    "A": dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512,
              use_sliding_window=False),
    # 3 layers, 3 heads on 1 key/value head, head 32, separate output head, theta 1e6, eps 1e-5,
    # widths that are no power of two
    "B": dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=3, num_key_value_heads=1, intermediate_size=200, vocab_size=320,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512),
    # 3 layers, 5 heads each with its own key/value head, head 48 (hidden != heads * head), odd
    # vocabulary, a window of 20 positions (no multiple of the page size) on the last two layers
    "C": dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3, hidden_size=80,
              num_attention_heads=5, num_key_value_heads=5, head_dim=48, intermediate_size=176, vocab_size=211,
              rope_theta=500000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=512,
              use_sliding_window=True, sliding_window=20, max_window_layers=1),
    # 2 layers, head 64 (the head size of the tcgen05 prefill attention), 4 heads in 2 groups, hidden != heads * head,
    # a window of 150 positions (more than one key block of 128) on the second layer
    "D": dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=128,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=192, vocab_size=300,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=1024,
              use_sliding_window=True, sliding_window=150, max_window_layers=1),
}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3}

# Largest allowed |engine - plain| as a fraction of the largest |plain logit| of the compared rows.
# float32: every product is a 32-bit FMA chain of a few hundred terms through a few layers (about 1e3 ulps
# of headroom); bfloat16: activations are rounded to 8 bits of mantissa at every kernel boundary.
# The plain side rounds what a bfloat16 engine stores, but it cannot reproduce the tensor cores' rounding of
# the softmax numerators block by block (they are rounded against a running maximum); with the sharp attention
# of the test models that independent 2^-9 noise is amplified by the next layers' softmax to a few percent.
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
MEAN_TOL = {"float32": 2e-5, "bfloat16": 8e-3}
# bfloat16 engine against the PURE 64-bit plain implementation (no rounding of stored tensors on the plain
# side): only meaningful for well-conditioned models, i.e. the benchmark's N(0, 0.02) weights
TOL_PURE_BF16 = 4e-2


def write_tiny_model(path, name, dtype="float32", std=0.25, seed=None):
    from boring_llm_b200 import Qwen2Config, write_random_model
    cfg = Qwen2Config.from_dict(TINY[name])
    write_random_model(path, cfg, SEEDS[name] if seed is None else seed, dtype, std)
    return cfg


def plain_logits(model_dir, tokens, dtype="float32"):
    """float64 logits of every position from the plain implementation. For a bfloat16 engine the
    plain side rounds what such an engine stores between kernels (see plain_model.forward)."""
    import plain_model
    cfg, W = plain_model.read_model_folder(model_dir)
    stored = plain_model.round_bf16 if dtype == "bfloat16" else None
    return plain_model.forward(cfg, W, tokens, stored=stored).numpy()


def random_tokens(vocab, n, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def assert_close(got, want, dtype, what="", tol=None, mean_tol=None):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(np.abs(want).max(), 1e-6)
    err = np.abs(got - want)
    worst = np.unravel_index(np.argmax(err), err.shape)
    tol = TOL[dtype] if tol is None else tol
    assert err.max() <= tol * scale, (
        f"{what}: max |diff| {err.max():.3e} at {worst} exceeds {tol:.0e} * {scale:.3f}")
    if mean_tol is None:
        mean_tol = MEAN_TOL[dtype]
    assert err.mean() <= mean_tol * scale, (
        f"{what}: mean |diff| {err.mean():.3e} exceeds {mean_tol:.0e} * {scale:.3f}")


# ---- traces ------------------------------------------------------------------------------------------
def cut_whole(tokens):
    return [len(tokens)]


def cut_tail_singly(tokens, tail=32):
    tail = min(tail, len(tokens) - 1)
    return [len(tokens) - tail] + [1] * tail if tail > 0 else [len(tokens)]


def cut_varying(tokens, seed):
    """Portions of changing size, many of them of two tokens."""
    rng = np.random.default_rng(seed)
    sizes, left = [], len(tokens)
    while left > 0:
        n = int(rng.choice([2, 2, 3, 5, 7, 13, 16, 17, 31]))
        n = min(n, left)
        if left - n == 1:          # never leave a single token: the smallest portion is two
            n = left
        sizes.append(n)
        left -= n
    return sizes


def solo_trace(rid, tokens, sizes, first_step=0):
    """Steps that feed one request in the given portions and want every position's logits."""
    steps, at = [], 0
    for i, n in enumerate(sizes):
        last = i == len(sizes) - 1
        steps.append({"step": first_step + i,
                      "entries": [{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}],
                      "end": [rid] if last else []})
        at += n
    assert at == len(tokens)
    return steps


def mixed_trace(requests, seed, max_live=4, first_step=0):
    """Up to `max_live` live requests: each is fed in portions (a prompt part in random cuts, then its
    tail token by token), so steps hold portions of some beside single tokens of others; some
    requests sit a step out now and then. Returns (steps, peak tokens held rounded up to 64 each)."""
    rng = np.random.default_rng(seed)
    plans = {}
    for rid, tokens in requests.items():
        n_tail = int(rng.integers(3, 12))
        n_tail = min(n_tail, len(tokens) - 1)
        head = tokens[:len(tokens) - n_tail]
        sizes = cut_varying(head, int(rng.integers(1 << 30))) if len(head) > 1 else [len(head)]
        plans[rid] = sizes + [1] * n_tail
    waiting = list(requests)
    live, at, idx = [], {}, {}
    steps, step_no, peak = [], first_step, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid = waiting.pop(0)
            live.append(rid); at[rid] = 0; idx[rid] = 0
        entries, ended = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # this request sits the step out
            n = plans[rid][idx[rid]]
            toks = requests[rid][at[rid]:at[rid] + n]
            entries.append({"id": rid, "tokens": toks, "want": list(range(n))})
            at[rid] += n; idx[rid] += 1
            if idx[rid] == len(plans[rid]):
                ended.append(rid)
        if not entries:
            continue
        peak = max(peak, sum(-(-at[r] // 64) * 64 for r in live))
        steps.append({"step": step_no, "entries": entries, "end": ended})
        step_no += 1
        for rid in ended:
            live.remove(rid)
    return steps, peak


def collect_rows(steps, outputs):
    """{(request id, position): logits row} from the per-step outputs {step: array [wanted, vocab]}."""
    pos = {}
    rows = {}
    for s in steps:
        k = 0
        out = outputs.get(s["step"])
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], base + w)] = out[k]
                k += 1
            pos[e["id"]] = base + len(e["tokens"])
        assert out is None or k == out.shape[0]
    return rows


def run_inprocess(model_dir, dtype, steps, max_tokens, cuda_graphs=True, step_graph_after=2, debug_poison=False):
    """Replays steps through the engine's runner in this process (what bin/trace_run does)."""
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine.runner import ModelRunner, StepEntry
    from boring_llm_b200.models import load_model
    cfg, model = load_model(model_dir, dtype, "cuda:0")
    cap = -(-max_tokens // 16) * 16
    opts = EngineOptions(dtype=dtype, page_size=16, max_tokens=cap, ctx_size=min(cfg.max_position_embeddings, cap),
                         max_num_seqs=8, cuda_graphs=cuda_graphs, step_graph_after=step_graph_after,
                         debug_poison=debug_poison)
    runner = ModelRunner(model, opts)
    outputs = {}
    for s in steps:
        for t in s.get("truncate", []):
            runner.truncate(t["id"], t["keep"])
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = runner.step(entries)
        if logits.shape[0]:
            outputs[s["step"]] = logits.float().cpu().numpy()
        for rid in s["end"]:
            runner.free_request(rid)
    runner.cache.check()
    assert runner.cache.stats()["live_requests"] == 0
    return outputs, runner


def run_trace_program(model_dir, dtype, steps, max_tokens, out_dir, vocab, env=None, extra=()):
    """Drives bin/trace_run as a user would: one line in, wait for `done <step>`, next line."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)] + list(extra)
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline()
            assert line.strip() == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    outputs = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n:
            outputs[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n, vocab)
        else:
            assert not os.path.exists(path)
    return outputs
