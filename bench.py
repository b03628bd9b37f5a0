#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decoded tokens per second at batch 8 (the default `value`), batch 1 and 64,
prefill tokens per second at 2,048 tokens (in one step and in four portions of 512), and a mixed step (one portion
of 512 beside 63 decoding requests), for the Qwen2.5-0.5B layer sizes with random weights, each with the fraction of
its roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--sizes 0.5b|3b|7b] [--layers L]

One JSON line on standard output. A "step" is one decode step of the whole batch. Requests are real ones: random
prompts admitted by the scheduler, prefilled in portions through the engine, then decoded; the model comes from the
engine's own random-weights mode. `value` is timed on the device (CUDA events around K steps of `Engine.step`,
median of three such regions); `e2e` is the wall clock of the same call (host token ids in, sampled token ids back on
the host every step). `checked` says that the tokens of one decode step equal those of the same step run by the plain
kernels on the same cache.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the Qwen2.5 models (the benchmark's configurations); 0.5b is the headline
SIZES = {
    "0.5b": dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                 intermediate_size=4864, vocab_size=151936, tie_word_embeddings=True),
    "3b": dict(num_hidden_layers=36, hidden_size=2048, num_attention_heads=16, num_key_value_heads=2, head_dim=128,
               intermediate_size=11008, vocab_size=151936, tie_word_embeddings=True),
    "7b": dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
               intermediate_size=18944, vocab_size=152064, tie_word_embeddings=False),
}
COMMON = dict(architectures=["Qwen2ForCausalLM"], rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=32768)
CONTEXT = 4096
LONG_CONTEXT = 32768           # a further decode point (not the headline): the cache of the live requests outweighs the weights
PREFILL_TOKENS = 2048
PORTION = 512                     # the reference's default portion of a prompt (-ub, src/cli_config.br:24-25)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_engine(sizes, n_layers, max_seqs, cuda_graphs=True, context=CONTEXT):
    import boring_llm_b200 as b
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine import Engine
    cfg = b.Qwen2Config.from_dict({**COMMON, **SIZES[sizes], "num_hidden_layers": n_layers})
    opts = EngineOptions(dtype="bfloat16", ctx_size=context, max_num_seqs=max_seqs, max_tokens=(context + 16) * max_seqs,
                         max_num_batched_tokens=PREFILL_TOKENS, prefill_chunk=PORTION, cuda_graphs=cuda_graphs)
    return cfg, Engine.from_random(cfg, 0, opts)               # N(0, 0.02) weights made on the device, no file


def random_prompt(vocab, n, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def start_requests(eng, lengths, seed, sampled=False):
    """Admits one request per prompt length and steps the engine until every one of them has been prefilled (in
    portions, several requests to a step, as the scheduler cuts them) and has its first token. `sampled`: the
    requests draw their tokens (temperature 0.8, top-k 40, top-p 0.95) instead of taking the largest logit."""
    from boring_llm_b200.sampling.params import SamplingParams
    vocab = eng.runner.vocab_size
    how = dict(temperature=0.8, top_k=40, top_p=0.95, seed=seed) if sampled else {}
    reqs = [eng.add_request(random_prompt(vocab, n, seed * 1000 + i), SamplingParams(n_predict=-1, ignore_eos=True, **how))
            for i, n in enumerate(lengths)]
    while not all(r.output for r in reqs):
        eng.step()
    eng.drain()
    return reqs


def end_requests(eng, reqs):
    eng.drain()
    for r in reqs:
        eng.scheduler.abort(r.request_id)
    assert eng.runner.cache.stats()["live_requests"] == 0


def check_one_step(eng, reqs):
    """The next decode step twice on the same cache: first by the plain kernels (every kernel's twin, launched one by
    one, 32-bit accumulation in a fixed order), rolled back, then by the serving path (captured graph, fused and
    tensor-core kernels, the sampler on the device). Greedy tokens must agree; where they do not, the plain
    logits of the two tokens must be closer than bfloat16 rounding explains."""
    import torch
    from boring_llm_b200.engine.runner import StepEntry
    run = eng.runner
    entries = [StepEntry(r.request_id, [r.output[-1]], [0]) for r in reqs]
    before = [run.cache.get(r.request_id).num_tokens for r in reqs]
    run.fast = False
    logits = run.step(entries).float()
    run.fast = True
    plain_tokens = logits.argmax(-1).tolist()
    for r, n in zip(reqs, before):
        run.truncate(r.request_id, n)
    rows = [(r.params, r.rng, r) for r in reqs]
    fast_tokens = run.step_and_sample(entries, rows, eng.sampler)
    for r, n in zip(reqs, before):                            # the engine's own next step computes this position again
        run.truncate(r.request_id, n)
    scale = logits.abs().max().item()
    ties = 0
    for i, (a, b) in enumerate(zip(plain_tokens, fast_tokens)):
        if a != b:
            if (logits[i, a] - logits[i, b]).item() > 0.02 * scale:
                return {"ok": False, "rows": len(reqs), "row": i, "plain": a, "fast": b}
            ties += 1
    return {"ok": True, "rows": len(reqs), "equal": len(reqs) - ties, "near_ties": ties}


def measure_decode(eng, batch, steps, warmup, value_regions=3, e2e_regions=0, check=False, seed=1, sampled=False,
                   context=CONTEXT):
    """Decode steps of `batch` requests whose contexts end just below the context size. Returns a dict with the
    device-timed figures (median region of `steps` steps), the wall-clock figures when asked for, the kernels launched
    in a region, the mean context inside the timed regions and the result of the one-step check."""
    import torch
    run = eng.runner
    per_step = eng.options.max_num_batched_tokens
    need = warmup + (value_regions + e2e_regions) * steps + 8
    # the requests that finish their prompts first decode while the others are still being prefilled
    ctx0 = context - need
    prefill_steps = -(-batch * ctx0 // per_step) + 2
    ctx0 -= prefill_steps
    reqs = start_requests(eng, [ctx0] * batch, seed, sampled)
    out = {}
    if check:
        out["checked"] = check_one_step(eng, reqs)
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    regions = []
    torch.cuda.profiler.start()               # a profiler started with --profile-from-start off sees the timed steps only
    for _ in range(value_regions):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx_a = sum(len(r.prompt) + len(r.output) for r in reqs) / batch
        launches = 0
        e0.record()
        for _ in range(steps):
            eng.step()
            launches += run.last_step_graph_kernels
        e1.record()
        torch.cuda.synchronize()
        ctx_b = sum(len(r.prompt) + len(r.output) for r in reqs) / batch
        regions.append((e0.elapsed_time(e1), launches, (ctx_a + ctx_b) / 2))
    torch.cuda.profiler.stop()
    ms, launches, ctx = sorted(regions)[len(regions) // 2]
    out.update(tokens_per_s=batch * steps / (ms / 1e3), ms_per_step=ms / steps, launches=launches, mean_ctx=ctx,
               region_ms=[round(r[0], 3) for r in regions])
    walls = []
    for _ in range(e2e_regions):
        torch.cuda.synchronize()
        h2d = d2h = 0
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.step()
            h2d += run.last_h2d_bytes
            d2h += run.last_d2h_bytes
        torch.cuda.synchronize()
        walls.append((time.perf_counter() - t0, h2d // steps, d2h // steps))
    if walls:
        dt, h2d, d2h = sorted(walls)[len(walls) // 2]
        # per step, counted by the runner from the tensors it copies: token ids, positions, lengths, slots, sampling
        # parameters (and block-table rows when a request got a new page) go up from pinned memory, one int32 per
        # row of the captured batch comes back
        out.update(e2e_tokens_per_s=batch * steps / dt, h2d=h2d, d2h=d2h)
    assert all(r.state == "running" for r in reqs), "a request ended inside the timed region"
    gr = next((g for (rows, _), g in run._graphs.items() if rows >= batch), None)
    if gr is not None:              # the captured step alone, replayed back to back: the GPU's share of a step
        end_requests(eng, reqs)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            gr.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        out["graph_replay_ms"] = e0.elapsed_time(e1) / 20
    else:
        end_requests(eng, reqs)
    return out


def prefill_timed(eng, portions, reps=5):
    """A prompt of 2,048 tokens through the step function, whole or in portions; the last position's logits are
    wanted. Median of `reps` after two untimed runs (a padded shape is captured the second time it comes).
    Returns (device ms, wall ms)."""
    import torch
    from boring_llm_b200.engine.runner import StepEntry
    vocab = eng.runner.vocab_size
    dev, wall = [], []
    for i in range(reps + 2):
        toks = random_prompt(vocab, PREFILL_TOKENS, 7000 + i)
        rid = f"prefill{i}"
        torch.cuda.synchronize()
        if i == reps + 1:
            torch.cuda.profiler.start()       # a profiler started with --profile-from-start off sees the last run only
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        at = 0
        for n in portions:
            last = at + n == PREFILL_TOKENS
            logits = eng.runner.step([StepEntry(rid, toks[at:at + n], [n - 1] if last else [])])
            at += n
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        if i == reps + 1:
            torch.cuda.profiler.stop()
        eng.runner.check_kernels()
        eng.runner.free_request(rid)
        if i >= 2:
            dev.append(e0.elapsed_time(e1)); wall.append((t1 - t0) * 1e3)
    return statistics.median(dev), statistics.median(wall)


def mixed_timed(eng, n_decoding=63, arrivals=6):
    """Steps that hold one portion of 512 prompt tokens beside `n_decoding` single tokens: the decoding requests'
    contexts are spread from 512 to about 3,600, then prompts of 2,048 tokens arrive one after the other and are
    prefilled in four steps each while the others go on decoding. Returns the medians over these steps of the device
    time, the wall time of `Engine.step` (host in, tokens out), their difference, and the tokens of a step."""
    import torch
    from boring_llm_b200.sampling.params import SamplingParams
    lengths = [512 + (3100 * i) // max(1, n_decoding - 1) for i in range(n_decoding)]
    reqs = start_requests(eng, lengths, seed=5)
    vocab = eng.runner.vocab_size
    rec = []
    for a in range(arrivals):
        new = eng.add_request(random_prompt(vocab, PREFILL_TOKENS, 9000 + a), SamplingParams(n_predict=4, ignore_eos=True))
        for s in range(PREFILL_TOKENS // PORTION):
            torch.cuda.synchronize()
            last = a == arrivals - 1 and s == PREFILL_TOKENS // PORTION - 2
            if last:
                torch.cuda.profiler.start()   # a profiler started with --profile-from-start off sees this step only
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            eng.step()
            e1.record()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            if last:
                torch.cuda.profiler.stop()
            if a >= 2:                                          # the first two arrivals' steps meet and capture their shapes
                rec.append((e0.elapsed_time(e1), (t1 - t0) * 1e3))
        assert new.num_computed >= PREFILL_TOKENS
        while new.state == "running":
            eng.step()
        eng.drain()
    end_requests(eng, reqs)
    dev = statistics.median(r[0] for r in rec)
    wall = statistics.median(r[1] for r in rec)
    return dev, wall, max(0.0, wall - dev), PORTION + n_decoding


def cpu_baseline(sizes):
    """The plain implementation (tests/plain_model.py: float64, whole sequence, no cache, one function per part) on the
    host cores: one forward of 64 tokens through two layers of these sizes, the last position's logits. The only
    implementation of this architecture that runs on this machine's CPU; the reference's own is Boring source."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_model
    import boring_llm_b200 as b
    from boring_llm_b200.weights import random_tensors
    cfg = b.Qwen2Config.from_dict({**COMMON, **SIZES[sizes], "num_hidden_layers": 2})
    specs = b.build_model(cfg).tensor_specs()
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    lazy = random_tensors(specs, 0, torch.bfloat16, 0.02, device=dev)
    W = {n: lazy[n].cpu().double() for n in lazy}
    toks = random_prompt(cfg.vocab_size, 64, 3)
    t0 = time.perf_counter()
    plain_model.forward(cfg.to_dict(), W, toks, rows=[63])
    return 64 / (time.perf_counter() - t0)


def model_figures(sizes, n_layers):
    s = SIZES[sizes]
    d, H, KV, dh, F, V = (s[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                         "intermediate_size", "vocab_size"))
    per_layer = d * (H + 2 * KV) * dh + H * dh * d + 3 * d * F
    weight_bytes = 2 * (n_layers * per_layer + V * d)            # every matrix a decode step uses, once (the output head included)
    kv_bytes_per_token = 2 * n_layers * KV * dh * 2
    T = PREFILL_TOKENS
    prefill_flops = 2 * T * n_layers * per_layer + 2 * d * V + n_layers * 4 * H * dh * T * (T + 1) // 2
    return weight_bytes, kv_bytes_per_token, prefill_flops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sizes", default="0.5b", choices=sorted(SIZES), help="layer sizes; 0.5b is the headline, the others are extra points")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel singly (for profilers)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "prefill4", "mixed"],
                    help="run one part only and print its figures (for profilers; not the benchmark line)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "mlanoe/boring-llm is not a Python package (pip: neither setup.py nor pyproject.toml); it is "
                          "written in the Boring language for Metal/wgpu, and neither its compiler nor a graphics stack exists here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built (single-GPU tier)")
        return 2
    import torch
    assert torch.cuda.is_available(), "bench.py needs a GPU"
    pk = peaks()
    warmup = max(3, args.warmup)
    n_layers = args.layers or SIZES[args.sizes]["num_hidden_layers"]
    cfg, eng = build_engine(args.sizes, n_layers, 64, not args.no_graphs)
    weight_bytes, kv_tok, prefill_flops = model_figures(args.sizes, n_layers)

    def hbm_frac(batch, m):
        return (weight_bytes + batch * m["mean_ctx"] * kv_tok) / (m["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"]

    if args.only == "decode":
        m = measure_decode(eng, args.batch, args.steps, warmup, value_regions=1)
        print(json.dumps({"only": "decode", "batch": args.batch, "tokens_per_s": round(m["tokens_per_s"], 1),
                          "ms_per_step": round(m["ms_per_step"], 4), "launches": m["launches"], "layers": n_layers,
                          "hbm_frac": round(hbm_frac(args.batch, m), 4),
                          "graph_replay_ms": round(m.get("graph_replay_ms", 0.0), 4)}))
        return 0
    if args.only in ("prefill", "prefill4"):
        portions = [PREFILL_TOKENS] if args.only == "prefill" else [PORTION] * (PREFILL_TOKENS // PORTION)
        dev, wall = prefill_timed(eng, portions, reps=2)
        print(json.dumps({"only": args.only, "tokens": PREFILL_TOKENS, "ms": round(dev, 3), "wall_ms": round(wall, 3), "layers": n_layers}))
        return 0
    if args.only == "mixed":
        dev, wall, host, toks = mixed_timed(eng)
        print(json.dumps({"only": "mixed", "tokens": toks, "ms": round(dev, 3), "wall_ms": round(wall, 3), "layers": n_layers}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    m8 = measure_decode(eng, args.batch, args.steps, warmup, value_regions=3, e2e_regions=2, check=True, seed=1)
    clk = clocks.stop()
    k_small = min(args.steps, 32)
    m1 = measure_decode(eng, 1, k_small, 3, seed=2)
    m64 = measure_decode(eng, 64, k_small, 3, seed=3)
    m8s = measure_decode(eng, args.batch, k_small, 3, seed=4, sampled=True)     # the same step with drawn tokens
    pre_ms, pre_wall = prefill_timed(eng, [PREFILL_TOKENS])
    pre4_ms, pre4_wall = prefill_timed(eng, [PORTION] * (PREFILL_TOKENS // PORTION))
    mix_ms, mix_wall, mix_host, mix_tokens = mixed_timed(eng)
    cpu_tps = None if args.no_cpu_baseline else cpu_baseline(args.sizes)
    # a further point: the same batch at eight times the context (an engine of its own: the pool is sized by the context)
    del eng
    import gc, torch
    gc.collect(); torch.cuda.empty_cache()
    _, eng_long = build_engine(args.sizes, n_layers, args.batch, context=LONG_CONTEXT)
    mlong = measure_decode(eng_long, args.batch, 16, 3, value_regions=3, seed=5, context=LONG_CONTEXT)
    del eng_long
    achieved = hbm_frac(args.batch, m8) * pk["hbm_gbs"]
    headline = args.sizes == "0.5b"
    s = SIZES[args.sizes]
    line = {
        "metric": f"decode tok/s at batch {args.batch}, context 4096 (Qwen2.5-{args.sizes.upper()} sizes)",
        "value": round(m8["tokens_per_s"], 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(m8["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours", "headline": headline,
        "config": {"model": f"Qwen2.5-{args.sizes.upper()} sizes, random weights N(0,0.02)", "global_batch": args.batch,
                   "seq_len": CONTEXT, "parallelism": "single GPU", "layers": n_layers, "layers_full": s["num_hidden_layers"],
                   "hidden": s["hidden_size"], "heads": s["num_attention_heads"], "kv_heads": s["num_key_value_heads"],
                   "head_dim": s["head_dim"], "intermediate": s["intermediate_size"], "vocab": s["vocab_size"],
                   "page_size": 16, "prefill_tokens": PREFILL_TOKENS, "mean_ctx": round(m8["mean_ctx"]),
                   "timed": "median of 3 regions of K steps", "l2": "inputs larger than L2 (weights + cache read every step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(m8["e2e_tokens_per_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": m8["h2d"],
                "d2h_bytes_per_step": m8["d2h"]},
        "gpu_launches": m8["launches"],
        "clocks": clk,
        "checked": m8["checked"],
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(prefill_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {
            "decode_b1": round(m1["tokens_per_s"], 1), "decode_b64": round(m64["tokens_per_s"], 1),
            "decode_b1_hbm_frac": round(hbm_frac(1, m1), 4), "decode_b8_hbm_frac": round(hbm_frac(args.batch, m8), 4),
            "decode_b64_hbm_frac": round(hbm_frac(64, m64), 4),
            "decode_b1_ms": round(m1["ms_per_step"], 4), "decode_b64_ms": round(m64["ms_per_step"], 4),
            "decode_b8_graph_replay_ms": round(m8.get("graph_replay_ms", 0.0), 4),
            "decode_b8_sampled_ms": round(m8s["ms_per_step"], 4),
            f"decode_b8_ctx{LONG_CONTEXT}_ms": round(mlong["ms_per_step"], 4),
            f"decode_b8_ctx{LONG_CONTEXT}_hbm_frac": round(hbm_frac(args.batch, mlong), 4),
            f"decode_b8_ctx{LONG_CONTEXT}_graph_replay_ms": round(mlong.get("graph_replay_ms", 0.0), 4),
            "prefill_wall_ms": round(pre_wall, 3),
            "prefill_4x512": round(PREFILL_TOKENS / (pre4_ms / 1e3), 1), "prefill_4x512_ms": round(pre4_ms, 3),
            "prefill_4x512_wall_ms": round(pre4_wall, 3),
            "prefill_4x512_frac": round(prefill_flops / (pre4_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
            "mixed_b64_tokens": mix_tokens, "mixed_b64_ms": round(mix_ms, 3), "mixed_b64_wall_ms": round(mix_wall, 3),
            "mixed_b64_host_ms": round(mix_host, 3),
            "cpu_plain_tok_s_2_layers_64_tokens": None if cpu_tps is None else round(cpu_tps, 1),
        },
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
