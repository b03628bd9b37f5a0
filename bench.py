#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decoded tokens per second at batch 8 (the default `value`),
batch 1 and 64, and prefill tokens per second at 2,048 tokens, for the Qwen2.5-0.5B layer sizes with
random weights, each with the fraction of its roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

One JSON line on standard output. A "step" is one decode step of the whole batch. `value` is timed on
the device (CUDA events around each step: metadata copy, every kernel of the step, the sampler);
`e2e` runs the same steps through the Python entry point (`Engine.step`: host token ids in, sampled
token ids back on the host every step).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of Qwen2.5-0.5B (the benchmark configuration)
SIZES = dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
             intermediate_size=4864, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
             tie_word_embeddings=True, max_position_embeddings=32768)
CONTEXT = 4096
PREFILL_TOKENS = 2048
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


def build_engine(n_layers, max_seqs, steps_total, cuda_graphs=True):
    import torch
    import boring_llm_b200 as b
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine import Engine
    from boring_llm_b200.models import build_model
    cfg = b.Qwen2Config.from_dict(dict(SIZES, architectures=["Qwen2ForCausalLM"], num_hidden_layers=n_layers))
    model = build_model(cfg)
    g = torch.Generator(device="cuda").manual_seed(0)
    tensors = {}
    for name, spec in sorted(model.tensor_specs().items()):
        t = torch.randn(spec.shape, generator=g, device="cuda", dtype=torch.float32) * 0.02
        if spec.kind == "norm":
            t += 1.0
        tensors[name] = t.to(torch.bfloat16)
    model.load(tensors, torch.bfloat16, torch.device("cuda:0"))
    del tensors
    opts = EngineOptions(dtype="bfloat16", ctx_size=CONTEXT, max_num_seqs=max_seqs, max_tokens=(CONTEXT + 16) * max_seqs,
                         max_num_batched_tokens=max(PREFILL_TOKENS, max_seqs), prefill_chunk=PREFILL_TOKENS,
                         cuda_graphs=cuda_graphs)
    return cfg, Engine.from_model(cfg, model, opts)


def fill_requests(eng, batch, ctx0, seed):
    """`batch` live requests that already hold `ctx0` tokens: pages are reserved through the cache manager
    and filled with random keys and values (a decode step's time does not depend on the values)."""
    import torch
    from boring_llm_b200.sampling.params import SamplingParams
    from boring_llm_b200.engine.scheduler import Request, RUNNING
    from boring_llm_b200.sampling.params import XorShift64
    g = torch.Generator().manual_seed(seed)
    reqs = []
    for i in range(batch):
        rid = f"bench{seed}_{i}"
        eng.runner.cache.add_request(rid)
        assert eng.runner.cache.reserve(rid, ctx0)
        eng.runner.cache.commit(rid, ctx0)
        prompt = torch.randint(0, SIZES["vocab_size"], (ctx0 + 1,), generator=g).tolist()
        params = SamplingParams(n_predict=-1, ignore_eos=True)
        req = Request(rid, prompt[:ctx0], params, output=[prompt[ctx0]], num_computed=ctx0, state=RUNNING,
                      max_new=CONTEXT - ctx0, arrival=i, rng=XorShift64(i))
        eng.scheduler.running.append(req)
        reqs.append(req)
    for kv in eng.runner.storage.kv:
        kv.normal_(0.0, 0.5)
    return reqs


def drop_requests(eng, reqs):
    for r in reqs:
        if r in eng.scheduler.running:
            eng.scheduler.running.remove(r)
        if r.request_id in eng.runner.cache:
            eng.runner.cache.free(r.request_id)


def decode_device_timed(eng, batch, steps, warmup):
    """Tokens per second of `steps` decode steps of `batch` requests ending at the full context, timed on the
    device around all of them; returns (tokens/s, ms per step, kernel launches in the timed steps). Every step
    copies its inputs in, runs every kernel and the sampler, and brings its token ids back; the step after is
    launched before they are read (its tokens are fed back on the device), as `Engine.step` does."""
    import torch
    from boring_llm_b200.engine.runner import StepEntry
    from boring_llm_b200.kernels import ops
    ctx0 = CONTEXT - (steps + warmup) - 1
    reqs = fill_requests(eng, batch, ctx0, seed=batch)
    toks = [r.output[-1] for r in reqs]
    rows = [(r.params, r.rng, r.tokens) for r in reqs]          # greedy
    run = eng.runner
    for _ in range(warmup):
        toks = run.step_and_sample([StepEntry(r.request_id, [t], [0]) for r, t in zip(reqs, toks)], rows, eng.sampler)
    torch.cuda.synchronize()
    l0, graph_kernels = ops.launch_count, 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    first = [StepEntry(r.request_id, [t], [0]) for r, t in zip(reqs, toks)]
    pending = run.launch_decode(first, rows)
    if pending is None:                                            # no captured graphs: one step after the other
        toks = run.step_and_sample(first, rows, eng.sampler)
        for _ in range(steps - 1):
            toks = run.step_and_sample([StepEntry(r.request_id, [t], [0]) for r, t in zip(reqs, toks)], rows, eng.sampler)
    else:
        graph_kernels = run.last_step_graph_kernels
        for _ in range(steps - 1):
            ahead = run.launch_decode([StepEntry(r.request_id, [0], [0]) for r in reqs], rows, from_device=True)
            graph_kernels += run.last_step_graph_kernels
            toks = run.collect_decode(pending)
            pending = ahead
        toks = run.collect_decode(pending)
    e1.record()
    torch.cuda.synchronize()
    total_ms = e0.elapsed_time(e1)
    launches = ops.launch_count - l0 + graph_kernels
    drop_requests(eng, reqs)
    return batch * steps / (total_ms / 1e3), total_ms / steps, launches


def decode_end_to_end(eng, batch, steps, warmup):
    """The same steps through Engine.step(): scheduling, pinned host -> device copy of the step's inputs,
    kernels, sampling, device -> host read of the sampled ids, bookkeeping. Wall clock between device syncs."""
    import torch
    ctx0 = CONTEXT - (steps + warmup) - 1
    reqs = fill_requests(eng, batch, ctx0, seed=1000 + batch)
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    h2d = d2h = 0
    for _ in range(steps):
        eng.step()
        h2d += eng.runner.last_h2d_bytes
        d2h += eng.runner.last_d2h_bytes
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert all(len(r.output) == 1 + warmup + steps for r in reqs)
    eng.drain()                                                    # the step that was launched ahead of the last one read
    drop_requests(eng, reqs)
    # per step, counted by the runner from the tensors it copies: token ids, positions, lengths, slots, sampling
    # parameters (and block-table rows when a request got a new page) go up from pinned memory, one int32 per
    # row of the captured batch comes back
    return batch * steps / dt, h2d // steps, d2h // steps


def prefill_timed(eng, reps=3):
    import torch
    from boring_llm_b200.engine.runner import StepEntry
    g = torch.Generator().manual_seed(7)
    best = None
    for i in range(reps + 1):
        toks = torch.randint(0, SIZES["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.runner.step([StepEntry(f"prefill{i}", toks, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        eng.runner.free_request(f"prefill{i}")
        ms = e0.elapsed_time(e1)
        if i > 0:
            best = ms if best is None else min(best, ms)
    return best


def model_figures(n_layers):
    d, H, KV, dh, F, V = (SIZES[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                             "intermediate_size", "vocab_size"))
    per_layer = d * (H + 2 * KV) * dh + H * dh * d + 3 * d * F
    weight_bytes = 2 * (n_layers * per_layer + V * d)            # every matrix once, the output head included
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
    ap.add_argument("--layers", type=int, default=SIZES["num_hidden_layers"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step singly (for profilers)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only and print its figures (for profilers; not the benchmark line)")
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
    cfg, eng = build_engine(args.layers, 64, args.steps + warmup, not args.no_graphs)
    weight_bytes, kv_tok, prefill_flops = model_figures(args.layers)
    if args.only == "decode":
        tps, ms_step, launches = decode_device_timed(eng, args.batch, args.steps, warmup)
        out = {"only": "decode", "batch": args.batch, "tokens_per_s": round(tps, 1), "ms_per_step": round(ms_step, 4),
               "launches": launches, "layers": args.layers}
        rows = 1
        while rows < args.batch:
            rows *= 2
        gr = eng.runner._graphs.get(rows)
        if gr is not None:          # the captured step alone, replayed back to back: the GPU's share of a step
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                gr.graph.replay()
            e1.record()
            torch.cuda.synchronize()
            out["graph_replay_ms"] = round(e0.elapsed_time(e1) / 20, 4)
        print(json.dumps(out))
        return 0
    if args.only == "prefill":
        pre_ms = prefill_timed(eng, reps=1)
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3), "layers": args.layers}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    tps, ms_step, launches = decode_device_timed(eng, args.batch, args.steps, warmup)
    e2e, h2d, d2h = decode_end_to_end(eng, args.batch, args.steps, warmup)
    clk = clocks.stop()
    b1, _, _ = decode_device_timed(eng, 1, min(args.steps, 32), 3)
    b64, _, _ = decode_device_timed(eng, 64, min(args.steps, 32), 3)
    pre_ms = prefill_timed(eng)
    mean_ctx = CONTEXT - args.steps / 2
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_tok
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8, context 4096 (Qwen2.5-0.5B sizes)", "value": round(tps, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "Qwen2.5-0.5B sizes, random weights N(0,0.02)", "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": args.layers, "layers_full": SIZES["num_hidden_layers"],
                   "hidden": SIZES["hidden_size"], "heads": SIZES["num_attention_heads"],
                   "kv_heads": SIZES["num_key_value_heads"], "head_dim": SIZES["head_dim"],
                   "intermediate": SIZES["intermediate_size"], "vocab": SIZES["vocab_size"], "page_size": 16,
                   "prefill_tokens": PREFILL_TOKENS, "l2": "inputs larger than L2 (weights + cache read every step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clk,
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(prefill_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1)},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
