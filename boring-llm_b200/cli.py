"""The command line, in the manner of the reference's `main` (src/main.br:549-1254): a hand-rolled
argument loop in which an unknown or incomplete flag is an error (:1194-1195), `LLAMA_ARG_*`
environment variables give defaults that explicit flags override (:75-77, 552-639), and the id-only
entry points take comma-separated token ids (:115-120, 741-746):

  --model DIR --prompt-tokens IDS   generate through chunked prefill + decode, print `generated: id,id,...`
                                    (the reference's --generate-tokens, which is accepted too)
  --model DIR --tokens IDS          one whole-sequence pass, print the top-5 logits of every position
                                    (`pos P (token T): top5 = [...]`, src/main.br:127-145)
  --dump-metadata                   print the configuration and the tensor list

Value parsers are pure functions so that they can be tested without a model (as src/cli_config.br).
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


class UsageError(ValueError):
    pass


def parse_int_arg(name: str, s: str) -> int:
    try:
        return int(s.strip())
    except ValueError:
        raise UsageError(f"invalid {name} value: '{s}'") from None


def parse_float_arg(name: str, s: str) -> float:
    try:
        return float(s.strip())
    except ValueError:
        raise UsageError(f"invalid {name} value: '{s}'") from None


def parse_token_ids(csv: str) -> List[int]:
    """src/main.br:115-120."""
    out = []
    for part in csv.split(","):
        try:
            out.append(int(part.strip()))
        except ValueError:
            raise UsageError(f"invalid token id: '{part}'") from None
    return out


def parse_cache_type_arg(name: str, s: str) -> str:
    """The reference stores the cache as f32, f16 or q8_0 (src/cli_config.br:4-7); this engine stores it
    in its compute dtype, so the flag chooses that: f32 -> float32, bf16 -> bfloat16."""
    v = s.strip().lower()
    if v in ("f32", "float32"):
        return "float32"
    if v in ("bf16", "bfloat16"):
        return "bfloat16"
    raise UsageError(f"{name} supports f32 or bf16 (quantized and f16 caches are not built)")


def effective_prefill_chunk(batch_size: int, ubatch_size: int) -> int:
    """src/cli_config.br:24-25."""
    return batch_size if batch_size < ubatch_size else ubatch_size


@dataclass
class CliArgs:
    model: str = ""
    mode: str = ""                       # "generate" | "tokens" | "metadata"
    token_ids: List[int] = field(default_factory=list)
    n_predict: int = 40
    temperature: float = 0.0
    seed: int = 0
    ctx_size: int = 4096
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    batch_size: int = 2048
    ubatch_size: int = 512
    dtype: str = "bfloat16"
    bench_iters: int = 0
    ignore_eos: bool = False
    kv_cache: bool = True
    help: bool = False
    version: bool = False


_VALUE_FLAGS = {
    # flag spellings -> (field, parser, LLAMA_ARG_* name)
    ("-m", "--model", "--gguf"): ("model", lambda n, s: s, "LLAMA_ARG_MODEL"),
    ("-n", "--predict", "--n-predict", "--max-tokens"): ("n_predict", parse_int_arg, "LLAMA_ARG_N_PREDICT"),
    ("--temp", "--temperature"): ("temperature", parse_float_arg, "LLAMA_ARG_TEMPERATURE"),
    ("-s", "--seed"): ("seed", parse_int_arg, "LLAMA_ARG_SEED"),
    ("-c", "--ctx-size"): ("ctx_size", parse_int_arg, "LLAMA_ARG_CTX_SIZE"),
    ("--top-k",): ("top_k", parse_int_arg, "LLAMA_ARG_TOP_K"),
    ("--top-p",): ("top_p", parse_float_arg, "LLAMA_ARG_TOP_P"),
    ("--min-p",): ("min_p", parse_float_arg, "LLAMA_ARG_MIN_P"),
    ("--repeat-penalty",): ("repeat_penalty", parse_float_arg, "LLAMA_ARG_REPEAT_PENALTY"),
    ("--repeat-last-n",): ("repeat_last_n", parse_int_arg, "LLAMA_ARG_REPEAT_LAST_N"),
    ("-b", "--batch-size"): ("batch_size", parse_int_arg, "LLAMA_ARG_BATCH"),
    ("-ub", "--ubatch-size"): ("ubatch_size", parse_int_arg, "LLAMA_ARG_UBATCH"),
    ("--bench-iters",): ("bench_iters", parse_int_arg, None),
    ("--dtype",): ("dtype", lambda n, s: parse_cache_type_arg(n, s), None),
    ("-ctk", "--cache-type-k", "-ctv", "--cache-type-v"): ("dtype", parse_cache_type_arg, None),
}


def parse_args(argv: Sequence[str], env: Optional[Dict[str, str]] = None) -> CliArgs:
    env = os.environ if env is None else env
    a = CliArgs()
    for names, (fld, parser, env_name) in _VALUE_FLAGS.items():
        if env_name and env_name in env and not any(n in argv for n in names):
            setattr(a, fld, parser(env_name, env[env_name]))
    i = 0
    argv = list(argv)
    while i < len(argv):
        arg = argv[i]
        matched = False
        for names, (fld, parser, _) in _VALUE_FLAGS.items():
            if arg in names:
                if i + 1 >= len(argv):
                    raise UsageError(f"unknown or incomplete argument: {arg}")
                setattr(a, fld, parser(arg, argv[i + 1]))
                i += 2
                matched = True
                break
        if matched:
            continue
        if arg in ("--prompt-tokens", "--generate-tokens", "--tokens"):
            if i + 1 >= len(argv):
                raise UsageError(f"unknown or incomplete argument: {arg}")
            a.mode = "tokens" if arg == "--tokens" else "generate"
            a.token_ids = parse_token_ids(argv[i + 1])
            i += 2
        elif arg == "--dump-metadata":
            a.mode = "metadata"; i += 1
        elif arg == "--kv-cache":
            a.kv_cache = True; i += 1           # incremental decoding is the only generation path here
        elif arg == "--ignore-eos":
            a.ignore_eos = True; i += 1
        elif arg in ("-h", "--help", "--usage"):
            a.help = True; i += 1
        elif arg == "--version":
            a.version = True; i += 1
        else:
            raise UsageError(f"unknown or incomplete argument: {arg}")
    if a.ctx_size <= 0:
        raise UsageError("--ctx-size must be positive")
    if a.batch_size <= 0 or a.ubatch_size <= 0:
        raise UsageError("--batch-size and --ubatch-size must be positive")
    return a


USAGE = """usage: boring-llm --model DIR (--prompt-tokens IDS | --tokens IDS | --dump-metadata) [options]
  -m, --model DIR            folder with config.json and model.safetensors      [LLAMA_ARG_MODEL]
  --prompt-tokens IDS        comma-separated prompt token ids; prints `generated: id,id,...`
  --tokens IDS               whole-sequence pass; prints the top-5 logits of every position
  -n, --n-predict N          tokens to generate (default 40, -1: up to the context size)
  --temp T                   temperature (default 0: greedy)      -s, --seed S   generator seed (default 0)
  --top-k K  --top-p P  --min-p P  --repeat-penalty R  --repeat-last-n N       sampler options
  -c, --ctx-size N           prompt + reply limit (default 4096)
  -b, --batch-size N / -ub, --ubatch-size N   step token budget / prompt portion (default 2048 / 512)
  --dtype bf16|f32           compute and cache dtype (default bf16)   --kv-cache   accepted (always on)
  --bench-iters N            timed repetitions of prefill + decode     --ignore-eos   do not stop at end tokens
"""


def print_top5(logits, tokens) -> None:
    """src/main.br:127-145."""
    import torch
    vals, idx = torch.topk(logits, min(5, logits.shape[1]), dim=1)
    for p, tok in enumerate(tokens):
        pairs = ", ".join(f"({int(i)}, {float(v):.6g})" for i, v in zip(idx[p], vals[p]))
        print(f"pos {p} (token {tok}): top5 = [{pairs}]")


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    try:
        a = parse_args(argv)
    except UsageError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if a.help:
        print(USAGE, end="")
        return 0
    if a.version:
        from . import __version__
        print(f"boring-llm_b200 {__version__}")
        return 0
    if not a.model:
        print("error: --model DIR is required", file=sys.stderr)
        return 2
    if not a.mode:
        print("error: one of --prompt-tokens, --tokens or --dump-metadata is required", file=sys.stderr)
        return 2
    from .config import ConfigError, EngineOptions, load_config
    from .weights import WeightsError
    try:
        if a.mode == "metadata":
            from .models import build_model
            cfg = load_config(a.model)
            for k, v in cfg.to_dict().items():
                print(f"{k} = {v}")
            for name, spec in sorted(build_model(cfg).tensor_specs().items()):
                print(f"tensor {name} {list(spec.shape)} {spec.kind}")
            return 0
        from .engine import Engine, SamplingParams, StepEntry
        from .engine.scheduler import AdmissionError
        opts = EngineOptions(dtype=a.dtype, ctx_size=a.ctx_size, max_num_seqs=1, max_tokens=a.ctx_size,
                             max_num_batched_tokens=a.batch_size, prefill_chunk=a.ubatch_size)
        eng = Engine(a.model, opts)
        if a.mode == "tokens":
            logits = eng.runner.step([StepEntry("tokens", a.token_ids, list(range(len(a.token_ids))))])
            print_top5(logits.float().cpu(), a.token_ids)
            return 0
        params = dict(n_predict=a.n_predict, temperature=a.temperature, seed=a.seed, top_k=a.top_k, top_p=a.top_p,
                      min_p=a.min_p, repeat_penalty=a.repeat_penalty, repeat_last_n=a.repeat_last_n,
                      ignore_eos=a.ignore_eos)
        import torch
        for rep in range(a.bench_iters):
            # as the reference's bench loop (src/main.br:180-213): prefill timed alone, then the decode steps
            req = eng.add_request(a.token_ids, SamplingParams(**params))
            torch.cuda.synchronize(); t0 = time.perf_counter()
            while not req.output and eng.scheduler.has_work():
                eng.step()
            torch.cuda.synchronize(); t1 = time.perf_counter()
            eng.run_until_done()
            torch.cuda.synchronize(); t2 = time.perf_counter()
            print(f"[diag] bench rep {rep}: prompt={len(a.token_ids)} prefill_us={int((t1 - t0) * 1e6)} "
                  f"gen={max(0, len(req.output) - 1)} decode_us={int((t2 - t1) * 1e6)}")
        out = eng.generate([a.token_ids], **params)[0]
        print("generated: " + ",".join(str(t) for t in out))
        return 0
    except (ConfigError, WeightsError, AdmissionError, ValueError, RuntimeError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
