"""Command-line parsing without a model (as test/test_cli_config.br), and the command itself on the GPU."""
import os
import subprocess
import sys

import pytest

import helpers
from boring_llm_b200.cli import (UsageError, effective_prefill_chunk, parse_args, parse_cache_type_arg,
                                 parse_token_ids)


def test_value_parsers():
    assert parse_token_ids("3,1, 4") == [3, 1, 4]
    with pytest.raises(UsageError, match="invalid token id: 'x'"):
        parse_token_ids("3,x")
    assert effective_prefill_chunk(2048, 512) == 512 and effective_prefill_chunk(8, 512) == 8
    assert parse_cache_type_arg("-ctk", "F32") == "float32" and parse_cache_type_arg("--dtype", "bf16") == "bfloat16"
    with pytest.raises(UsageError, match="supports"):
        parse_cache_type_arg("-ctk", "q8_0")


def test_flags_defaults_and_environment():
    a = parse_args(["--model", "M", "--prompt-tokens", "1,2"], env={})
    assert (a.n_predict, a.temperature, a.seed, a.ctx_size, a.top_k, a.top_p) == (40, 0.0, 0, 4096, 0, 1.0)
    assert a.mode == "generate" and a.token_ids == [1, 2] and (a.batch_size, a.ubatch_size) == (2048, 512)
    a = parse_args(["-m", "M", "--generate-tokens", "5", "-n", "7", "--temp", "0.8", "-s", "3", "-c", "64", "--kv-cache",
                    "--top-k", "40", "--top-p", "0.9", "--min-p", "0.05", "-ub", "8", "--dtype", "f32"], env={})
    assert (a.n_predict, a.temperature, a.seed, a.ctx_size, a.top_k, a.top_p, a.min_p) == (7, 0.8, 3, 64, 40, 0.9, 0.05)
    assert a.ubatch_size == 8 and a.dtype == "float32" and a.kv_cache
    env = {"LLAMA_ARG_MODEL": "E", "LLAMA_ARG_N_PREDICT": "9", "LLAMA_ARG_CTX_SIZE": "100"}
    a = parse_args(["--tokens", "1"], env=env)
    assert a.model == "E" and a.n_predict == 9 and a.ctx_size == 100 and a.mode == "tokens"
    a = parse_args(["--tokens", "1", "-n", "2", "--model", "X"], env=env)          # explicit flags win
    assert a.model == "X" and a.n_predict == 2


def test_unknown_or_incomplete_arguments_are_errors():
    for argv in (["--frobnicate"], ["--model"], ["--prompt-tokens"], ["-n"]):
        with pytest.raises(UsageError, match="unknown or incomplete argument"):
            parse_args(argv, env={})
    with pytest.raises(UsageError, match="invalid -n value"):
        parse_args(["-n", "many"], env={})


@pytest.mark.gpu
def test_the_command_generates_and_prints_top5(model_folders):
    import plain_model as plain
    d = model_folders("A", "float32", 0.02)
    exe = [sys.executable, os.path.join(helpers.ROOT, "bin", "boring-llm")]
    prompt = helpers.random_tokens(256, 9, 3)
    ids = ",".join(map(str, prompt))
    p = subprocess.run(exe + ["--model", d, "--prompt-tokens", ids, "--n-predict", "6", "--dtype", "f32", "--ctx-size", "64",
                              "--ignore-eos", "--bench-iters", "1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    lines = p.stdout.strip().splitlines()
    assert lines[0].startswith("[diag] bench rep 0: prompt=9 prefill_us=")
    cfg, W = plain.read_model_folder(d)
    assert lines[-1] == "generated: " + ",".join(map(str, plain.greedy_generate(cfg, W, prompt, 6)))
    p = subprocess.run(exe + ["--model", d, "--tokens", ids, "--dtype", "f32", "-c", "64"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    out = p.stdout.strip().splitlines()
    logits = plain.forward(cfg, W, prompt).numpy()
    assert len(out) == 9
    for pos, line in enumerate(out):
        assert line.startswith(f"pos {pos} (token {prompt[pos]}): top5 = [({int(logits[pos].argmax())}, ")
    p = subprocess.run(exe + ["--model", d, "--bogus"], capture_output=True, text=True)
    assert p.returncode == 2 and "unknown or incomplete argument" in p.stderr
    p = subprocess.run(exe + ["--model", d + "_missing", "--tokens", "1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 1 and "config.json" in p.stderr
