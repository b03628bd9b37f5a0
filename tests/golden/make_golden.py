#!/usr/bin/env python3
"""Compares the plain implementation (tests/plain_model.py) with the reference's own model code and
writes the small outputs that tests/test_plain_golden.py checks.

The reference's engine is written in the Boring language and cannot be compiled or imported here.
What can be imported on the CPU is its float64 numpy transcription of the model graph,
`reference()` in tools/make_arch_test_ggufs.py:109-211, the oracle of its architecture test
(test/test_arch.br:1-37). This script

1. builds three tiny random Qwen2 models that differ in every size and option (one with a window on
   every layer), runs the same tokens through `reference()` and through the plain implementation, and
   stores weights, tokens and the REFERENCE's logits in `tests/golden/<case>.npz`;
2. rebuilds the reference's `plain` fixture weights (`default_rng(7)`, make_weights,
   tools/make_arch_test_ggufs.py:214-227, 437-442) and compares the plain implementation with the
   committed file test/fixtures/arch-plain.logits.f32 (tolerance of the reference: 0.002,
   test/test_arch.br:35) and its greedy continuation arch-plain.generated.txt.

Usage:  python tests/golden/make_golden.py --reference <checkout of mlanoe/boring-llm>
"""
import argparse
import importlib.util
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_model as plain  # noqa: E402

CASES = {
    # name: config.json of the tiny model, number of tokens, seed
    "tied_gqa": (dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=32,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=8, intermediate_size=40,
                      vocab_size=48, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                      max_position_embeddings=128), 23, 11),
    "untied_mqa": (dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3, hidden_size=24,
                        num_attention_heads=3, num_key_value_heads=1, head_dim=16, intermediate_size=56,
                        vocab_size=37, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                        max_position_embeddings=256), 40, 12),
    "windowed": (dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=32,
                      num_attention_heads=2, num_key_value_heads=2, head_dim=16, intermediate_size=48,
                      vocab_size=29, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                      max_position_embeddings=128, use_sliding_window=True, sliding_window=5,
                      max_window_layers=0), 19, 13),
}


def tensor_shapes(cfg):
    d, H = cfg["hidden_size"], cfg["num_attention_heads"]
    KV, dh, F, V = cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    s = {"model.embed_tokens.weight": (V, d), "model.norm.weight": (d,)}
    if not cfg["tie_word_embeddings"]:
        s["lm_head.weight"] = (V, d)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        s.update({p + "input_layernorm.weight": (d,), p + "post_attention_layernorm.weight": (d,),
                  p + "self_attn.q_proj.weight": (H * dh, d), p + "self_attn.q_proj.bias": (H * dh,),
                  p + "self_attn.k_proj.weight": (KV * dh, d), p + "self_attn.k_proj.bias": (KV * dh,),
                  p + "self_attn.v_proj.weight": (KV * dh, d), p + "self_attn.v_proj.bias": (KV * dh,),
                  p + "self_attn.o_proj.weight": (d, H * dh), p + "mlp.gate_proj.weight": (F, d),
                  p + "mlp.up_proj.weight": (F, d), p + "mlp.down_proj.weight": (d, F)})
    return s


def random_weights(cfg, seed):
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        if name.endswith("norm.weight"):
            W[name] = rng.uniform(0.5, 1.5, shape)
        elif name.endswith(".bias"):
            W[name] = rng.normal(0, 0.08, shape)
        else:
            W[name] = rng.normal(0, 0.3, shape)
    return {k: v.astype(np.float32) for k, v in W.items()}       # float32-representable, stored as such


def to_reference_weights(cfg, W):
    """Our checkpoint names -> the dictionary that `reference(W, c)` reads."""
    W = {k: v.astype(np.float64) for k, v in W.items()}
    out = {"emb": W["model.embed_tokens.weight"], "out_norm": W["model.norm.weight"], "layers": []}
    out["out"] = out["emb"] if cfg["tie_word_embeddings"] else W["lm_head.weight"]
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        out["layers"].append({
            "attn_norm": W[p + "input_layernorm.weight"], "ffn_norm": W[p + "post_attention_layernorm.weight"],
            "q": W[p + "self_attn.q_proj.weight"], "k": W[p + "self_attn.k_proj.weight"],
            "v": W[p + "self_attn.v_proj.weight"], "o": W[p + "self_attn.o_proj.weight"],
            "q_b": W[p + "self_attn.q_proj.bias"], "k_b": W[p + "self_attn.k_proj.bias"],
            "v_b": W[p + "self_attn.v_proj.bias"], "gate": W[p + "mlp.gate_proj.weight"],
            "up": W[p + "mlp.up_proj.weight"], "down": W[p + "mlp.down_proj.weight"]})
    return out


def run_reference(ref, cfg, W, tokens):
    ref.NL, ref.D, ref.NH, ref.NKV = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    ref.FFN, ref.VOCAB, ref.EPS, ref.TOKENS = cfg["intermediate_size"], cfg["vocab_size"], cfg["rms_norm_eps"], list(tokens)
    dh = cfg["head_dim"]
    c = dict(d_head=dh, base=cfg["rope_theta"], neox=True, act="silu", embd_scale=1.0,
             rope=ref.rope_table(dh, cfg["rope_theta"]))
    if cfg.get("use_sliding_window"):
        c.update(window=cfg["sliding_window"], all_swa=True)
    return ref.reference(to_reference_weights(cfg, W), c)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of mlanoe/boring-llm")
    args = ap.parse_args()
    spec = importlib.util.spec_from_file_location(
        "make_arch_test_ggufs", os.path.join(args.reference, "tools", "make_arch_test_ggufs.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    report = {}
    for name, (cfg, n_tok, seed) in CASES.items():
        W = random_weights(cfg, seed)
        tokens = np.random.default_rng(seed + 100).integers(0, cfg["vocab_size"], n_tok).tolist()
        want = run_reference(ref, cfg, W, tokens)
        got = plain.forward(cfg, {k: torch.from_numpy(v.astype(np.float64)) for k, v in W.items()}, tokens).numpy()
        diff = float(np.abs(want - got).max())
        report[name] = {"max_abs_diff_plain_vs_reference": diff, "max_abs_logit": float(np.abs(want).max())}
        np.savez_compressed(os.path.join(HERE, name + ".npz"), config=json.dumps(cfg), tokens=np.array(tokens),
                            reference_logits=want, **{"w:" + k: v for k, v in W.items()})
        print(f"{name}: plain vs reference max |diff| = {diff:.3e} (max |logit| {np.abs(want).max():.3f})")
    # the reference's own committed fixture of arch `qwen2`
    ref.NL, ref.D, ref.NH, ref.NKV, ref.FFN, ref.VOCAB, ref.EPS = 2, 16, 4, 2, 24, 10, 1e-6
    rw = ref.make_weights(np.random.default_rng(7), 4, False)
    cfg = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=16, num_attention_heads=4,
               num_key_value_heads=2, head_dim=4, intermediate_size=24, vocab_size=10, rope_theta=10000.0,
               rms_norm_eps=1e-6, tie_word_embeddings=False)
    W = {"model.embed_tokens.weight": rw["emb"], "lm_head.weight": rw["out"], "model.norm.weight": rw["out_norm"]}
    for l, L in enumerate(rw["layers"]):
        p = f"model.layers.{l}."
        W.update({p + "input_layernorm.weight": L["attn_norm"], p + "post_attention_layernorm.weight": L["ffn_norm"],
                  p + "self_attn.q_proj.weight": L["q"], p + "self_attn.k_proj.weight": L["k"],
                  p + "self_attn.v_proj.weight": L["v"], p + "self_attn.o_proj.weight": L["o"],
                  p + "mlp.gate_proj.weight": L["gate"], p + "mlp.up_proj.weight": L["up"],
                  p + "mlp.down_proj.weight": L["down"]})
    Wt = {k: torch.from_numpy(np.asarray(v, dtype=np.float64)) for k, v in W.items()}
    tokens = [3, 1, 4, 1, 5, 9, 2, 6]
    got = plain.forward(cfg, Wt, tokens).numpy()
    fixture = np.fromfile(os.path.join(args.reference, "test", "fixtures", "arch-plain.logits.f32"), dtype="<f4").reshape(8, 10)
    gen_fixture = [int(t) for t in open(os.path.join(args.reference, "test", "fixtures", "arch-plain.generated.txt")).read().split()]
    gen = plain.greedy_generate(cfg, Wt, tokens, len(gen_fixture))
    diff = float(np.abs(fixture - got).max())
    report["reference_fixture_arch_plain"] = {"max_abs_diff_plain_vs_fixture": diff, "fixture_greedy": gen_fixture,
                                              "plain_greedy": gen, "reference_tolerance": 0.002}
    print(f"arch-plain fixture: max |diff| = {diff:.3e}; greedy {gen} vs fixture {gen_fixture}")
    with open(os.path.join(HERE, "report.json"), "w") as f:
        json.dump(report, f, indent=2)
        f.write("\n")


if __name__ == "__main__":
    main()
