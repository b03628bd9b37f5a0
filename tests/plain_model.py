"""A plain, slow implementation of the dense Qwen2 decoder, written from the reference's formulas:
whole sequences, no cache, no batching, one function for each part, float64 by default.

It shares no code with the engine: it has its own reader for model folders and its own math, and it
is what every engine result is compared with. Each function cites the reference's file:line it
restates. `tests/golden/make_golden.py` compared it once with the reference's own numpy graph
(tools/make_arch_test_ggufs.py:109-211) on tiny random models; the outputs are in tests/golden/.
"""
import json
import math
import os
import struct

import numpy as np
import torch


# ---- reading a model folder (independent of the engine's loader) -----------------------------------
def read_safetensors(path):
    """{name: float64 tensor}. Format: 8-byte little-endian header length, JSON header, raw data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        raw = data[b:en]
        if e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        elif e["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"plain reader: dtype {e['dtype']} of {name}")
        out[name] = torch.from_numpy(a.reshape(e["shape"]).copy())
    return out


def read_model_folder(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


def layer_windows(cfg):
    """Window of each layer (0: none): `layer_types` when present, else layers from
    `max_window_layers` on when `use_sliding_window` is set."""
    n = cfg["num_hidden_layers"]
    if cfg.get("layer_types") is not None:
        sliding = [t == "sliding_attention" for t in cfg["layer_types"]]
    elif cfg.get("use_sliding_window", False):
        sliding = [i >= cfg.get("max_window_layers", n) for i in range(n)]
    else:
        sliding = [False] * n
    return [cfg["sliding_window"] if s else 0 for s in sliding]


# ---- one function for each part --------------------------------------------------------------------
def rms_norm(x, weight, eps):
    """src/math.br:18-36: ss = sum x^2; inv = 1 / sqrt(ss / d + eps); y = x * inv * weight."""
    mean_sq = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(mean_sq + eps)) * weight


def linear(x, w, b=None):
    """src/math.br:68-93: y[p, o] = sum_i x[p, i] * w[o, i]; the bias is added after the product."""
    y = x @ w.T
    return y if b is None else y + b


def rope_inv_freq(head_dim, base):
    """src/math.br:161-171: theta_j = 1 / base^(2j / n_rot), computed in 32-bit like the reference."""
    j = np.arange(head_dim // 2, dtype=np.float32)
    expo = (np.float32(2.0) * j) / np.float32(head_dim)
    return np.float32(1.0) / np.power(np.float32(base), expo, dtype=np.float32)


def rope_neox(x, positions, inv_freq):
    """src/math.br:128-157 with neox == 1: pairs (j, j + d_head/2) inside each head;
    angle = float32(abs_pos) * theta_j (a 32-bit product, as in the reference), then
    x0' = x0 cos - x1 sin, x1' = x0 sin + x1 cos. x: [seq, heads, d_head]."""
    half = x.shape[-1] // 2
    ang32 = positions.astype(np.float32)[:, None] * inv_freq[None, :]        # float32 product
    ang = torch.from_numpy(ang32.astype(np.float64)).to(dtype=x.dtype, device=x.device)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def gqa_attention(q, k, v, scale, window=0, p_stored=None):
    """src/math.br:304-359: kv head = head / (H / KV); score = dot * scale; query i sees keys j <= i
    and, with a window, only j + window > i; softmax with the maximum subtracted; out = p . v.
    q: [seq, H, dh]; k, v: [seq, KV, dh]. `p_stored` rounds the softmax numerators exp(s - max) the way a
    bfloat16 engine's tensor cores take them as an operand of p . v (the sum that divides stays exact)."""
    seq, H, dh = q.shape
    KV = k.shape[1]
    group = H // KV
    out = torch.zeros_like(q)
    idx = torch.arange(seq, device=q.device)
    allowed = idx[None, :] <= idx[:, None]
    if window > 0:
        allowed &= idx[None, :] + window > idx[:, None]
    for h in range(H):
        kv = h // group
        sc = (q[:, h] @ k[:, kv].T) * scale
        sc = torch.where(allowed, sc, torch.full_like(sc, -1e30))
        p = torch.exp(sc - sc.max(-1, keepdim=True).values)
        total = p.sum(-1, keepdim=True)
        if p_stored is not None:
            p = p_stored(p)
        out[:, h] = (p @ v[:, kv]) / total
    return out


def silu(x):
    """src/math.br:232-233: x / (1 + exp(-x))."""
    return x / (1.0 + torch.exp(-x))


def swiglu_ffn(x, w_gate, w_up, w_down):
    """src/math.br:246-261 with act == 0: down(silu(gate(x)) * up(x)), no biases."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


# ---- the whole model -------------------------------------------------------------------------------
def round_bf16(x):
    """Rounds to the nearest bfloat16 value (ties to even) and widens back."""
    return x.to(torch.bfloat16).to(x.dtype)


def forward(cfg, W, tokens, dtype=torch.float64, stored=None, rows=None):
    """Logits of every position of one whole sequence: src/model.br:1280-1362 with every optional
    branch neutral, as the reference runs GGUF arch `qwen2`.

    `stored`: None computes everything in `dtype`. `round_bf16` additionally rounds the tensors that a
    bfloat16 engine STORES between its kernels (normed rows, rotated q and k, v, the attention output,
    the SwiGLU product); everything inside a formula (products' sums, softmax, norms' statistics,
    rotation, the residual stream, logits) stays in `dtype`. With it the comparison is about the
    formulas and the cache, not about how well a random model happens to be conditioned.

    `rows`: positions whose logits are returned (default: all). The tensors of `W` may live on any device.
    """
    st = stored if stored is not None else (lambda t: t)
    W = {k: v.to(dtype) for k, v in W.items()}
    H, KV = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    dh = cfg.get("head_dim") or cfg["hidden_size"] // H
    eps = cfg.get("rms_norm_eps", 1e-6)
    inv_freq = rope_inv_freq(dh, cfg.get("rope_theta", 10000.0))
    windows = layer_windows(cfg)
    tokens = list(tokens)
    seq = len(tokens)
    pos = np.arange(seq)
    x = W["model.embed_tokens.weight"][tokens]                                   # :1286-1295
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = st(rms_norm(x, W[p + "input_layernorm.weight"], eps))                # :1310
        bias = (p + "self_attn.q_proj.bias") in W
        q = linear(h, W[p + "self_attn.q_proj.weight"], W[p + "self_attn.q_proj.bias"] if bias else None)
        k = linear(h, W[p + "self_attn.k_proj.weight"], W[p + "self_attn.k_proj.bias"] if bias else None)
        v = st(linear(h, W[p + "self_attn.v_proj.weight"], W[p + "self_attn.v_proj.bias"] if bias else None))
        q = st(rope_neox(q.reshape(seq, H, dh), pos, inv_freq))                  # :1317-1319
        k = st(rope_neox(k.reshape(seq, KV, dh), pos, inv_freq))
        a = st(gqa_attention(q, k, v.reshape(seq, KV, dh), 1.0 / math.sqrt(dh), windows[l], stored))   # :1323-1324
        x = x + linear(a.reshape(seq, H * dh), W[p + "self_attn.o_proj.weight"])  # :1328-1334
        h = st(rms_norm(x, W[p + "post_attention_layernorm.weight"], eps))       # :1340
        act = st(silu(linear(h, W[p + "mlp.gate_proj.weight"])) * linear(h, W[p + "mlp.up_proj.weight"]))
        x = x + linear(act, W[p + "mlp.down_proj.weight"])                       # :1346-1356, src/math.br:246-261
    if rows is not None:
        x = x[list(rows)]
    y = st(rms_norm(x, W["model.norm.weight"], eps))                             # :1360
    out_w = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else W["lm_head.weight"]
    return linear(y, out_w)                                                      # :1361


def greedy_generate(cfg, W, prompt, n):
    """Greedy continuation by full re-forwards, as tools/make_arch_test_ggufs.py:417-425:
    first maximum wins (src/sampling.br:239-249)."""
    tokens = list(prompt)
    out = []
    for _ in range(n):
        logits = forward(cfg, W, tokens)
        out.append(int(torch.argmax(logits[-1]).item()))
        tokens.append(out[-1])
    return out


# ---- sampling, host side, in the reference's semantics ---------------------------------------------
MASK64 = (1 << 64) - 1


def seed_rng(seed):
    """src/sampling.br:35-40."""
    return 88172645463325252 if seed == 0 else (seed & MASK64) ^ 88172645463325252


def rng_next_u64(state):
    """xorshift64, src/sampling.br:42-47."""
    x = state
    x ^= (x << 13) & MASK64
    x ^= x >> 7
    x ^= (x << 17) & MASK64
    return x, x


def rng_next_f32(state):
    """src/sampling.br:51-54: float32(x) / 2^64."""
    x, state = rng_next_u64(state)
    return float(np.float32(x) / np.float32(18446744073709551616.0)), state


def sample(state, logits, temperature, top_k=0, top_p=1.0, min_p=0.0):
    """(token, new state): src/sampling.br:490-607, 742-760 without the filters this engine leaves
    out. Greedy when temperature <= 0 (the generator is not advanced). Otherwise candidates in
    descending order (top_k of them, or all), untempered softmax, top-p and min-p prefix cuts, then
    weights exp((l - l_first) / T) and the first candidate whose running sum reaches u * total."""
    logits = np.asarray(logits, dtype=np.float64)
    if temperature <= 0:
        return int(np.argmax(logits)), state
    order = np.argsort(-logits, kind="stable")
    if top_k > 0:
        order = order[:top_k]
    vals = logits[order]
    probs = np.exp(vals - vals[0])
    probs /= probs.sum()
    cutoff = len(vals)
    if top_p < 1.0:
        cum = np.cumsum(probs)
        cutoff = int(np.searchsorted(cum, top_p, side="left")) + 1
        cutoff = min(cutoff, len(vals))
    if min_p > 0.0:
        thr = probs[0] * min_p
        mc = 1
        while mc < cutoff and probs[mc] >= thr:
            mc += 1
        cutoff = mc
    w = np.exp((vals[:cutoff] - vals[0]) / temperature)
    u, state = rng_next_f32(state)
    target = u * w.sum()
    run = np.cumsum(w)
    slot = int(np.searchsorted(run, target, side="left"))
    slot = min(slot, cutoff - 1)
    return int(order[slot]), state
