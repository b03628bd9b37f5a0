"""The plain implementation against the reference's own numpy graph (outputs stored by
tests/golden/make_golden.py) and its parts against hand-computed values, as test/test_math.br does."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_model as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("case", ["tied_gqa", "untied_mqa", "windowed"])
def test_plain_equals_the_reference_graph(case):
    z = np.load(os.path.join(GOLDEN, case + ".npz"))
    cfg = json.loads(str(z["config"]))
    W = {k[2:]: torch.from_numpy(z[k].astype(np.float64)) for k in z.files if k.startswith("w:")}
    got = plain.forward(cfg, W, z["tokens"].tolist()).numpy()
    want = z["reference_logits"]
    # the reference computes rotation angles in float64, the engine's formulas (src/math.br:143) in float32
    assert np.abs(got - want).max() < 5e-6 * np.abs(want).max()


def test_golden_report_is_within_the_reference_tolerance():
    with open(os.path.join(GOLDEN, "report.json")) as f:
        rep = json.load(f)
    fx = rep["reference_fixture_arch_plain"]
    assert fx["max_abs_diff_plain_vs_fixture"] < 0.002            # test/test_arch.br:35
    assert fx["plain_greedy"] == fx["fixture_greedy"]


def test_rms_norm_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 0.5, 2.0, 1.0], dtype=torch.float64)
    inv = 1.0 / math.sqrt(30.0 / 4 + 1e-6)
    assert torch.allclose(plain.rms_norm(x, w, 1e-6), x * inv * w, atol=1e-12)


def test_rope_position_zero_is_identity_and_norm_is_kept():
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    f = plain.rope_inv_freq(8, 10000.0)
    assert torch.allclose(plain.rope_neox(x[:1], np.array([0]), f), x[:1])
    y = plain.rope_neox(x, np.array([5, 6, 7]), f)
    a = x[..., :4] ** 2 + x[..., 4:] ** 2
    b = y[..., :4] ** 2 + y[..., 4:] ** 2
    assert torch.allclose(a, b, atol=1e-12)
    assert abs(f[0] - 1.0) < 1e-7 and abs(f[1] - 10000.0 ** (-2 / 8)) < 1e-7


def test_attention_of_one_token_is_its_value_and_window_masks():
    q = torch.randn(1, 4, 8, dtype=torch.float64); k = torch.randn(1, 2, 8, dtype=torch.float64)
    v = torch.randn(1, 2, 8, dtype=torch.float64)
    out = plain.gqa_attention(q, k, v, 1 / math.sqrt(8))
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])
    q = torch.randn(6, 1, 4, dtype=torch.float64); k = torch.randn(6, 1, 4, dtype=torch.float64)
    v = torch.eye(6, dtype=torch.float64)[:, None, :4]
    v = torch.randn(6, 1, 4, dtype=torch.float64)
    full = plain.gqa_attention(q, k, v, 0.5)
    win = plain.gqa_attention(q, k, v, 0.5, window=2)
    assert torch.allclose(full[:2], win[:2]) and not torch.allclose(full[3], win[3])
    # with window 2 the last query sees keys 4 and 5 only
    s = torch.tensor([q[5, 0] @ k[4, 0], q[5, 0] @ k[5, 0]]) * 0.5
    p = torch.softmax(s, 0)
    assert torch.allclose(win[5, 0], p[0] * v[4, 0] + p[1] * v[5, 0])


def test_silu_and_swiglu():
    assert plain.silu(torch.tensor(0.0)) == 0.0
    x = torch.randn(2, 3, dtype=torch.float64)
    g, u, d = (torch.randn(5, 3, dtype=torch.float64), torch.randn(5, 3, dtype=torch.float64),
               torch.randn(3, 5, dtype=torch.float64))
    want = ((x @ g.T) * torch.sigmoid(x @ g.T) * (x @ u.T)) @ d.T
    assert torch.allclose(plain.swiglu_ffn(x, g, u, d), want, atol=1e-12)


def test_generator_and_sampler_semantics():
    s = plain.seed_rng(0)
    assert s == 88172645463325252 and plain.seed_rng(5) == 5 ^ 88172645463325252   # src/sampling.br:35-40
    u, s2 = plain.rng_next_f32(s)
    assert 0.0 <= u < 1.0 and s2 != s
    logits = np.array([0.1, 2.0, -1.0, 2.0, 0.5])
    tok, s3 = plain.sample(s, logits, 0.0)
    assert tok == 1 and s3 == s                       # greedy: first maximum, generator untouched
    peaked = np.array([0.0, 0.0, 30.0, 0.0])
    for seed in range(10):
        assert plain.sample(plain.seed_rng(seed), peaked, 0.8)[0] == 2
    for seed in range(20):
        st = plain.seed_rng(seed)
        assert plain.sample(st, logits, 1.0, top_k=2)[0] in (1, 3)
        assert plain.sample(st, logits, 1.0, top_p=0.05)[0] == 1
        assert plain.sample(st, logits, 1.0, min_p=0.9)[0] in (1, 3)
    counts = np.zeros(5)
    st = plain.seed_rng(1)
    for _ in range(4000):
        tok, st = plain.sample(st, logits, 1.0)
        counts[tok] += 1
    p = np.exp(logits - logits.max()); p /= p.sum()
    assert np.abs(counts / 4000 - p).max() < 0.03
