"""Each CUDA kernel alone against a plain 64-bit PyTorch restatement of the same formula, at sizes
other than the engine's (odd widths, head sizes in steps of 16, group sizes 1/7/8, ragged pages)."""
import math

import numpy as np
import pytest
import torch

import plain_model as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from boring_llm_b200.kernels import ops as o
    return o


def close(got, want, dtype, what=""):
    tol = 2e-5 if dtype == torch.float32 else 1.6e-2
    got, want = got.double().cpu(), want.double().cpu()
    scale = max(want.abs().max().item(), 1e-6)
    err = (got - want).abs().max().item()
    assert err <= tol * scale, f"{what}: max |diff| {err:.3e} > {tol:.0e} * {scale:.3f}"


def data(shape, salt, dtype=torch.float32):
    """Deterministic values that are not exactly representable in half precision
    (as test/test_math_gpu_real.br:25-31 chooses them)."""
    n = int(np.prod(shape))
    i = torch.arange(n, dtype=torch.float64)
    x = ((i * 7 + salt * 13) % 101) / 101 * 4 - 2
    return x.reshape(shape).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    table = data((77, 100), 1, dtype)
    ids = torch.tensor([0, 76, 5, 5, 33], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 100, device=DEV)
    ops().embed(table, ids, out)
    assert torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("d", [1, 70, 896, 1000])
@pytest.mark.parametrize("wdtype,ydtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                           (torch.float32, torch.bfloat16)])
def test_rmsnorm(d, wdtype, ydtype):
    x = data((9, d), 2) * 3
    w = (data((d,), 3) * 0.25 + 1).to(wdtype)
    y = torch.empty(9, d, dtype=ydtype, device=DEV)
    ops().rmsnorm(x, w, 1e-5, y)
    want = plain.rms_norm(x.double().cpu(), w.double().cpu(), 1e-5)
    close(y, want, ydtype, "rmsnorm")
    idx = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    y2 = torch.empty(3, d, dtype=ydtype, device=DEV)
    ops().rmsnorm(x, w, 1e-5, y2, idx)
    assert torch.equal(y2, y[idx.long()])                 # a row's result does not depend on the row count


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (33, 129, 70), (130, 64, 257), (5, 200, 96)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_plain_epilogues(M, N, K, dtype):
    o = ops()
    x = (data((M, K), 4) * 0.5).to(dtype)
    w = (data((2 * N, K), 5) * 0.25).to(dtype)
    b = (data((N,), 6)).to(dtype)
    xd, wd, bd = x.double().cpu(), w.double().cpu(), b.double().cpu()
    out = torch.empty(M, N, device=DEV)
    o.gemm_plain(x, w[:N].contiguous(), out)
    close(out, xd @ wd[:N].T, torch.float32, "none")
    o.gemm_plain(x, w[:N].contiguous(), out, b, o.EPI_BIAS)
    close(out, xd @ wd[:N].T + bd, torch.float32, "bias")
    res = data((M, N), 7)
    acc = res.clone()
    o.gemm_plain(x, w[:N].contiguous(), acc, None, o.EPI_RESIDUAL)
    close(acc, res.double().cpu() + xd @ wd[:N].T, torch.float32, "residual")
    act = torch.empty(M, N, dtype=dtype, device=DEV)
    o.gemm_plain(x, w, act, None, o.EPI_SWIGLU)
    g, u = xd @ wd[:N].T, xd @ wd[N:].T
    close(act, plain.silu(g) * u, dtype, "swiglu")
    # rows do not depend on how many rows the call has
    one = torch.empty(1, N, device=DEV)
    o.gemm_plain(x[M - 1:M].contiguous(), w[:N].contiguous(), one)
    o.gemm_plain(x, w[:N].contiguous(), out)
    assert torch.equal(one[0], out[M - 1])


def paged_setup(ctx_lens, q_lens, KV, dh, page, dtype, seed, extra_pages=5):
    """Random block tables over a shuffled pool; pages nobody owns and rows past a request's length
    hold large junk that must never be read into a result."""
    rng = np.random.default_rng(seed)
    R = len(ctx_lens)
    n_pages = [-(-c // page) for c in ctx_lens]
    total = sum(n_pages) + extra_pages
    perm = rng.permutation(total)
    width = max(n_pages) + 2
    table = np.full((R, width), -1, dtype=np.int32)
    at = 0
    for r in range(R):
        table[r, :n_pages[r]] = perm[at:at + n_pages[r]]
        at += n_pages[r]
    kc = torch.full((total, KV, page, dh), 1.0e4, dtype=dtype, device=DEV)
    vc = torch.full((total, KV, page, dh), -1.0e4, dtype=dtype, device=DEV)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    T = int(cu[-1])
    tok_req = np.repeat(np.arange(R), q_lens).astype(np.int32)
    positions = np.concatenate([np.arange(c - q, c) for c, q in zip(ctx_lens, q_lens)]).astype(np.int32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return dict(R=R, T=T, table=t(table), table_np=table, kc=kc, vc=vc, cu_q=t(cu), ctx_len=t(np.array(ctx_lens, dtype=np.int32)),
                tok_req=t(tok_req), positions=t(positions), positions_np=positions, tok_req_np=tok_req)


def fill_cache(s, k_full, v_full, page):
    """k_full[r]: [ctx, KV, dh] -> pages."""
    for r, (k, v) in enumerate(zip(k_full, v_full)):
        for p in range(k.shape[0]):
            pg = int(s["table_np"][r, p // page])
            s["kc"][pg, :, p % page, :] = k[p].to(s["kc"].dtype)
            s["vc"][pg, :, p % page, :] = v[p].to(s["vc"].dtype)


def rope_pairs(x, positions, inv_freq, rot, layout):
    """Rotation of the first `rot` dimensions of each head: pairs (j, j + rot/2) or (2j, 2j + 1) (src/math.br:128-157)."""
    if layout == 0:
        return torch.cat([plain.rope_neox(x[..., :rot], positions, inv_freq), x[..., rot:]], dim=-1)
    ang = torch.from_numpy((positions.astype(np.float32)[:, None] * inv_freq[None, :]).astype(np.float64))
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:rot:2], x[..., 1:rot:2]
    out[..., 0:rot:2] = a * c - b * s
    out[..., 1:rot:2] = a * s + b * c
    return out


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,dh,rot", [(4, 2, 16, 16), (7, 1, 48, 48), (8, 8, 64, 32), (2, 1, 128, 128)])
def test_rope_and_cache_write(dtype, H, KV, dh, rot, layout):
    o = ops()
    page = 16
    ctx_lens, q_lens = [5, 40, 17], [5, 9, 1]
    s = paged_setup(ctx_lens, q_lens, KV, dh, page, dtype, 3)
    T = s["T"]
    qkv = data((T, (H + 2 * KV) * dh), 8)
    base = 1.0e6
    j = np.arange(rot // 2, dtype=np.float32)
    inv = np.zeros(dh // 2, dtype=np.float32)
    inv[:rot // 2] = np.float32(1.0) / np.power(np.float32(base), (np.float32(2.0) * j) / np.float32(rot), dtype=np.float32)
    q_out = torch.empty(T, H * dh, dtype=dtype, device=DEV)
    before_k = s["kc"].clone()
    o.rope_kv_write(qkv, s["positions"], s["tok_req"], s["table"], torch.from_numpy(inv).to(DEV), rot // 2, 1.0,
                    q_out, s["kc"], s["vc"], H, KV, dh, layout)
    x = qkv.double().cpu()
    pos = s["positions_np"]

    def rot_ref(t, n_heads):
        return rope_pairs(t.reshape(T, n_heads, dh), pos, inv[:rot // 2], rot, layout)

    q_ref = rot_ref(x[:, :H * dh], H).reshape(T, H * dh)
    k_ref = rot_ref(x[:, H * dh:(H + KV) * dh], KV)
    v_ref = x[:, (H + KV) * dh:].reshape(T, KV, dh)
    close(q_out, q_ref, dtype, "q")
    touched = torch.zeros(s["kc"].shape[0], page, dtype=torch.bool)                  # [pages, rows]
    for t in range(T):
        pg = int(s["table_np"][s["tok_req_np"][t], pos[t] // page]); row = pos[t] % page
        close(s["kc"][pg, :, row, :], k_ref[t], dtype, "k page")
        close(s["vc"][pg, :, row, :], v_ref[t], dtype, "v page")
        touched[pg, row] = True
    # nothing else in the pool was written
    mask = touched.to(DEV)[:, None, :, None].expand_as(s["kc"])
    assert torch.equal(s["kc"][~mask], before_k[~mask])
    # without caches only q is produced
    q2 = torch.empty_like(q_out)
    o.rope_kv_write(qkv, s["positions"], s["tok_req"], s["table"], torch.from_numpy(inv).to(DEV), rot // 2, 1.0,
                    q2, None, None, H, KV, dh, layout)
    assert torch.equal(q2, q_out)


def attention_case(o, fn, dtype, H, KV, dh, ctx_lens, q_lens, window, seed, plant=True):
    page = 16
    s = paged_setup(ctx_lens, q_lens, KV, dh, page, dtype, seed)
    g = torch.Generator().manual_seed(seed)
    k_full = [torch.randn(c, KV, dh, generator=g, dtype=torch.float64) for c in ctx_lens]
    v_full = [torch.randn(c, KV, dh, generator=g, dtype=torch.float64) for c in ctx_lens]
    q_rows = [torch.randn(q, H, dh, generator=g, dtype=torch.float64) for q in q_lens]
    if callable(plant):
        plant(k_full, v_full, q_rows)
    elif plant:
        # one far key per request gets a score that stands out for the last query: a kernel that
        # skips it, reads a neighbour or the wrong page changes the output beyond any tolerance
        for r, c in enumerate(ctx_lens):
            far = 0 if window == 0 else max(0, c - window)       # the first key the last query may see
            k_full[r][far] = 0.0
            k_full[r][far, :, 0] = 6.0
            q_rows[r][-1, :, 0] = 3.0 * math.sqrt(dh)           # its score: 3 sqrt(dh) * 6 / sqrt(dh) = 18
            if window > 0 and far > 0:
                # the key just outside the window would score 30: a window that is one too wide shows
                k_full[r][far - 1] = 0.0
                k_full[r][far - 1, :, 0] = 10.0
    k_full = [k.to(dtype).double() for k in k_full]
    v_full = [v.to(dtype).double() for v in v_full]
    q_rows = [q.to(dtype).double() for q in q_rows]
    fill_cache(s, k_full, v_full, page)
    q = torch.cat([x.reshape(x.shape[0], H * dh) for x in q_rows]).to(dtype).to(DEV)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(dh)
    fn(q, s["kc"], s["vc"], s["tok_req"], s["cu_q"], s["ctx_len"], s["table"], out, H, window, scale)
    at = 0
    for r, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        # whole-sequence plain attention; the chunk's queries are the last n rows
        q_all = torch.zeros(c, H, dh, dtype=torch.float64)
        q_all[c - n:] = q_rows[r]
        want = plain.gqa_attention(q_all, k_full[r], v_full[r], scale, window)[c - n:].reshape(n, H * dh)
        close(out[at:at + n], want, dtype, f"request {r} (ctx {c}, q {n}, window {window})")
        at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,dh", [(4, 2, 16), (7, 1, 64), (8, 1, 128), (3, 3, 48), (2, 1, 256), (14, 2, 64)])
def test_attention_plain_shapes(dtype, H, KV, dh):
    o = ops()
    # decode at 1, 37, 300, 520 keys (test/test_math_gpu_real.br:57-73), chunks over an existing cache with
    # offsets off every tile size, a whole prompt, a two-token portion
    attention_case(o, o.attention_plain, dtype, H, KV, dh, [1, 37, 300, 520], [1, 1, 1, 1], 0, 1)
    attention_case(o, o.attention_plain, dtype, H, KV, dh, [333, 70, 16, 33], [70, 70, 2, 17], 0, 2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [1, 15, 16, 17, 40])
def test_attention_plain_window_edges(dtype, window):
    o = ops()
    attention_case(o, o.attention_plain, dtype, 4, 2, 32, [50, 16, 90, 17], [1, 16, 33, 2], window, 5)


def test_argmax_first_maximum_wins():
    o = ops()
    x = data((6, 1000), 9)
    x[0, 17] = 50; x[0, 900] = 50
    x[1, 999] = 60
    x[2, 0] = 70
    x[3] = -5.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    o.argmax(x, out)
    want = [int(torch.argmax(r).item()) for r in x.cpu()]
    assert out.cpu().tolist()[:3] == [17, 999, 0] and out.cpu().tolist()[3] == 0
    assert out.cpu().tolist()[4:] == want[4:]


@pytest.mark.parametrize("vocab,rows", [(37, 24), (1000, 24), (151936, 24), (5000, 48), (3001, 96), (2000, 192)])
def test_sampler_matches_the_plain_sampler(vocab, rows):
    """Every combination of the cuts against the plain sampler, token for token. The row counts make the launch use
    clusters of 8, 4, 2 blocks and single blocks per row; 3,001 logits are not a multiple of four (scalar loads)."""
    o = ops()
    rng = np.random.default_rng(vocab)
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    logits[5, 10] = logits[5, 20] = logits[5].max() + 1      # exact ties at the top
    temps = np.array([0.0, 0.8, 1.0, 0.3, 2.0, 1.0] * (rows // 6), dtype=np.float32)
    top_k = np.array([0, 0, 40, 5, 0, 2, 0, 1] * (rows // 8), dtype=np.int32)
    top_p = np.array([1.0, 0.9, 1.0, 0.5, 1.0, 1.0, 0.1, 1.0] * (rows // 8), dtype=np.float32)
    min_p = np.array([0.0, 0.0, 0.0, 0.05, 0.2, 0.0] * (rows // 6), dtype=np.float32)
    state = plain.seed_rng(7)
    us = []
    want = []
    for r in range(rows):
        u = 0.0
        if temps[r] > 0:
            before = state
            tok, state = plain.sample(before, logits[r], float(temps[r]), int(top_k[r]), float(top_p[r]), float(min_p[r]))
            u, _ = plain.rng_next_f32(before)
        else:
            tok, _ = plain.sample(state, logits[r], 0.0)
        us.append(u); want.append(tok)
    t = lambda a: torch.from_numpy(a).to(DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    o.sample(t(logits), t(temps), t(top_k), t(top_p), t(min_p), t(np.array(us, dtype=np.float32)), out)
    assert out.cpu().tolist() == want
    out2 = torch.empty_like(out)
    o.sample(t(logits), t(temps), t(top_k), t(top_p), t(min_p), t(np.array(us, dtype=np.float32)), out2)
    assert torch.equal(out, out2)                             # the same on every run


def plain_tokens(logits, temps, top_k, top_p, min_p, seed=7):
    state = plain.seed_rng(seed)
    us, want = [], []
    for r in range(logits.shape[0]):
        u = 0.0
        if temps[r] > 0:
            before = state
            tok, state = plain.sample(before, logits[r], float(temps[r]), int(top_k[r]), float(top_p[r]), float(min_p[r]))
            u, _ = plain.rng_next_f32(before)
        else:
            tok, _ = plain.sample(state, logits[r], 0.0)
        us.append(u); want.append(tok)
    return np.array(us, dtype=np.float32), want


@pytest.mark.parametrize("shape", ["peaked", "equal", "two values", "wide", "steps"])
def test_sampler_on_rows_that_are_not_bell_shaped(shape):
    """Rows that stress the sampler's bucketing: one token far above the rest (everything else in the last
    buckets), all logits equal (one bucket holds the row: the radix fallback, ties by id), two values, a spread
    of hundreds (most weights are zero), and plateaus of equal logits larger than shared memory."""
    o = ops()
    vocab, rows = 20000, 16
    rng = np.random.default_rng(len(shape))
    if shape == "peaked":
        logits = (rng.standard_normal((rows, vocab)) * 0.5).astype(np.float32)
        logits[np.arange(rows), rng.integers(0, vocab, rows)] += 12.0
    elif shape == "equal":
        logits = np.full((rows, vocab), 1.25, dtype=np.float32)
    elif shape == "two values":
        logits = np.where(rng.random((rows, vocab)) < 0.3, 2.0, -1.0).astype(np.float32)
    elif shape == "wide":
        logits = (rng.standard_normal((rows, vocab)) * 120).astype(np.float32)
    else:
        logits = np.floor(rng.standard_normal((rows, vocab)) * 2).astype(np.float32)      # about 15 distinct values
    temps = np.array([0.7, 1.0, 1.5, 0.2] * 4, dtype=np.float32)
    top_k = np.array([0, 0, 50, 6000, 0, 3, 0, 0] * 2, dtype=np.int32)
    top_p = np.array([1.0, 0.9, 1.0, 1.0, 0.45, 0.99, 1.0, 0.7] * 2, dtype=np.float32)     # (not 0.5: half of 20,000 equal weights
    min_p = np.array([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.3, 0.01] * 2, dtype=np.float32)      # is a boundary that 64-bit sums round either way)
    us, want = plain_tokens(logits, temps, top_k, top_p, min_p, seed=11)
    t = lambda a: torch.from_numpy(a).to(DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    o.sample(t(logits), t(temps), t(top_k), t(top_p), t(min_p), t(us), out)
    got = out.cpu().tolist()
    for r in range(rows):
        if got[r] != want[r]:
            # a draw that lands on the boundary between two candidates may fall either way in 32-bit weights: then the
            # two candidates are neighbours in the descending order and the draw is within rounding of the boundary
            order = np.argsort(-logits[r].astype(np.float64), kind="stable").tolist()
            assert abs(order.index(got[r]) - order.index(want[r])) == 1, (shape, r, got[r], want[r])
    assert sum(g != w for g, w in zip(got, want)) <= 1


def test_sampler_distribution():
    o = ops()
    logits = torch.tensor([0.1, 2.0, -1.0, 1.5, 0.5], device=DEV).repeat(4000, 1)
    g = plain.seed_rng(3)
    us = []
    for _ in range(4000):
        u, g = plain.rng_next_f32(g)
        us.append(u)
    n = 4000
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    one = lambda v, dt: torch.full((n,), v, dtype=dt, device=DEV)
    o.sample(logits, one(1.0, torch.float32), one(0, torch.int32), one(1.0, torch.float32), one(0.0, torch.float32),
             torch.tensor(us, device=DEV), out)
    p = torch.softmax(logits[0].double().cpu(), 0)
    freq = torch.bincount(out.cpu().long(), minlength=5).double() / n
    assert (freq - p).abs().max() < 0.03


def test_repeat_penalty():
    o = ops()
    logits = torch.tensor([[1.0, -2.0, 3.0, 0.0], [1.0, -2.0, 3.0, 4.0]], device=DEV)
    o.repeat_penalty(logits, torch.tensor([0, 1, 3, 2], dtype=torch.int32, device=DEV),
                     torch.tensor([0, 3, 4], dtype=torch.int32, device=DEV), torch.tensor([2.0, 1.0], device=DEV))
    assert logits.cpu().tolist() == [[0.5, -4.0, 3.0, 0.0], [1.0, -2.0, 3.0, 4.0]]


def test_kernels_refuse_what_they_cannot_run():
    from boring_llm_b200.kernels import KernelError
    o = ops()
    q = torch.zeros(1, 2 * 272, device=DEV)
    kc = torch.zeros(1, 1, 16, 272, device=DEV)
    i = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="head size"):
        o.attention_plain(q, kc, kc, i, torch.tensor([0, 1], dtype=torch.int32, device=DEV), i + 1, i.view(1, 1), q.clone(), 2, 0, 1.0)
    with pytest.raises(KernelError, match="share"):
        o.attention_plain(torch.zeros(1, 3 * 16, device=DEV), torch.zeros(1, 2, 16, 16, device=DEV),
                          torch.zeros(1, 2, 16, 16, device=DEV), i, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                          i + 1, i.view(1, 1), torch.zeros(1, 48, device=DEV), 3, 0, 1.0)
    with pytest.raises(KernelError, match="contiguous"):
        o.gemm_plain(torch.zeros(4, 8, device=DEV).t(), torch.zeros(3, 4, device=DEV), torch.zeros(8, 3, device=DEV))
    with pytest.raises(KernelError, match="CUDA"):
        o.argmax(torch.zeros(2, 3), torch.zeros(2, dtype=torch.int32))


@pytest.mark.parametrize("M,N,K", [(1, 7, 8), (8, 1152, 896), (5, 200, 96), (17, 129, 80), (33, 64, 264), (64, 4864 // 8, 176),
                                   (100, 50, 64), (3, 9500, 72), (20, 9481, 40), (40, 9600, 64),
                                   (8, 896, 4864), (3, 130, 2056), (8, 2400, 2048), (1, 16, 4096), (7, 1184, 2048),
                                   (16, 896, 4864), (9, 130, 2056), (12, 1184, 2048)])
def test_gemm_skinny_epilogues(M, N, K):
    """(The last shapes have a long K and at most 16 rows: with few column blocks K is cut over the two blocks of a
    cluster, the second handing its sums to the first: 56, 9, 1 and 74 column blocks, a K that is no multiple of 32;
    2,400 columns are too many blocks for that and run the long-K kernel unsplit.)"""
    o = ops()
    dtype = torch.bfloat16
    x = (data((M, K), 14) * 0.5).to(dtype)
    w = (data((2 * N, K), 15) * 0.25).to(dtype)
    b = data((N,), 16)
    xd, wd, bd = x.double().cpu(), w.double().cpu(), b.double().cpu()
    wn = w[:N].contiguous()
    out = torch.empty(M, N, device=DEV)
    o.gemm_skinny(x, wn, out)
    close(out, xd @ wd[:N].T, torch.float32, "none")
    o.gemm_skinny(x, wn, out, b, o.EPI_BIAS)
    close(out, xd @ wd[:N].T + bd, torch.float32, "bias f32")
    o.gemm_skinny(x, wn, out, b.to(dtype), o.EPI_BIAS)
    close(out, xd @ wd[:N].T + b.to(dtype).double().cpu(), torch.float32, "bias bf16")
    res = data((M, N), 17)
    acc = res.clone()
    o.gemm_skinny(x, wn, acc, None, o.EPI_RESIDUAL)
    close(acc, res.double().cpu() + xd @ wd[:N].T, torch.float32, "residual")
    act = torch.empty(M, N, dtype=dtype, device=DEV)
    o.gemm_skinny(x, w, act, None, o.EPI_SWIGLU)
    close(act, plain.silu(xd @ wd[:N].T) * (xd @ wd[N:].T), dtype, "swiglu")
    # a row's result does not depend on the other rows of the call
    one = torch.empty(1, N, device=DEV)
    o.gemm_skinny(x[M - 1:M].contiguous(), wn, one)
    o.gemm_skinny(x, wn, out)
    assert torch.equal(one[0], out[M - 1])
    # and it is the plain kernel's twin (where K is short enough for the plain kernel's one 32-bit chain per output
    # to stay inside this bound itself: at K = 4,864 it is 2.1e-5 of the scale off the 64-bit product, this kernel 1e-5)
    if K <= 1024:
        twin = torch.empty(M, N, device=DEV)
        o.gemm_plain(x, wn, twin)
        close(out, twin.double(), torch.float32, "twin")


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 151936 // 16, 896), (16, 1000, 200), (17, 333, 72), (32, 4100, 896), (5, 130, 8), (33, 700, 136), (64, 2100, 896)])
def test_gemm_tc_cols(M, N, K):
    """The output-head product (W as the M side of tcgen05.mma, persistent blocks, deep ring): tiles that overhang
    N and K, one row and sixty-four, against 64-bit arithmetic; a row does not depend on the other rows."""
    o = ops()
    x = (data((M, K), 31) * 0.5).to(torch.bfloat16)
    w = (data((N, K), 32) * 0.25).to(torch.bfloat16)
    assert o.gemm_tc_cols_supported(x, w)
    want = x.double().cpu() @ w.double().cpu().T
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
        o.gemm_tc_cols(x, w, out)
        o.check_status()
        close(out, want, dtype, f"cols {dtype}")
    out = torch.empty(M, N, device=DEV)
    o.gemm_tc_cols(x, w, out)
    one = torch.empty(1, N, device=DEV)
    o.gemm_tc_cols(x[M - 1:M].contiguous(), w, one)
    assert torch.equal(one[0], out[M - 1])
    twin = torch.empty(M, N, device=DEV)
    o.gemm_plain(x, w, twin)
    close(out, twin.double(), torch.float32, "twin")
    assert not o.gemm_tc_cols_supported(torch.zeros(65, K, dtype=torch.bfloat16, device=DEV), w)
    o.check_status()


def test_gemm_skinny_refuses_unaligned_k():
    from boring_llm_b200.kernels import KernelError
    o = ops()
    x = torch.zeros(2, 12, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(3, 12, dtype=torch.bfloat16, device=DEV)
    assert not o.gemm_skinny_supported(x, w)
    with pytest.raises(KernelError, match="multiple of 8"):
        o.gemm_skinny(x, w, torch.zeros(2, 3, device=DEV))


def mma_attention(q, kc, vc, tok_req, cu_q, ctx_len, table, out, H, window, scale, n_splits=None):
    """Runs the tensor-core kernels the way the attention part does: tiles for requests with several new
    tokens, the decode shape (with slices) for single tokens."""
    o = ops()
    cu = cu_q.cpu().tolist()
    q_lens = [b - a for a, b in zip(cu[:-1], cu[1:])]
    tiles = [(r, t0) for r, n in enumerate(q_lens) if n > 1 for t0 in range(0, n, 64)]
    singles = [r for r, n in enumerate(q_lens) if n == 1]
    out.fill_(float("nan"))
    if tiles:
        o.attention_prefill(q, kc, vc, cu_q, ctx_len, table, torch.tensor(tiles, dtype=torch.int32, device=DEV), out, H, window, scale)
    if singles:
        longest = max(ctx_len.cpu().tolist())
        for splits in ([n_splits] if n_splits else [1, 3, max(1, -(-longest // 64))]):
            o.attention_decode(q, kc, vc, cu_q, ctx_len, table, torch.tensor(singles, dtype=torch.int32, device=DEV),
                               splits, out, H, window, scale)
            if splits != 1:
                ref1 = out.clone()
                o.attention_decode(q, kc, vc, cu_q, ctx_len, table, torch.tensor(singles, dtype=torch.int32, device=DEV),
                                   1, out, H, window, scale)
                assert (out.float() - ref1.float()).abs().max().item() <= 2e-2 * max(1.0, out.float().abs().max().item())


@pytest.mark.parametrize("splits", [2, 5, 8, 13, 16])
@pytest.mark.parametrize("H,KV,dh,window", [(14, 2, 64, 0), (8, 1, 128, 0), (5, 5, 48, 200)])
def test_attention_decode_slices_merged_in_a_cluster(H, KV, dh, window, splits):
    """Up to 16 slices of a request's keys are the blocks of one thread-block cluster and merge their partial results
    through distributed shared memory (no scratch, no ticket); the same slices through scratch memory, and one slice,
    must give the same attention (other order of sums: rounding only), and all must equal the plain attention. Short
    contexts leave slices without keys; a request of one key has fifteen of them."""
    o = ops()

    def clustered(q, kc, vc, tok_req, cu_q, ctx_len, table, out, H_, window_, scale):
        reqs = torch.arange(cu_q.shape[0] - 1, dtype=torch.int32, device=DEV)
        o.attention_decode(q, kc, vc, cu_q, ctx_len, table, reqs, splits, out, H_, window_, scale)
        through_scratch = torch.empty_like(out)
        scratch = torch.empty(o.attention_decode_scratch(reqs.shape[0], H_, q.shape[1] // H_, splits), dtype=torch.float32, device=DEV)
        o.attention_decode(q, kc, vc, cu_q, ctx_len, table, reqs, splits, through_scratch, H_, window_, scale, scratch=scratch)
        assert (out.float() - through_scratch.float()).abs().max().item() <= 1e-2 * max(1.0, out.float().abs().max().item())

    attention_case(o, clustered, torch.bfloat16, H, KV, dh, [1, 37, 300, 1033, 64, 520], [1] * 6, window, 31)


def tma_decode(splits, poison=True):
    """Runs `attention_decode_tma` on the single-token requests of a case. With `poison`, every row of the cache
    that no request owns (free pages, rows past a request's last key) is NaN first: a kernel that lets such a row
    into a sum, even with weight zero, shows it."""
    o = ops()

    def fn(q, kc, vc, tok_req, cu_q, ctx_len, table, out, H, window, scale):
        if poison:
            owned = torch.zeros(kc.shape[0], kc.shape[2], dtype=torch.bool, device=DEV)
            for r, c in enumerate(ctx_len.cpu().tolist()):
                for j in range(c):
                    owned[int(table[r, j // 16]), j % 16] = True
            kc.masked_fill_(~owned[:, None, :, None], float("nan"))
            vc.masked_fill_(~owned[:, None, :, None], float("nan"))
        reqs = torch.arange(cu_q.shape[0] - 1, dtype=torch.int32, device=DEV)
        out.fill_(float("nan"))
        o.attention_decode_tma(q, kc, vc, cu_q, ctx_len, table, reqs, splits, out, H, window, scale)
        o.check_status()
    return fn


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 16])
@pytest.mark.parametrize("H,KV,dh,window", [(14, 2, 64, 0), (8, 1, 128, 0), (7, 7, 64, 0), (24, 2, 64, 0), (40, 2, 128, 0), (28, 4, 128, 0),
                                            (14, 2, 64, 200), (16, 1, 128, 33), (6, 2, 64, 1)])
def test_attention_decode_tma(H, KV, dh, window, splits):
    """The TMA-fed decode attention against the plain attention: 7, 8, 1, 12, 20 and 16 query heads per key/value
    head (one and two n-tiles of heads, two blocks per key/value head), contexts of one key, of one page less and
    more than a unit, of many units per warp, windows that start inside a page and of one key, any number of slices
    (more slices than units leave slices without keys; more slices than heads leave blocks that own no row)."""
    o = ops()
    assert o.attention_decode_tma_supported(torch.bfloat16, dh, 16)
    attention_case(o, tma_decode(splits), torch.bfloat16, H, KV, dh, [1, 37, 300, 1033, 64, 520, 31, 32, 33, 2500], [1] * 10, window, 41)


def test_attention_decode_tma_refuses_other_shapes():
    from boring_llm_b200.kernels import KernelError
    o = ops()
    assert not o.attention_decode_tma_supported(torch.bfloat16, 96, 16)
    assert not o.attention_decode_tma_supported(torch.float32, 64, 16)
    i = torch.zeros(2, dtype=torch.int32, device=DEV)
    q = torch.zeros(1, 2 * 96, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(1, 1, 16, 96, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="head size"):
        o.attention_decode_tma(q, kc, kc, i, i[:1], i.view(2, 1)[:1], i[:1], 1, q.clone(), 2, 0, 1.0)
    q = torch.zeros(1, 2 * 64, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(1, 1, 16, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="slices"):
        o.attention_decode_tma(q, kc, kc, i, i[:1], i.view(2, 1)[:1], i[:1], 17, q.clone(), 2, 0, 1.0)


@pytest.mark.parametrize("H,KV,dh", [(4, 2, 16), (7, 1, 64), (8, 1, 128), (3, 3, 48), (14, 2, 64), (6, 2, 32), (34, 2, 96)])
def test_attention_mma_shapes(H, KV, dh):
    o = ops()
    assert o.attention_mma_supported(torch.bfloat16, dh, 16)
    attention_case(o, mma_attention, torch.bfloat16, H, KV, dh, [1, 37, 300, 520], [1, 1, 1, 1], 0, 1)
    attention_case(o, mma_attention, torch.bfloat16, H, KV, dh, [333, 70, 16, 33], [70, 70, 2, 17], 0, 2)
    attention_case(o, mma_attention, torch.bfloat16, H, KV, dh, [64, 65, 128, 200, 129], [64, 1, 128, 1, 65], 0, 3)


@pytest.mark.parametrize("window", [1, 15, 16, 17, 40, 64, 100])
def test_attention_mma_window_edges(window):
    o = ops()
    attention_case(o, mma_attention, torch.bfloat16, 4, 2, 32, [50, 16, 90, 17, 300], [1, 16, 33, 2, 1], window, 5)
    attention_case(o, mma_attention, torch.bfloat16, 4, 2, 64, [200, 131], [150, 1], window, 6)


def tc_attention(q, kc, vc, tok_req, cu_q, ctx_len, table, out, H, window, scale):
    """The tcgen05 prefill kernel for requests with several new tokens (tiles of 128 rows), the decode kernel for the rest."""
    o = ops()
    cu = cu_q.cpu().tolist()
    q_lens = [b - a for a, b in zip(cu[:-1], cu[1:])]
    from boring_llm_b200.parts.attention import tc_attention_tiles
    ctx_lens = ctx_len.cpu().tolist()
    tiles = tc_attention_tiles(q_lens, ctx_lens)
    singles = [r for r, n in enumerate(q_lens) if n == 1]
    out.fill_(float("nan"))
    if tiles:
        o.attention_prefill_tc(q, kc, vc, cu_q, ctx_len, table, torch.tensor(tiles, dtype=torch.int32, device=DEV), out, H, window, scale)
        o.check_status()
    if singles:
        o.attention_decode(q, kc, vc, cu_q, ctx_len, table, torch.tensor(singles, dtype=torch.int32, device=DEV), 1, out, H, window, scale)


@pytest.mark.parametrize("dh", [64, 128])
@pytest.mark.parametrize("H,KV", [(14, 2), (7, 1), (4, 4)])
def test_attention_tcgen05_shapes(H, KV, dh):
    """Prefill attention on tcgen05, head sizes 64 (two groups of row warps) and 128 (one group, two atoms of 64
    dimensions): portions over an existing cache with offsets off every tile and page size, whole prompts of several
    key blocks, rows past the end of a tile, several requests in one launch, portions from 2 to 600 tokens."""
    o = ops()
    assert o.attention_prefill_tc_supported(torch.bfloat16, 64, 16)
    assert o.attention_prefill_tc_supported(torch.bfloat16, 128, 16)
    assert not o.attention_prefill_tc_supported(torch.bfloat16, 96, 16)
    assert not o.attention_prefill_tc_supported(torch.float32, 64, 16)
    attention_case(o, tc_attention, torch.bfloat16, H, KV, dh, [333, 70, 16, 33], [70, 70, 2, 17], 0, 2)
    attention_case(o, tc_attention, torch.bfloat16, H, KV, dh, [64, 65, 128, 200, 129], [64, 1, 128, 1, 65], 0, 3)
    attention_case(o, tc_attention, torch.bfloat16, H, KV, dh, [1000, 515, 257], [1000, 300, 129], 0, 4)
    attention_case(o, tc_attention, torch.bfloat16, H, KV, dh, [900, 602, 450, 131], [600, 2, 33, 130], 0, 5)


@pytest.mark.parametrize("dh", [64, 128])
def test_attention_tcgen05_long_prompt(dh):
    """Twenty key blocks and ten row blocks: the rings of keys, values, P and output shares wrap around many times,
    and a planted key at position 0 decides the last row."""
    o = ops()
    attention_case(o, tc_attention, torch.bfloat16, 4, 2, dh, [2500, 1400], [2500, 700], 0, 8)
    attention_case(o, tc_attention, torch.bfloat16, 2, 1, dh, [3000], [1300], 1100, 9)


@pytest.mark.parametrize("dh", [64, 128])
@pytest.mark.parametrize("window", [1, 15, 16, 17, 100, 128, 200])
def test_attention_tcgen05_window_edges(window, dh):
    o = ops()
    attention_case(o, tc_attention, torch.bfloat16, 4, 2, dh, [200, 131, 700, 17], [150, 1, 500, 2], window, 6)


@pytest.mark.parametrize("dh", [64, 128])
def test_attention_tcgen05_moving_maximum(dh):
    """The output accumulates in tensor memory against a reference maximum that is moved only when a key block's
    maximum exceeds it by 2^8, and moving it rescales what has accumulated. Keys planted along the prompt score higher
    and higher for every query: by 17 (in powers of two) at keys 300, 700, 1,100, 1,500 and 1,900, which moves the
    reference in even and in odd key blocks after many blocks have been added, and by 4 at keys 450 and 1,300, which
    does not (those rows' weights exceed 1). Every planted key has its own value vector, so a rescale that is
    skipped, done twice or done with the wrong factor changes the output wholesale."""
    o = ops()
    at = {5: 0.5, 300: 1.5, 450: 1.85, 700: 3.0, 1100: 4.5, 1300: 4.85, 1500: 6.0, 1900: 7.5}

    def plant(k_full, v_full, q_rows):
        for r in range(len(k_full)):
            q_rows[r][:, :, 0] = math.sqrt(dh)                    # score of a planted key: 8 x its strength
            k_full[r][:, :, 0] = 0.0
            for pos, strength in at.items():
                if pos < k_full[r].shape[0]:
                    k_full[r][pos] = 0.0
                    k_full[r][pos, :, 0] = 8.0 * strength
                    v_full[r][pos] = 0.0
                    v_full[r][pos, :, pos % dh] = 30.0
    attention_case(o, tc_attention, torch.bfloat16, 4, 2, dh, [2100, 1400, 2048], [2100, 900, 333], 0, 21, plant=plant)
    attention_case(o, tc_attention, torch.bfloat16, 2, 1, dh, [2000], [2000], 500, 22, plant=plant)


def test_attention_tcgen05_padded_tile_lists():
    """The tile list of a step that is replayed is padded with tiles of a request without tokens: such blocks must
    leave at once and write nothing (no copy may be left in flight when they do)."""
    o = ops()
    for dh in (64, 128):
        s = paged_setup([300, 40, 1], [200, 40, 0], 2, dh, 16, torch.bfloat16, 12)
        g = torch.Generator().manual_seed(5)
        s["kc"].copy_(torch.randn(s["kc"].shape, generator=g).to(DEV)); s["vc"].copy_(torch.randn(s["vc"].shape, generator=g).to(DEV))
        q = torch.randn(240, 4 * dh, generator=g).to(torch.bfloat16).to(DEV)
        want, got = torch.full_like(q, 7.0), torch.full_like(q, 7.0)
        tiles = [[0, 0], [0, 128], [1, 0]]
        padded = [[2, 0]] * 5 + tiles
        t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        o.attention_prefill_tc(q, s["kc"], s["vc"], s["cu_q"], s["ctx_len"], s["table"], t(tiles), want, 4, 0, dh ** -0.5)
        o.attention_prefill_tc(q, s["kc"], s["vc"], s["cu_q"], s["ctx_len"], s["table"], t(padded), got, 4, 0, dh ** -0.5)
        o.check_status()
        assert torch.equal(got, want) and not (got == 7.0).all()


def test_attention_mma_is_refused_where_it_is_not_built():
    from boring_llm_b200.kernels import KernelError
    o = ops()
    assert not o.attention_mma_supported(torch.bfloat16, 80, 16)
    assert not o.attention_mma_supported(torch.bfloat16, 64, 32)
    assert not o.attention_mma_supported(torch.float32, 64, 16)
    i = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = torch.zeros(1, 80, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(1, 1, 16, 80, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="head size 80"):
        o.attention_decode(q, kc, kc, torch.tensor([0, 1], dtype=torch.int32, device=DEV), i + 1, i.view(1, 1), i, 1,
                           q.clone(), 1, 0, 1.0)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (1, 7, 8), (130, 200, 96), (257, 129, 264), (300, 608, 176),
                                   (2048, 1152, 896), (65, 896, 4864), (500, 320, 200), (64, 4864, 896), (512, 896, 448)])
@pytest.mark.parametrize("pair", [False, True, "splitk"])
def test_gemm_tc_epilogues(M, N, K, pair):
    """The tcgen05 products (one block per 128 x 128 tile; a pair of blocks per 256 x 256 tile; a cluster of blocks
    that cut K among them per 128 x 64 or 128 x 128 tile) against 64-bit arithmetic and against their plain twin: tiles
    that overhang M, N and K, one k block and seventy-six, every epilogue."""
    o = ops()
    gemm_tc = o.gemm_tc_splitk if pair == "splitk" else o.gemm_tc_pair if pair else o.gemm_tc
    dtype = torch.bfloat16
    x = (data((M, K), 24) * 0.5).to(dtype)
    w = (data((2 * N, K), 25) * 0.25).to(dtype)
    b = data((N,), 26)
    xd, wd, bd = x.double().cpu(), w.double().cpu(), b.double().cpu()
    wn = w[:N].contiguous()
    out = torch.full((M, N), float("nan"), device=DEV)
    gemm_tc(x, wn, out)
    o.check_status()
    close(out, xd @ wd[:N].T, torch.float32, "none")
    twin = torch.empty(M, N, device=DEV)
    o.gemm_plain(x, wn, twin)
    close(out, twin.double(), torch.float32, "twin")
    gemm_tc(x, wn, out, b, o.EPI_BIAS)
    close(out, xd @ wd[:N].T + bd, torch.float32, "bias")
    res = data((M, N), 27)
    acc = res.clone()
    gemm_tc(x, wn, acc, None, o.EPI_RESIDUAL)
    close(acc, res.double().cpu() + xd @ wd[:N].T, torch.float32, "residual")
    act = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
    gemm_tc(x, w, act, None, o.EPI_SWIGLU)
    close(act, plain.silu(xd @ wd[:N].T) * (xd @ wd[N:].T), dtype, "swiglu")
    half = torch.empty(M, N, dtype=dtype, device=DEV)
    gemm_tc(x, wn, half)
    close(half, xd @ wd[:N].T, dtype, "bfloat16 output")
    o.check_status()


@pytest.mark.parametrize("M,N,K", [(1, 7, 8), (8, 4864 // 16, 896), (17, 129, 96), (33, 50, 200), (64, 80, 264), (5, 1000, 80)])
def test_norm_gemm_fused(M, N, K):
    """The fused norm + product kernels against 64-bit arithmetic (the norm's output rounded to bfloat16, as
    the unfused kernels store it) and against the unfused kernels."""
    o = ops()
    bf = torch.bfloat16
    rows = M + 3
    x = data((rows, K), 31) * 3
    nw = (data((K,), 32) * 0.25 + 1).to(bf)
    w = (data((2 * N, K), 33) * 0.25).to(bf)
    b = data((N,), 34)
    idx = torch.tensor([(i * 7) % rows for i in range(M)], dtype=torch.int32, device=DEV)
    xs = x[idx.long()].contiguous()
    h = plain.round_bf16(plain.rms_norm(xs.double().cpu(), nw.double().cpu(), 1e-5))
    wd = w.double().cpu()
    wn = w[:N].contiguous()
    out = torch.full((M, N), float("nan"), device=DEV)
    o.norm_gemm(xs, nw, 1e-5, wn, out)
    close(out, h @ wd[:N].T, torch.float32, "plain")
    o.norm_gemm(x, nw, 1e-5, wn, out, None, o.EPI_NONE, idx)
    close(out, h @ wd[:N].T, torch.float32, "gathered rows")
    o.norm_gemm(xs, nw, 1e-5, wn, out, b, o.EPI_BIAS)
    close(out, h @ wd[:N].T + b.double().cpu(), torch.float32, "bias")
    act = torch.full((M, N), float("nan"), dtype=bf, device=DEV)
    o.norm_gemm(xs, nw, 1e-5, w, act, None, o.EPI_SWIGLU)
    close(act, plain.silu(h @ wd[:N].T) * (h @ wd[N:].T), bf, "swiglu")
    # the unfused twins
    hb = torch.empty(M, K, dtype=bf, device=DEV)
    o.rmsnorm(xs, nw, 1e-5, hb)
    twin = torch.empty(M, N, device=DEV)
    o.gemm_plain(hb, wn, twin)
    o.norm_gemm(xs, nw, 1e-5, wn, out)
    close(out, twin.double(), torch.float32, "twin")
    one = torch.empty(1, N, device=DEV)
    o.norm_gemm(xs[M - 1:M].contiguous(), nw, 1e-5, wn, one)
    assert torch.equal(one[0], out[M - 1])            # a row does not depend on the rows beside it


@pytest.mark.parametrize("H,KV,dh,d", [(4, 2, 16, 64), (3, 1, 32, 96), (5, 5, 48, 80), (14, 2, 64, 896), (2, 1, 128, 200)])
@pytest.mark.parametrize("bias,layout", [(True, 0), (False, 0), (True, 1)])
def test_norm_qkv_rope_fused(H, KV, dh, d, bias, layout):
    """One launch against the three kernels it replaces (norm, joined product with bias, rotation + cache write)."""
    o = ops()
    bf = torch.bfloat16
    page = 16
    ctx_lens, q_lens = [5, 40, 17, 300], [5, 9, 1, 1]
    s = paged_setup(ctx_lens, q_lens, KV, dh, page, bf, 9)
    s2 = paged_setup(ctx_lens, q_lens, KV, dh, page, bf, 9)
    before_k, before_v = s2["kc"].clone(), s2["vc"].clone()
    T = s["T"]
    x = data((T, d), 41) * 2
    nw = (data((d,), 42) * 0.25 + 1).to(bf)
    w = (data(((H + 2 * KV) * dh, d), 43) * 0.2).to(bf)
    b = (data(((H + 2 * KV) * dh,), 44) * 0.5).to(bf) if bias else None
    j = np.arange(dh // 2, dtype=np.float32)
    inv = torch.from_numpy(np.float32(1.0) / np.power(np.float32(1.0e4), (np.float32(2.0) * j) / np.float32(dh), dtype=np.float32)).to(DEV)
    # unfused
    h = torch.empty(T, d, dtype=bf, device=DEV)
    o.rmsnorm(x, nw, 1e-6, h)
    qkv = torch.empty(T, (H + 2 * KV) * dh, device=DEV)
    o.gemm_plain(h, w, qkv, b, o.EPI_BIAS if bias else o.EPI_NONE)
    q_ref = torch.empty(T, H * dh, dtype=bf, device=DEV)
    o.rope_kv_write(qkv, s["positions"], s["tok_req"], s["table"], inv, dh // 2, 1.0, q_ref, s["kc"], s["vc"], H, KV, dh, layout)
    # fused
    q = torch.full((T, H * dh), float("nan"), dtype=bf, device=DEV)
    o.norm_qkv_rope(x, nw, 1e-6, w, b, s2["positions"], s2["tok_req"], s2["table"], inv, 1.0, q, s2["kc"], s2["vc"], H, KV, dh, layout)
    close(q, q_ref.double(), bf, "q")
    # the rows that the step's tokens own, one by one (the pools are full of +-1e4 junk, which would set the scale of
    # a comparison of whole pools so high that a key in the wrong row, or no key at all, would pass) ...
    touched = torch.zeros(s["kc"].shape[0], page, dtype=torch.bool)
    for t in range(T):
        pg = int(s["table_np"][s["tok_req_np"][t], s["positions_np"][t] // page]); row = int(s["positions_np"][t]) % page
        close(s2["kc"][pg, :, row, :], s["kc"][pg, :, row, :].double(), bf, f"key of token {t}")
        close(s2["vc"][pg, :, row, :], s["vc"][pg, :, row, :].double(), bf, f"value of token {t}")
        assert s["kc"][pg, :, row, :].abs().max().item() < 1.0e3, "the unfused kernels did not write this row either"
        touched[pg, row] = True
    # ... and every other row of both pools still holds its junk
    mask = touched.to(DEV)[:, None, :, None].expand_as(s2["kc"])
    assert torch.equal(s2["kc"][~mask], before_k[~mask]) and torch.equal(s2["vc"][~mask], before_v[~mask])
    q_only = torch.empty_like(q)
    o.norm_qkv_rope(x, nw, 1e-6, w, b, s2["positions"], s2["tok_req"], s2["table"], inv, 1.0, q_only, None, None, H, KV, dh, layout)
    assert torch.equal(q_only, q)


@pytest.mark.parametrize("H,KV,dh,d,bias", [(14, 2, 64, 896, True), (6, 2, 64, 136, False), (2, 1, 128, 200, True), (16, 2, 128, 264, True), (3, 3, 64, 72, True)])
def test_qkv_rope_in_the_epilogue_of_the_tcgen05_product(H, KV, dh, d, bias):
    """The joined q/k/v product on pairs of SMs with bias, rotation and the writes of q, k and v in its epilogue,
    against the three kernels it replaces (product with bias, rotation + cache write) and their float64 formulas:
    prompts of several requests over existing caches, 700 rows (tiles that overhang M), heads that sit in the same
    128-column tile as the first key head, and the untouched rest of both pools."""
    o = ops()
    bf = torch.bfloat16
    page = 16
    ctx_lens, q_lens = [300, 640, 77, 1], [300, 333, 66, 1]
    s = paged_setup(ctx_lens, q_lens, KV, dh, page, bf, 9)
    s2 = paged_setup(ctx_lens, q_lens, KV, dh, page, bf, 9)
    before_k, before_v = s2["kc"].clone(), s2["vc"].clone()
    T = s["T"]
    x = (data((T, d), 41) * 0.5).to(bf)
    w = (data(((H + 2 * KV) * dh, d), 43) * 0.2).to(bf)
    b = (data(((H + 2 * KV) * dh,), 44) * 0.5).to(bf) if bias else None
    assert o.qkv_rope_tc_supported(x, w, H, KV, dh, page)
    j = np.arange(dh // 2, dtype=np.float32)
    inv = torch.from_numpy(np.float32(1.0) / np.power(np.float32(1.0e4), (np.float32(2.0) * j) / np.float32(dh), dtype=np.float32)).to(DEV)
    # unfused
    qkv = torch.empty(T, (H + 2 * KV) * dh, device=DEV)
    o.gemm_plain(x, w, qkv, b, o.EPI_BIAS if bias else o.EPI_NONE)
    q_ref = torch.empty(T, H * dh, dtype=bf, device=DEV)
    o.rope_kv_write(qkv, s["positions"], s["tok_req"], s["table"], inv, dh // 2, 0.75, q_ref, s["kc"], s["vc"], H, KV, dh, 0)
    # the table holds what the kernels that rotate on the fly work out
    cs, sn = o.rope_table(s2["positions"], inv, dh // 2, 0.75)
    ang = s2["positions"].cpu().float()[:, None] * inv.cpu()[None, :]
    assert torch.allclose(cs.cpu(), torch.cos(ang.double()).float() * 0.75, atol=2e-6)
    assert torch.allclose(sn.cpu(), torch.sin(ang.double()).float() * 0.75, atol=2e-6)
    # fused
    q = torch.full((T, H * dh), float("nan"), dtype=bf, device=DEV)
    o.qkv_rope_tc(x, w, b, s2["positions"], s2["tok_req"], s2["table"], cs, sn, q, s2["kc"], s2["vc"], H, KV, dh)
    o.check_status()
    close(q, q_ref.double(), bf, "q")
    # against the formulas: q of one row
    xd, wd = x.double().cpu(), w.double().cpu()
    t_chk = T - 2
    row = xd[t_chk] @ wd.T + (b.double().cpu() if bias else 0.0)
    qh = row[:H * dh].view(1, H, dh)
    want = plain.rope_neox(qh, s["positions_np"][t_chk:t_chk + 1], inv.cpu().numpy()) * 1.0
    # (the scale of cos and sin, 0.75, multiplies the rotated head)
    close(q[t_chk].view(1, H, dh), want * 0.75, bf, "q against the formula")
    touched = torch.zeros(s["kc"].shape[0], page, dtype=torch.bool)
    rows_k = torch.empty(T, KV, dh, dtype=bf, device=DEV); rows_k2 = torch.empty_like(rows_k)
    rows_v = torch.empty_like(rows_k); rows_v2 = torch.empty_like(rows_k)
    for t in range(T):
        pg = int(s["table_np"][s["tok_req_np"][t], s["positions_np"][t] // page]); r = int(s["positions_np"][t]) % page
        rows_k[t], rows_k2[t], rows_v[t], rows_v2[t] = s["kc"][pg, :, r, :], s2["kc"][pg, :, r, :], s["vc"][pg, :, r, :], s2["vc"][pg, :, r, :]
        touched[pg, r] = True
    assert rows_k.abs().max().item() < 1.0e3, "the unfused kernels did not write these rows either"
    close(rows_k2, rows_k.double(), bf, "keys")
    close(rows_v2, rows_v.double(), bf, "values")
    mask = touched.to(DEV)[:, None, :, None].expand_as(s2["kc"])
    assert torch.equal(s2["kc"][~mask], before_k[~mask]) and torch.equal(s2["vc"][~mask], before_v[~mask])
    q_only = torch.empty_like(q)
    o.qkv_rope_tc(x, w, b, s2["positions"], s2["tok_req"], s2["table"], cs, sn, q_only, None, None, H, KV, dh)
    assert torch.equal(q_only, q)
    o.check_status()


@pytest.mark.parametrize("M,N,K,F", [(2048, 896, 896, 1216), (700, 136, 264, 200), (300, 2048, 128, 320), (1500, 64, 72, 96)])
def test_rms_norm_shared_between_two_products(M, N, K, F):
    """The product that adds into the residual stream leaves the next RMS norm pending (rows times the norm's weight
    in bfloat16, sums of squares by tile), and the products that read the normed rows finish it in their epilogues:
    against the plain kernels (product, norm, product) and the float64 formulas, with 256- and 128-column tiles,
    rows and columns that overhang the tiles, and a row of zeros."""
    o = ops()
    bf = torch.bfloat16
    x = (data((M, K), 51) * 0.5).to(bf)
    w = (data((N, K), 52) * 0.2).to(bf)
    stream = data((M, N), 53) * 2
    stream[5] = 0.0
    x[5] = 0.0                                                # a row whose new stream is all zeros: scale 1 / sqrt(eps)
    nw = (data((N,), 54) * 0.25 + 1).to(bf)
    eps = 1e-5
    assert o.gemm_on_pairs(x, w, N, o.EPI_RESIDUAL)
    # the plain way
    ref = stream.clone()
    o.gemm_tc_pair(x, w, ref, None, o.EPI_RESIDUAL)
    h_ref = torch.empty(M, N, dtype=bf, device=DEV)
    o.rmsnorm(ref, nw, eps, h_ref)
    # the shared way
    out = stream.clone()
    hw, ss = o.gemm_residual_norm(x, w, out, nw)
    o.check_status()
    assert torch.equal(out, ref)                              # the stream itself is what the residual epilogue writes
    want = out.double().cpu()
    close(hw, want * nw.double().cpu(), bf, "stream times weight")
    close(ss.sum(dim=1), (want * want).sum(dim=1), torch.float32, "sums of squares")
    scale = torch.rsqrt((want * want).mean(dim=1) + eps)
    # SwiGLU over the pending rows against SwiGLU over the normed rows
    wg = (data((2 * F, N), 55) * 0.1).to(bf)
    act = torch.full((M, F), float("nan"), dtype=bf, device=DEV)
    o.gemm_swiglu_scaled(hw, wg, act, ss, eps)
    o.check_status()
    act_ref = torch.empty(M, F, dtype=bf, device=DEV)
    o.gemm_tc_pair(h_ref, wg, act_ref, None, o.EPI_SWIGLU)
    h64 = want * scale[:, None] * nw.double().cpu()
    wgd = wg.double().cpu()
    formula = plain.silu(h64 @ wgd[:F].T) * (h64 @ wgd[F:].T)
    close(act_ref, formula, bf, "SwiGLU of the normed rows (the kernels as they were)")
    close(act, formula, bf, "SwiGLU that finishes the norm")


@pytest.mark.parametrize("M,N,K,F", [(8, 896, 896, 4864), (1, 896, 4864, 304), (13, 136, 264, 72), (16, 2048, 2048, 640), (3, 40, 64, 24)])
def test_rms_norm_shared_between_two_products_of_a_decode_step(M, N, K, F):
    """The same on the register-streaming kernel (steps of up to 16 rows): the residual epilogue writes the stream, the
    stream times the next norm's weight in bfloat16 and each row's sums of squares by block of 16 columns; the product
    that reads those rows scales its sums by the rows' 1 / sqrt(mean + eps). Against the kernels as they were
    (product, norm, product), and the float64 formulas; widths that are no multiple of 16, one row, a row of zeros,
    the long-K form of the kernel (16 warps)."""
    o = ops()
    bf = torch.bfloat16
    x = (data((M, K), 51) * 0.5).to(bf)
    w = (data((N, K), 52) * 0.2).to(bf)
    stream = data((M, N), 53) * 2
    if M > 2:
        stream[2] = 0.0
        x[2] = 0.0                                            # a row whose new stream is all zeros: scale 1 / sqrt(eps)
    nw = (data((N,), 54) * 0.25 + 1).to(bf)
    eps = 1e-5
    assert o.gemm_skinny_links_norm(x, w, N, o.EPI_RESIDUAL) == (M >= 2)      # (the kernels take one row; the dispatch does not send it)
    ref = stream.clone()
    o.gemm_skinny(x, w, ref, None, o.EPI_RESIDUAL)
    h_ref = torch.empty(M, N, dtype=bf, device=DEV)
    o.rmsnorm(ref, nw, eps, h_ref)
    out = stream.clone()
    hw, ss = o.gemm_skinny_residual_norm(x, w, out, nw)
    assert torch.equal(out, ref)                              # the stream itself is what the residual epilogue writes
    assert ss.shape == (M, -(-N // 16))
    want = out.double().cpu()
    close(hw, want * nw.double().cpu(), bf, "stream times weight")
    close(ss.sum(dim=1), (want * want).sum(dim=1), torch.float32, "sums of squares")
    col = torch.arange(N) // 16
    by_block = torch.zeros(M, ss.shape[1], dtype=torch.float64).index_add_(1, col, want * want)
    close(ss, by_block, torch.float32, "sums of squares by block of 16 columns")
    scale = torch.rsqrt((want * want).mean(dim=1) + eps)
    h64 = want * scale[:, None] * nw.double().cpu()
    # SwiGLU over the pending rows against SwiGLU over the normed rows
    wg = (data((2 * F, N), 55) * 0.1).to(bf)
    act = torch.full((M, F), float("nan"), dtype=bf, device=DEV)
    o.gemm_skinny_scaled(hw, wg, act, ss, eps, None, o.EPI_SWIGLU)
    act_ref = torch.empty(M, F, dtype=bf, device=DEV)
    o.gemm_skinny(h_ref, wg, act_ref, None, o.EPI_SWIGLU)
    wgd = wg.double().cpu()
    formula = plain.silu(h64 @ wgd[:F].T) * (h64 @ wgd[F:].T)
    close(act_ref, formula, bf, "SwiGLU of the normed rows (the kernels as they were)")
    close(act, formula, bf, "SwiGLU that finishes the norm")
    # a plain product with a bias, 32-bit out
    b = data((F,), 56)
    y = torch.full((M, F), float("nan"), dtype=torch.float32, device=DEV)
    o.gemm_skinny_scaled(hw, wg[:F].contiguous(), y, ss, eps, b, o.EPI_BIAS)
    close(y, h64 @ wgd[:F].T + b.double().cpu(), bf, "product with bias that finishes the norm")


def test_qkv_product_finishes_a_pending_norm():
    """`qkv_rope_tc` with `row_sums`: q, keys and values equal those from the normed rows (norm kernel, then the same
    product) within bfloat16 rounding, and the float64 formula for q."""
    o = ops()
    bf = torch.bfloat16
    H, KV, dh, d, page = 6, 2, 64, 136, 16
    ctx_lens, q_lens = [400, 300], [400, 290]
    s = paged_setup(ctx_lens, q_lens, KV, dh, page, bf, 9)
    s2 = paged_setup(ctx_lens, q_lens, KV, dh, page, bf, 9)
    T = s["T"]
    stream = data((T, d), 61) * 3
    nw = (data((d,), 62) * 0.25 + 1).to(bf)
    w = (data(((H + 2 * KV) * dh, d), 63) * 0.2).to(bf)
    b = (data(((H + 2 * KV) * dh,), 64) * 0.5).to(bf)
    eps = 1e-6
    inv = torch.from_numpy(np.float32(1.0) / np.power(np.float32(1.0e4), (np.float32(2.0) * np.arange(dh // 2, dtype=np.float32)) / np.float32(dh), dtype=np.float32)).to(DEV)
    cs, sn = o.rope_table(s["positions"], inv, dh // 2, 1.0)
    # what the product before would leave: the stream times the weight, and its rows' sums of squares in three parts
    hw = (stream * nw.float()).to(bf)
    sq = (stream * stream)
    ss = torch.stack([sq[:, :40].sum(1), sq[:, 40:100].sum(1), sq[:, 100:].sum(1)], dim=1).contiguous()
    h = torch.empty(T, d, dtype=bf, device=DEV)
    o.rmsnorm(stream, nw, eps, h)
    q_ref = torch.empty(T, H * dh, dtype=bf, device=DEV)
    o.qkv_rope_tc(h, w, b, s["positions"], s["tok_req"], s["table"], cs, sn, q_ref, s["kc"], s["vc"], H, KV, dh)
    q = torch.full((T, H * dh), float("nan"), dtype=bf, device=DEV)
    o.qkv_rope_tc(hw, w, b, s2["positions"], s2["tok_req"], s2["table"], cs, sn, q, s2["kc"], s2["vc"], H, KV, dh, row_sums=ss, eps=eps)
    o.check_status()
    sd = stream.double().cpu()
    h64 = sd * torch.rsqrt((sd * sd).mean(1, keepdim=True) + eps) * nw.double().cpu()
    row = h64 @ w.double().cpu().T + b.double().cpu()
    want = plain.rope_neox(row[:, :H * dh].view(T, H, dh), s["positions_np"], inv.cpu().numpy()).reshape(T, H * dh)
    close(q_ref, want, bf, "q from the normed rows")
    close(q, want, bf, "q from the pending rows")
    owned = torch.zeros(s["kc"].shape[0], page, dtype=torch.bool)
    for t in range(T):
        owned[int(s["table_np"][s["tok_req_np"][t], s["positions_np"][t] // page]), int(s["positions_np"][t]) % page] = True
    mask = owned.to(DEV)[:, None, :, None].expand_as(s["kc"])
    close(s2["kc"][mask], s["kc"][mask].double(), bf, "keys")
    close(s2["vc"][mask], s["vc"][mask].double(), bf, "values")
    assert torch.equal(s2["kc"][~mask], s["kc"][~mask])
