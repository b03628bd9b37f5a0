"""The no-allocation decode attention entry point, called through its exported C symbol the way a C caller
would: its output must equal the allocating entry point's on two calls in a row (the second call finds the
first call's leftovers in the built-in scratch array), and sizes beyond the array must be refused."""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, n, H, KV, dh, ctx_lens):
    g = torch.Generator().manual_seed(seed)
    page = 16
    n_pages = [-(-c // page) for c in ctx_lens]
    total = sum(n_pages) + 3
    perm = torch.randperm(total, generator=g).tolist()
    width = max(n_pages) + 1
    table = np.full((n, width), -1, dtype=np.int32)
    at = 0
    for r in range(n):
        table[r, :n_pages[r]] = perm[at:at + n_pages[r]]
        at += n_pages[r]
    kc = torch.randn(total, KV, page, dh, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(total, KV, page, dh, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(n, H * dh, generator=g).to(torch.bfloat16).to(DEV)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return dict(q=q, kc=kc, vc=vc, table=t(table), cu_q=t(np.arange(n + 1, dtype=np.int32)),
                ctx_len=t(np.array(ctx_lens, dtype=np.int32)), reqs=t(np.arange(n, dtype=np.int32)))


def _call_no_alloc(lib, c, n_splits, H, KV, dh, out, window=0):
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    n = c["reqs"].shape[0]
    return lib.bl_attention_decode_no_alloc(
        p(c["q"]), p(c["kc"]), p(c["vc"]), p(c["cu_q"]), p(c["ctx_len"]), p(c["table"]), c["table"].shape[1],
        p(c["reqs"]), n, n_splits, p(out), H, KV, dh, 16, window, ctypes.c_float(1.0 / math.sqrt(abs(dh))),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _plain(c, r, H, KV, dh, ctx, window):
    """The last query of request r against its keys, by the plain 64-bit attention (whole sequence, no pages)."""
    import plain_model as plain
    table = c["table"][r].cpu().numpy()
    k = torch.stack([c["kc"][int(table[p // 16]), :, p % 16, :] for p in range(ctx)]).double().cpu()
    v = torch.stack([c["vc"][int(table[p // 16]), :, p % 16, :] for p in range(ctx)]).double().cpu()
    q_all = torch.zeros(ctx, H, dh, dtype=torch.float64)
    q_all[-1] = c["q"][r].double().cpu().reshape(H, dh)
    return plain.gqa_attention(q_all, k, v, 1.0 / math.sqrt(dh), window)[-1].reshape(H * dh)


def test_no_alloc_entry_point_matches_the_allocating_one_twice_in_a_row():
    from boring_llm_b200.kernels import library, ops
    lib = library.load()
    lib.bl_last_error.restype = ctypes.c_char_p
    H, KV, dh = 14, 2, 64
    for seed, n, ctx_lens, n_splits, window in [(1, 5, [700, 64, 1, 333, 520], 6, 0), (2, 3, [90, 2000, 17], 9, 0),
                                                (5, 4, [300, 45, 1000, 130], 4, 100)]:
        c = _case(seed, n, H, KV, dh, ctx_lens)
        want = torch.empty_like(c["q"])
        # (with scratch of its own the allocating entry point merges its slices the same way; without, up to 16 slices
        # merge inside a cluster of blocks, with sums in another order)
        own = torch.empty(ops.attention_decode_scratch(n, H, dh, n_splits), dtype=torch.float32, device=DEV)
        ops.attention_decode(c["q"], c["kc"], c["vc"], c["cu_q"], c["ctx_len"], c["table"], c["reqs"], n_splits, want,
                             H, window, 1.0 / math.sqrt(dh), scratch=own)
        got = torch.full_like(c["q"], float("nan"))
        assert _call_no_alloc(lib, c, n_splits, H, KV, dh, got, window) == 0, lib.bl_last_error().decode()
        torch.cuda.synchronize()
        # the same kernel with the same slices and the same order of additions: not one bit may differ
        assert torch.equal(got, want), f"seed {seed}: differs from the allocating entry point"
        # and against the plain implementation, which shares nothing with either (tolerance of the kernel tests)
        for r, ctx in enumerate(ctx_lens):
            ref = _plain(c, r, H, KV, dh, ctx, window)
            err = (got[r].double().cpu() - ref).abs().max().item()
            assert err <= 1.6e-2 * max(ref.abs().max().item(), 1e-6), f"seed {seed} request {r}: max |diff| {err:.3e}"
    # one slice needs no scratch at all
    c = _case(3, 2, H, KV, dh, [40, 100])
    want = torch.empty_like(c["q"]); got = torch.full_like(c["q"], float("nan"))
    ops.attention_decode(c["q"], c["kc"], c["vc"], c["cu_q"], c["ctx_len"], c["table"], c["reqs"], 1, want, H, 0, 1.0 / math.sqrt(dh))
    assert _call_no_alloc(lib, c, 1, H, KV, dh, got) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_no_alloc_entry_point_refuses_sizes_beyond_its_array():
    from boring_llm_b200.kernels import library
    lib = library.load()
    lib.bl_last_error.restype = ctypes.c_char_p
    H, KV, dh = 64, 8, 128
    c = _case(4, 64, H, KV, dh, [32] * 64)
    out = torch.zeros_like(c["q"])
    assert _call_no_alloc(lib, c, 8, H, KV, dh, out) != 0          # 64 * 64 * 8 * 130 floats > 2 Mi
    msg = lib.bl_last_error().decode()
    assert "scratch" in msg and "holds" in msg
    torch.cuda.synchronize()
    assert out.float().abs().max().item() == 0.0                    # nothing ran


def test_no_alloc_entry_point_refuses_more_requests_than_it_has_counters():
    """Tiny heads keep the partial results inside the scratch array while the (request, head group) pairs outgrow
    the 16,384 built-in counters: 4,200 requests x 4 key/value heads. The call must be refused before anything
    is launched (the arrays it is given hold no such batch; a launch would read past them)."""
    from boring_llm_b200.kernels import library
    lib = library.load()
    lib.bl_last_error.restype = ctypes.c_char_p
    H, KV, dh, n = 4, 4, 16, 4200
    c = _case(6, 2, H, KV, dh, [20, 30])
    out = torch.zeros(2, H * dh, dtype=torch.bfloat16, device=DEV)
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    assert n * H * 2 * (dh + 2) <= 2 * 1024 * 1024 and n * KV > 16384
    rc = lib.bl_attention_decode_no_alloc(
        p(c["q"]), p(c["kc"]), p(c["vc"]), p(c["cu_q"]), p(c["ctx_len"]), p(c["table"]), c["table"].shape[1],
        p(c["reqs"]), n, 2, p(out), H, KV, dh, 16, 0, ctypes.c_float(0.25),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and "counters" in lib.bl_last_error().decode()
    torch.cuda.synchronize()
    assert out.float().abs().max().item() == 0.0


def test_no_alloc_entry_point_checks_its_arguments_before_it_computes_with_them():
    """Zero key/value heads with several slices once reached a host-side division; every bad size is an error code."""
    from boring_llm_b200.kernels import library
    lib = library.load()
    lib.bl_last_error.restype = ctypes.c_char_p
    c = _case(7, 2, 4, 2, 32, [20, 30])
    out = torch.zeros_like(c["q"])
    for H, KV, dh, n_splits in [(4, 0, 32, 3), (-4, 2, 32, 3), (4, 2, -32, 3), (4, 3, 32, 3), (4, 2, 32, 0), (4, 2, 32, 300)]:
        assert _call_no_alloc(lib, c, n_splits, H, KV, dh, out) != 0, (H, KV, dh, n_splits)
        assert lib.bl_last_error().decode()
    torch.cuda.synchronize()
    assert out.float().abs().max().item() == 0.0
