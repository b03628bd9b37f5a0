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


def _call_no_alloc(lib, c, n_splits, H, KV, dh, out):
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    n = c["reqs"].shape[0]
    return lib.bl_attention_decode_no_alloc(
        p(c["q"]), p(c["kc"]), p(c["vc"]), p(c["cu_q"]), p(c["ctx_len"]), p(c["table"]), c["table"].shape[1],
        p(c["reqs"]), n, n_splits, p(out), H, KV, dh, 16, 0, ctypes.c_float(1.0 / math.sqrt(dh)),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_matches_the_allocating_one_twice_in_a_row():
    from boring_llm_b200.kernels import library, ops
    lib = library.load()
    lib.bl_last_error.restype = ctypes.c_char_p
    H, KV, dh = 14, 2, 64
    for seed, n, ctx_lens, n_splits in [(1, 5, [700, 64, 1, 333, 520], 6), (2, 3, [90, 2000, 17], 9)]:
        c = _case(seed, n, H, KV, dh, ctx_lens)
        want = torch.empty_like(c["q"])
        ops.attention_decode(c["q"], c["kc"], c["vc"], c["cu_q"], c["ctx_len"], c["table"], c["reqs"], n_splits, want,
                             H, 0, 1.0 / math.sqrt(dh))
        got = torch.full_like(c["q"], float("nan"))
        assert _call_no_alloc(lib, c, n_splits, H, KV, dh, got) == 0, lib.bl_last_error().decode()
        torch.cuda.synchronize()
        # same kernels, same slices, same order of additions: the tolerance of the kernel tests is generous here
        assert torch.isfinite(got.float()).all()
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 1.6e-2 * max(want.float().abs().max().item(), 1e-6), f"seed {seed}: max |diff| {err:.3e}"
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
