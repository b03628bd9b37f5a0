"""Trace replay against the plain implementation: each request alone and whole; most of it in one step
and the last 32 tokens one by one; in portions of changing size down to two tokens; and mixed, up to
four live requests with portions of some beside single tokens of others and so few pages that they
are used again. In float32 and in bfloat16, for three tiny configurations."""
import os

import numpy as np
import torch
import pytest

import helpers

pytestmark = pytest.mark.gpu

# prompts + continuations, as lengths: a one-token prompt, lengths off every page edge, one over 4 pages
LENGTHS = {"A": [7 + 8, 16 + 8, 33 + 8, 70], "B": [1 + 12, 5 + 12, 19 + 12, 64 + 12], "C": [3, 45, 64, 90],
           "D": [300, 131, 260, 17]}


def requests_for(name):
    vocab = helpers.TINY[name]["vocab_size"]
    return {f"{name}{i}": helpers.random_tokens(vocab, n, 100 * helpers.SEEDS[name] + i)
            for i, n in enumerate(LENGTHS[name])}


def check_rows(rows, expected, dtype, what):
    for rid, want in expected.items():
        got = np.stack([rows[(rid, p)] for p in range(want.shape[0])])
        helpers.assert_close(got, want, dtype, f"{what}, request {rid}")


@pytest.fixture(scope="module")
def expected(model_folders):
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            d = model_folders(name, dtype)
            cache[(name, dtype)] = {rid: helpers.plain_logits(d, toks, dtype) for rid, toks in requests_for(name).items()}
        return cache[(name, dtype)]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_all_ways_of_cutting_agree_with_the_plain_implementation(model_folders, expected, name, dtype):
    d = model_folders(name, dtype)
    reqs = requests_for(name)
    want = expected(name, dtype)
    by_mode = {}
    for mode, cut in [("whole", helpers.cut_whole), ("tail one by one", helpers.cut_tail_singly),
                      ("changing portions", None)]:
        steps, n0 = [], 0
        for i, (rid, toks) in enumerate(reqs.items()):
            sizes = cut(toks) if cut else helpers.cut_varying(toks, 17 + i)
            s = helpers.solo_trace(rid, toks, sizes, n0)
            steps += s; n0 += len(s)
        outputs, runner = helpers.run_inprocess(d, dtype, steps, max_tokens=128)
        rows = helpers.collect_rows(steps, outputs)
        check_rows(rows, want, dtype, f"{name} {dtype} {mode}")
        by_mode[mode] = rows
    steps, peak = helpers.mixed_trace(reqs, seed=5, max_live=4)
    assert any(len(s["entries"]) > 1 and min(len(e["tokens"]) for e in s["entries"]) == 1
               and max(len(e["tokens"]) for e in s["entries"]) > 1 for s in steps), "no step mixes portions and single tokens"
    # run the same mixed trace twice over in one pool, so the second pass lands on used pages
    again = [dict(s, step=s["step"] + len(steps),
                  entries=[dict(e, id=e["id"] + "'") for e in s["entries"]], end=[r + "'" for r in s["end"]]) for s in steps]
    outputs, runner = helpers.run_inprocess(d, dtype, steps + again, max_tokens=peak)
    assert max(runner.cache.stats()["pages_high_water"]) <= peak // 16
    rows = helpers.collect_rows(steps + again, outputs)
    check_rows(rows, want, dtype, f"{name} {dtype} mixed")
    check_rows({(rid[:-1], p): v for (rid, p), v in rows.items() if rid.endswith("'")}, want, dtype,
               f"{name} {dtype} mixed, second pass on used pages")
    by_mode["mixed"] = rows
    if dtype == "float32":
        # the 32-bit path computes a position the same way however the work is cut
        # bit for bit: every 32-bit kernel sums an output's terms in an order that the cut does not change
        ref = by_mode["whole"]
        for mode, rows in by_mode.items():
            for k in ref:
                assert np.array_equal(rows[k], ref[k]), (
                    f"{name}: '{mode}' differs from 'whole' at {k} by {np.abs(rows[k] - ref[k]).max():.3e}")


def test_tcgen05_prefill_attention_inside_the_engine(model_folders, expected, monkeypatch):
    """Head size 64: every portion of more than one token goes through the tcgen05 attention kernel (its
    threshold is set to 0 for the test): whole prompts of several key blocks, portions of changing size over
    an existing cache, a window wider than a key block, portions beside single tokens on reused pages."""
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts import attention
    monkeypatch.setattr(attention, "PREFILL_TC_MIN_TOKENS", 0)
    calls = []
    real = ops.attention_prefill_tc
    monkeypatch.setattr(ops, "attention_prefill_tc", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    d = model_folders("D", "bfloat16")
    reqs = requests_for("D")
    want = expected("D", "bfloat16")
    for mode, cut in [("whole", helpers.cut_whole), ("changing portions", None)]:
        steps, n0 = [], 0
        for i, (rid, toks) in enumerate(reqs.items()):
            sizes = cut(toks) if cut else helpers.cut_varying(toks, 23 + i)
            s = helpers.solo_trace(rid, toks, sizes, n0)
            steps += s; n0 += len(s)
        outputs, runner = helpers.run_inprocess(d, "bfloat16", steps, max_tokens=320)
        check_rows(helpers.collect_rows(steps, outputs), want, "bfloat16", f"D {mode}")
    steps, peak = helpers.mixed_trace(reqs, seed=7, max_live=4)
    outputs, runner = helpers.run_inprocess(d, "bfloat16", steps, max_tokens=peak)
    check_rows(helpers.collect_rows(steps, outputs), want, "bfloat16", "D mixed")
    assert len(calls) >= 2 * len(reqs), "the tcgen05 kernel did not run"
    ops.check_status()


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_captured_general_steps_replay_what_the_kernels_compute_singly(model_folders, expected, monkeypatch, name):
    """Steps that mix portions and single tokens are padded to a shape, run kernel by kernel the first time the shape
    comes and replayed from a captured graph afterwards (here: captured at first sight). The same mixed trace runs
    twice in one pool: the second pass replays what the first captured, on other pages, and must give the same
    bits; both must equal the plain implementation."""
    from boring_llm_b200.parts import attention
    if name == "D":
        monkeypatch.setattr(attention, "PREFILL_TC_MIN_TOKENS", 0)     # the tcgen05 attention, with padded tile lists
    d = model_folders(name, "bfloat16")
    reqs = requests_for(name)
    want = expected(name, "bfloat16")
    steps, peak = helpers.mixed_trace(reqs, seed=13, max_live=4)
    again = [dict(s, step=s["step"] + len(steps),
                  entries=[dict(e, id=e["id"] + "'") for e in s["entries"]], end=[r + "'" for r in s["end"]]) for s in steps]
    outputs, runner = helpers.run_inprocess(d, "bfloat16", steps + again, max_tokens=peak + 64, step_graph_after=1)
    general = [s for s in steps if any(len(e["tokens"]) > 1 for e in s["entries"])]
    assert len(runner._step_graphs) >= 1 and runner.graph_steps >= len(general) // 2
    rows = helpers.collect_rows(steps + again, outputs)
    check_rows({k: v for k, v in rows.items() if not k[0].endswith("'")}, want, "bfloat16", f"{name} first pass")
    second = {(rid[:-1], p): v for (rid, p), v in rows.items() if rid.endswith("'")}
    check_rows(second, want, "bfloat16", f"{name} replayed")
    for k, v in second.items():
        assert np.array_equal(v, rows[k]), f"{name}: the replay differs from the first run at {k}"
    runner.check_kernels()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_bfloat16_against_the_pure_plain_implementation(model_folders, name):
    """No rounding on the plain side: a bfloat16 engine stays within a few percent of exact arithmetic
    on a well-conditioned model (weights N(0, 0.02), the benchmark's distribution)."""
    d = model_folders(name, "bfloat16", 0.02)
    reqs = requests_for(name)
    steps, peak = helpers.mixed_trace(reqs, seed=11, max_live=4)
    outputs, _ = helpers.run_inprocess(d, "bfloat16", steps, max_tokens=peak)
    rows = helpers.collect_rows(steps, outputs)
    for rid, toks in reqs.items():
        want = helpers.plain_logits(d, toks, "float32")
        got = np.stack([rows[(rid, p)] for p in range(len(toks))])
        helpers.assert_close(got, want, "bfloat16", f"pure {name} {rid}", tol=helpers.TOL_PURE_BF16, mean_tol=8e-3)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_the_trace_run_program(model_folders, expected, tmp_path, name, dtype):
    """bin/trace_run as a user drives it: a line in, `done <step>` out, files per step, exit code 0."""
    d = model_folders(name, dtype)
    reqs = requests_for(name)
    steps, peak = helpers.mixed_trace(reqs, seed=9, max_live=4)
    steps.append({"step": steps[-1]["step"] + 1, "entries": [{"id": "nolog", "tokens": [1, 2, 3], "want": []}], "end": ["nolog"]})
    out = str(tmp_path / "out")
    env = dict(os.environ, HOME=str(tmp_path / "home"))
    outputs = helpers.run_trace_program(d, dtype, steps, peak, out, helpers.TINY[name]["vocab_size"], env)
    rows = helpers.collect_rows(steps, outputs)
    check_rows(rows, expected(name, dtype), dtype, f"trace_run {name} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_freed_pages_full_of_nan_change_nothing(model_folders, expected, name, dtype):
    """Pages are filled with NaN when they are given back (and all of them, with the spare page, at the start): a
    kernel that reads a key or value past a request's length, in a page of a finished request or behind a window,
    even to multiply it by zero, would turn logits into NaN. The mixed trace runs twice over in a pool that is
    just large enough, so every request of the second pass lives in poisoned pages."""
    d = model_folders(name, dtype)
    reqs = requests_for(name)
    steps, peak = helpers.mixed_trace(reqs, seed=21, max_live=4)
    again = [dict(s, step=s["step"] + len(steps),
                  entries=[dict(e, id=e["id"] + "'") for e in s["entries"]], end=[r + "'" for r in s["end"]]) for s in steps]
    outputs, runner = helpers.run_inprocess(d, dtype, steps + again, max_tokens=peak, debug_poison=True,
                                            step_graph_after=1)
    runner.storage.poison_freed_pages()
    # (all but the spare page at the end, where the rows that pad a replayed step write)
    assert all(torch.isnan(kv[:, :, :-1].float()).all() for kv in runner.storage.kv), "every page was given back: all are poisoned"
    rows = helpers.collect_rows(steps + again, outputs)
    check_rows({(rid.rstrip("'"), p): v for (rid, p), v in rows.items() if rid.endswith("'")}, expected(name, dtype), dtype,
               f"{name} {dtype} on poisoned pages")
    check_rows({k: v for k, v in rows.items() if not k[0].endswith("'")}, expected(name, dtype), dtype, f"{name} {dtype} first pass")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_truncation_between_steps(model_folders, tmp_path, dtype):
    """40 tokens are fed, the cache is cut back to its first 23, other tokens follow (in a portion, then one by
    one): every row must equal the plain implementation on (the first 23 + the other tokens), as if the 17 had
    never been there; the pages behind the cut come back to the pool. Once in-process with poisoned pages, once
    through bin/trace_run's `truncate` event. (The reference truncates by setting the length, src/model.br:2313-2314.)"""
    d = model_folders("A", dtype)
    vocab = helpers.TINY["A"]["vocab_size"]
    first = helpers.random_tokens(vocab, 40, 31)
    other = helpers.random_tokens(vocab, 30, 32)
    steps = [
        {"step": 0, "entries": [{"id": "t", "tokens": first, "want": list(range(40))}], "end": []},
        {"step": 1, "truncate": [{"id": "t", "keep": 23}],
         "entries": [{"id": "t", "tokens": other[:9], "want": list(range(9))}], "end": []},
    ] + [{"step": 2 + i, "entries": [{"id": "t", "tokens": [tok], "want": [0]}], "end": ["t"] if i == 20 else []}
         for i, tok in enumerate(other[9:])]
    want_first = helpers.plain_logits(d, first, dtype)
    want_cut = helpers.plain_logits(d, first[:23] + other, dtype)

    def check(outputs, what):
        helpers.assert_close(outputs[0], want_first, dtype, f"{what}: before the cut")
        got = np.concatenate([outputs[s["step"]] for s in steps[1:]])
        helpers.assert_close(got, want_cut[23:], dtype, f"{what}: after the cut")

    outputs, runner = helpers.run_inprocess(d, dtype, steps, max_tokens=64, debug_poison=True)
    check(outputs, "in process")
    assert runner.cache.stats()["pages_high_water"] == [4]            # 40 tokens, then 23 + 30 = 53: the pool's 4 pages suffice
    out = str(tmp_path / "out")
    check(helpers.run_trace_program(d, dtype, steps, 64, out, vocab, extra=["--poison"]), "trace_run")
    with pytest.raises(Exception, match="truncate"):
        runner.add_request("u"); runner.truncate("u", 5)


def test_long_decoding_and_first_tokens(model_folders):
    """300 tokens decoded one by one after a short prompt (19 pages, past a window many times over), and
    the very first positions of a sequence, where a page, a chunk and a window all begin."""
    for name, dtype in [("C", "float32"), ("C", "bfloat16"), ("A", "bfloat16")]:
        d = model_folders(name, dtype)
        toks = helpers.random_tokens(helpers.TINY[name]["vocab_size"], 5 + 300, 77)
        steps = helpers.solo_trace("long", toks, [5] + [1] * 300)
        outputs, _ = helpers.run_inprocess(d, dtype, steps, max_tokens=320)
        rows = helpers.collect_rows(steps, outputs)
        want = helpers.plain_logits(d, toks, dtype)
        got = np.stack([rows[("long", p)] for p in range(len(toks))])
        helpers.assert_close(got, want, dtype, f"long decoding {name} {dtype}")
        helpers.assert_close(got[:3], want[:3], dtype, f"first tokens {name} {dtype}")
        steps = helpers.solo_trace("one", toks[:4], [1, 1, 2])
        outputs, _ = helpers.run_inprocess(d, dtype, steps, max_tokens=64)
        rows = helpers.collect_rows(steps, outputs)
        helpers.assert_close(np.stack([rows[("one", p)] for p in range(4)]), want[:4], dtype, "token by token from the start")


def test_a_far_key_decides_the_answer(model_folders):
    """With the benchmark's N(0, 0.02) weights attention is near-uniform, and a key skipped among hundreds
    would hide inside the bfloat16 tolerance. The test models' weights (std 0.25) give scores with a spread
    of about 6, so a handful of keys, anywhere in the sequence, carry most of a query's weight: here a
    260-token prompt (17 pages) is replayed whole, with its tail token by token, and in changing portions.
    A kernel that drops, repeats or misplaces a key (a page's edge, a portion's start) moves whole rows."""
    d = model_folders("B", "bfloat16")
    toks = helpers.random_tokens(320, 260, 5)
    want = helpers.plain_logits(d, toks, "bfloat16")
    for sizes in ([260], [200] + [1] * 60, helpers.cut_varying(toks, 3)):
        steps = helpers.solo_trace("s", toks, sizes)
        outputs, _ = helpers.run_inprocess(d, "bfloat16", steps, max_tokens=320)
        rows = helpers.collect_rows(steps, outputs)
        helpers.assert_close(np.stack([rows[("s", p)] for p in range(260)]), want, "bfloat16", f"sharp attention, cuts {sizes[:4]}...")


def test_steps_that_cannot_run_are_refused(model_folders):
    from boring_llm_b200.engine.runner import OutOfPages, StepEntry, StepError
    d = model_folders("A", "float32")
    _, runner = helpers.run_inprocess(d, "float32", [], max_tokens=64)
    with pytest.raises(StepError, match="outside the vocabulary"):
        runner.step([StepEntry("a", [1, 256], [0])])
    with pytest.raises(StepError, match="wanted place"):
        runner.step([StepEntry("a", [1, 2], [2])])
    with pytest.raises(StepError, match="twice"):
        runner.step([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("a", [1] * 40, []), StepEntry("b", [1] * 40, [])])
    assert runner.cache.free_pages() == [4] and not runner.cache.live_requests()     # nothing was changed
    runner.step([StepEntry("a", [1] * 40, [])])
    with pytest.raises(StepError, match="context size"):
        runner.step([StepEntry("a", [1] * 30, [])])
