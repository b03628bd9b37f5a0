"""Generation through the Python entry point: greedy tokens equal the plain implementation's, sampled
tokens are reproducible and follow the plain sampler, the scheduler's preemption does not change them."""
import numpy as np
import pytest
import torch

import helpers
import plain_model as plain

pytestmark = pytest.mark.gpu

PROMPTS = {"A": [7, 16, 33], "B": [1, 5, 19, 64]}
N_NEW = {"A": 8, "B": 12}


def prompts_for(name):
    vocab = helpers.TINY[name]["vocab_size"]
    return [helpers.random_tokens(vocab, n, 500 + n) for n in PROMPTS[name]]


def check_greedy(d, prompt, out, dtype):
    """Every generated token is the plain implementation's arg-max given the engine's own prefix; in
    bfloat16 a near-tie (gap below the tolerance) may go either way."""
    cfg, W = plain.read_model_folder(d)
    logits = plain.forward(cfg, W, prompt + out, stored=plain.round_bf16 if dtype == "bfloat16" else None).numpy()
    scale = np.abs(logits).max()
    for i, tok in enumerate(out):
        row = logits[len(prompt) - 1 + i]
        best = int(np.argmax(row))
        if tok != best:
            gap = row[best] - row[tok]
            assert dtype == "bfloat16" and gap <= 2 * helpers.TOL[dtype] * scale, (
                f"token {i}: engine chose {tok}, plain {best} (gap {gap:.3e})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_equals_the_plain_implementation(model_folders, name, dtype):
    from boring_llm_b200 import Engine
    d = model_folders(name, dtype, 0.02)                  # the benchmark's weight scale
    eng = Engine(d, dtype=dtype, ctx_size=128, max_num_seqs=4, max_tokens=512, prefill_chunk=8)
    prompts = prompts_for(name)
    outs = eng.generate(prompts, n_predict=N_NEW[name], ignore_eos=True)
    assert [len(o) for o in outs] == [N_NEW[name]] * len(prompts)
    for p, o in zip(prompts, outs):
        check_greedy(d, p, o, dtype)
        if dtype == "float32":
            cfg, W = plain.read_model_folder(d)
            assert o == plain.greedy_generate(cfg, W, p, len(o))
    # one by one gives the same tokens as the batch
    solo = [eng.generate([p], n_predict=N_NEW[name], ignore_eos=True)[0] for p in prompts]
    assert solo == outs
    s = eng.stats()
    assert s["live_requests"] == 0 and s["pages_in_use"] == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_does_not_change_the_tokens(model_folders, dtype):
    from boring_llm_b200 import Engine
    d = model_folders("B", dtype)
    prompts = [helpers.random_tokens(320, n, 900 + n) for n in (30, 41, 25, 38)]
    roomy = Engine(d, dtype=dtype, ctx_size=128, max_num_seqs=4, max_tokens=1024, prefill_chunk=16)
    want = roomy.generate(prompts, n_predict=24, ignore_eos=True)
    tight = Engine(d, dtype=dtype, ctx_size=128, max_num_seqs=4, max_tokens=160, prefill_chunk=16,
                   max_num_batched_tokens=32)
    got = tight.generate(prompts, n_predict=24, ignore_eos=True)
    assert tight.stats()["preemptions"] >= 1
    if dtype == "float32":
        assert got == want
    else:
        for p, o in zip(prompts, got):
            check_greedy(d, p, o, dtype)
    tight.runner.cache.check()
    assert tight.stats()["pages_in_use"] == [0]


def test_temperature_sampling_is_seeded_and_follows_the_plain_sampler(model_folders):
    from boring_llm_b200 import Engine
    d = model_folders("B", "float32")
    eng = Engine(d, dtype="float32", ctx_size=128, max_num_seqs=4, max_tokens=512, prefill_chunk=8)
    prompts = prompts_for("B")
    a = eng.generate(prompts, n_predict=12, temperature=0.8, seed=3, ignore_eos=True)
    b = eng.generate(prompts, n_predict=12, temperature=0.8, seed=3, ignore_eos=True)
    c = eng.generate(prompts, n_predict=12, temperature=0.8, seed=4, ignore_eos=True)
    assert a == b and a != c
    # request i draws from the generator seeded with seed + i: replay it on the plain side
    cfg, W = plain.read_model_folder(d)
    for i, (p, out) in enumerate(zip(prompts, a)):
        state = plain.seed_rng(3 + i)
        toks = list(p)
        for tok in out:
            logits = plain.forward(cfg, W, toks)[-1].numpy()
            want, state = plain.sample(state, logits, 0.8)
            assert tok == want
            toks.append(tok)
    k = eng.generate(prompts[:2], n_predict=6, temperature=1.5, seed=1, top_k=1, ignore_eos=True)
    g = eng.generate(prompts[:2], n_predict=6, ignore_eos=True)
    assert k == g                                           # top_k 1 is greedy


def test_end_token_and_context_limit(model_folders):
    from boring_llm_b200 import Engine
    from boring_llm_b200.engine import AdmissionError
    d = model_folders("A", "float32")
    eng = Engine(d, dtype="float32", ctx_size=48, max_num_seqs=2, max_tokens=128)
    p = helpers.random_tokens(256, 10, 1)
    free = eng.generate([p], n_predict=10, ignore_eos=True)[0]
    stop = free[3]
    cut = eng.generate([p], n_predict=10, eos_token_ids=[stop])[0]
    assert cut == free[:free.index(stop) + 1]               # returned, not fed (src/model.br:2299-2300)
    full = eng.generate([p], n_predict=-1, ignore_eos=True)[0]
    assert len(p) + len(full) == 48
    with pytest.raises(AdmissionError):
        eng.generate([list(range(48))], n_predict=1)
    with pytest.raises(ValueError, match="vocabulary"):
        eng.generate([[1, 2, 999]], n_predict=1)


def test_lookahead_gives_the_same_tokens_as_stepping_in_turn(model_folders):
    """Decode steps launched one ahead (their tokens fed back on the device) against the same engine without:
    greedy and sampled, with requests that end on an end token while their row is already in the step ahead,
    ends by length at different steps, and a request that arrives while a step is in flight."""
    from boring_llm_b200 import Engine
    from boring_llm_b200.sampling.params import SamplingParams
    d = model_folders("B", "bfloat16", 0.02)
    prompts = [helpers.random_tokens(320, n, 700 + n) for n in (9, 21, 14, 30)]
    kw = dict(dtype="bfloat16", ctx_size=128, max_num_seqs=4, max_tokens=1024, prefill_chunk=16)
    ahead, turn = Engine(d, lookahead=True, **kw), Engine(d, lookahead=False, **kw)
    free = turn.generate(prompts, n_predict=20, ignore_eos=True)
    assert ahead.generate(prompts, n_predict=20, ignore_eos=True) == free
    assert ahead.runner.graph_steps > 0 and ahead._inflight is None
    # every request stops at a token of its own free run, at different steps
    for cut in (2, 7, 13):
        stops = [o[cut] for o in free]
        want = turn.generate(prompts, n_predict=20, eos_token_ids=stops)
        got = ahead.generate(prompts, n_predict=20, eos_token_ids=stops)
        assert got == want and any(len(o) < 20 for o in got)
    for seed in (1, 2):
        want = turn.generate(prompts, n_predict=17, temperature=0.9, seed=seed, top_k=40, top_p=0.95, ignore_eos=True)
        assert ahead.generate(prompts, n_predict=17, temperature=0.9, seed=seed, top_k=40, top_p=0.95, ignore_eos=True) == want
    # different lengths: the batch shrinks while a step is ahead; then a request arrives in the middle
    outs = {}
    for eng in (turn, ahead):
        reqs = [eng.add_request(p, SamplingParams(n_predict=5 + 4 * i, ignore_eos=True)) for i, p in enumerate(prompts[:3])]
        for _ in range(6):
            eng.step()
        if eng is ahead:                                        # a step is in flight: reading it adds one token to each
            before = [len(r.output) + (r.state == "running") for r in reqs]
            assert eng._inflight is not None and eng.drain() == [] and eng._inflight is None
            assert [len(r.output) for r in reqs] == before
        reqs.append(eng.add_request(prompts[3], SamplingParams(n_predict=9, ignore_eos=True)))
        eng.run_until_done()
        outs[eng] = [list(r.output) for r in reqs]
        assert [len(o) for o in outs[eng]] == [5, 9, 13, 9]
        eng.runner.cache.check()
        s = eng.stats()
        assert s["live_requests"] == 0 and s["pages_in_use"] == [0]
        for p, o in zip(prompts, outs[eng]):                    # (the arrival meets the others one step apart in the two
            check_greedy(d, p, o, "bfloat16")                   # engines, in kernels that round differently: no equality)


def test_a_failed_step_with_another_one_ahead_leaves_scheduler_and_cache_in_step(model_folders):
    """The step in flight fails when its result is checked (here: the check itself is made to raise, no kernel is
    harmed) while the step ahead has already been launched: both steps' requests end with reason 'error', their
    pages and slots come back, nothing stays in flight, and the engine serves the next request as if nothing had
    happened."""
    from boring_llm_b200 import Engine
    from boring_llm_b200.kernels.ops import KernelError
    from boring_llm_b200.sampling.params import SamplingParams
    d = model_folders("B", "bfloat16", 0.02)
    prompts = [helpers.random_tokens(320, n, 700 + n) for n in (9, 21, 14)]
    eng = Engine(d, dtype="bfloat16", ctx_size=128, max_num_seqs=4, max_tokens=1024, prefill_chunk=16)
    want = eng.generate(prompts, n_predict=12, ignore_eos=True)
    reqs = [eng.add_request(p, SamplingParams(n_predict=12, ignore_eos=True)) for p in prompts]
    while eng._inflight is None:
        eng.step()
    eng.step()
    real = eng.runner.check_kernels

    def fail():
        raise KernelError("a block gave up on a bounded wait (made up by the test)")
    eng.runner.check_kernels = fail
    with pytest.raises(KernelError):
        eng.step()
    eng.runner.check_kernels = real
    assert eng._inflight is None and not eng.scheduler.has_work()
    assert all(r.state == "finished" and r.finish_reason == "error" for r in reqs)
    eng.runner.cache.check()
    s = eng.stats()
    assert s["live_requests"] == 0 and s["pages_in_use"] == [0]
    assert eng.generate(prompts, n_predict=12, ignore_eos=True) == want


def test_an_engine_from_random_weights_in_memory_equals_one_from_the_folder(tmp_path):
    """`Engine.from_random` builds the model on the device without a file; `write_random_model` + `Engine(dir)` go through
    the file: same configuration and seed, same tokens (greedy and sampled), in both dtypes."""
    from boring_llm_b200 import Engine, EngineOptions, Qwen2Config, write_random_model
    cfg = Qwen2Config.from_dict(helpers.TINY["B"])
    prompts = [helpers.random_tokens(320, n, 40 + n) for n in (3, 18)]
    for dtype in ("bfloat16", "float32"):
        d = str(tmp_path / dtype)
        write_random_model(d, cfg, 17, dtype, 0.05)
        opts = dict(dtype=dtype, ctx_size=64, max_num_seqs=2, max_tokens=128)
        a = Engine(d, **opts)
        b = Engine.from_random(cfg, 17, EngineOptions(**opts), std=0.05)
        for kw in (dict(), dict(temperature=0.7, seed=5)):
            assert a.generate(prompts, n_predict=10, ignore_eos=True, **kw) == b.generate(prompts, n_predict=10, ignore_eos=True, **kw)


def test_captured_steps_are_dropped_least_recently_used_first(model_folders, monkeypatch):
    """With room for only three captured general steps, a stream of differently shaped steps keeps capturing and
    dropping graphs; every request still gets the tokens it gets without any captured step."""
    from boring_llm_b200 import Engine
    from boring_llm_b200.engine import runner as runner_module
    monkeypatch.setattr(runner_module, "STEP_GRAPH_CACHE", 3)
    d = model_folders("A", "bfloat16", 0.02)
    prompts = [helpers.random_tokens(256, n, 300 + n) for n in (5, 37, 18, 61, 9, 44, 23, 70)]
    kw = dict(dtype="bfloat16", ctx_size=128, max_num_seqs=3, max_tokens=512, prefill_chunk=16, max_num_batched_tokens=24)
    plain_engine = Engine(d, cuda_graphs=False, **kw)
    want = plain_engine.generate(prompts, n_predict=6, ignore_eos=True)
    eng = Engine(d, step_graph_after=1, **kw)
    got = eng.generate(prompts, n_predict=6, ignore_eos=True)
    assert len(eng.runner._step_graphs) <= 3 and eng.runner.graph_steps > 10
    for p, o in zip(prompts, got):
        check_greedy(d, p, o, "bfloat16")
    same = sum(a == b for x, y in zip(want, got) for a, b in zip(x, y))
    assert same >= 0.9 * 6 * len(prompts)              # (decode graphs cut their attention slices for a bound: rounding may differ)
    eng.runner.check_kernels()


HEAD128 = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=192,
               num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=328, vocab_size=1000,
               rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024)


def test_head_size_128_through_the_tensor_core_paths(tmp_path):
    """Head size 128 (hidden 192 != 4 x 128, two key/value heads) end to end in bfloat16: prompts of 330 and 290
    tokens run on the products on pairs of SMs (q/k/v with rotation and cache write in its epilogue, norms shared
    between products) and the tcgen05 attention, the 24 decoded tokens on the TMA-fed decode attention inside captured
    graphs. Every token is the plain implementation's choice given the engine's own prefix (near-ties may go either
    way), and the kernels are seen on the path."""
    import boring_llm_b200 as b
    from boring_llm_b200.kernels import ops
    cfg = b.Qwen2Config.from_dict(HEAD128)
    d = str(tmp_path / "head128")
    b.write_random_model(d, cfg, seed=5, dtype="bfloat16", std=0.05)
    used = set()
    real_call = ops._call

    def spy(fn, *args):
        used.add(fn.__name__)
        return real_call(fn, *args)

    ops._call = spy
    try:
        eng = b.Engine(d, dtype="bfloat16", ctx_size=512, max_num_seqs=4, max_tokens=2048, max_num_batched_tokens=1024,
                       prefill_chunk=512)
        prompts = [helpers.random_tokens(1000, 330, 61), helpers.random_tokens(1000, 290, 62)]
        outs = eng.generate(prompts, n_predict=24, ignore_eos=True)
    finally:
        ops._call = real_call
    for p_, o_ in zip(prompts, outs):
        check_greedy(d, p_, o_, "bfloat16")
    for name in ("bl_gemm_tc_pair_qkv_rope", "bl_gemm_tc_pair_residual_norm", "bl_gemm_tc_pair_swiglu_scaled",
                 "bl_attention_prefill_tc", "bl_attention_decode_tma", "bl_rope_table"):
        assert name in used, f"{name} was not on the path"
    assert eng.runner.graph_steps >= 10
