"""The scheduler's decisions on the host, with a stand-in for the GPU step: admission, portions under
the token budget, decoding, finishing and freeing, and what happens when pages run out."""
import random

import pytest

from boring_llm_b200.cache import CacheManager, PagedKVSpec
from boring_llm_b200.config import EngineOptions
from boring_llm_b200.engine.scheduler import AdmissionError, Scheduler
from boring_llm_b200.sampling.params import SamplingParams

VOCAB = 50


def next_token(tokens):
    """A 'model' whose next token depends on the whole history, so any lost or repeated token shows."""
    h = 7
    for t in tokens:
        h = (h * 31 + t + 1) % 1000003
    return h % VOCAB


def make(tokens=256, seqs=4, budget=64, chunk=16, ctx=128):
    opts = EngineOptions(max_tokens=tokens, max_num_seqs=seqs, max_num_batched_tokens=budget,
                         prefill_chunk=chunk, ctx_size=ctx)
    cache = CacheManager([PagedKVSpec(1, 16, 0)], 16, tokens, seqs)
    return Scheduler(cache, opts), cache, opts


def drive(sched, cache, on_step=None, limit=5000):
    steps = []
    for _ in range(limit):
        if not sched.has_work():
            break
        st = sched.schedule()
        if st is None:
            assert not sched.running and not sched.waiting
            break
        sampled = []
        for e, req, samp in zip(st.entries, st.requests, st.samples):
            assert list(e.tokens) == req.tokens[req.num_computed:req.num_computed + len(e.tokens)]
            cache.commit(e.request_id, len(e.tokens))          # what the runner does after a step
            if samp:
                sampled.append(next_token(req.tokens))
        steps.append(st)
        if on_step:
            on_step(st)
        sched.apply(st, sampled)
        cache.check()
    else:
        raise AssertionError("the scheduler did not finish")
    return steps


def solo(prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        out.append(next_token(toks)); toks.append(out[-1])
    return out


def test_prompt_is_cut_into_portions_then_decoded():
    sched, cache, _ = make(chunk=16, budget=64)
    r = sched.add("a", list(range(40)), SamplingParams(n_predict=3))
    steps = drive(sched, cache)
    assert [len(s.entries[0].tokens) for s in steps] == [16, 16, 8, 1, 1]
    assert [s.samples[0] for s in steps] == [False, False, True, True, True]
    assert [list(s.entries[0].want) for s in steps] == [[], [], [7], [0], [0]]
    assert r.output == solo(range(40), 3) and r.finish_reason == "length"
    assert cache.free_pages() == [cache.num_pages] and not cache.live_requests()


def test_budget_is_shared_decodes_first():
    sched, cache, _ = make(chunk=32, budget=20)
    a = sched.add("a", list(range(5)), SamplingParams(n_predict=30))
    seen = []
    drive_steps = 0
    st = sched.schedule(); assert [len(e.tokens) for e in st.entries] == [5]
    cache.commit("a", 5); sched.apply(st, [next_token(a.tokens)])
    b = sched.add("b", list(range(30)), SamplingParams(n_predict=2))
    st = sched.schedule()
    assert [(e.request_id, len(e.tokens)) for e in st.entries] == [("a", 1), ("b", 19)]   # 1 + 19 = budget
    for e in st.entries:
        cache.commit(e.request_id, len(e.tokens))
    sched.apply(st, [next_token(a.tokens)])
    st = sched.schedule()
    assert [(e.request_id, len(e.tokens)) for e in st.entries] == [("a", 1), ("b", 11)]
    assert st.samples == [True, True]


def test_effective_chunk_is_min_of_batch_and_ubatch():
    sched, cache, _ = make(chunk=512, budget=10)
    sched.add("a", list(range(25)), SamplingParams(n_predict=1))
    steps = drive(sched, cache)
    assert [len(s.entries[0].tokens) for s in steps] == [10, 10, 5]


def test_admission_refusals_and_clamps():
    sched, cache, opts = make(ctx=32)
    with pytest.raises(AdmissionError, match="empty"):
        sched.add("e", [], SamplingParams())
    with pytest.raises(AdmissionError, match="context_length_exceeded"):
        sched.add("l", list(range(32)), SamplingParams())
    r = sched.add("c", list(range(30)), SamplingParams(n_predict=40))
    assert r.max_new == 2
    r2 = sched.add("m", list(range(10)), SamplingParams(n_predict=-1))
    assert r2.max_new == 22
    drive(sched, cache)
    assert len(r.output) == 2 and r.finish_reason == "length"
    assert len(r2.output) == 22 and len(r2.prompt) + len(r2.output) == opts.ctx_size
    small, c2, _ = make(tokens=32, ctx=128)
    with pytest.raises(AdmissionError, match="out_of_cache"):
        small.add("big", list(range(40)), SamplingParams())


def test_end_token_is_returned_but_not_fed():
    sched, cache, _ = make()
    prompt = [1, 2, 3]
    want = solo(prompt, 10)
    stop = want[4]
    r = sched.add("a", prompt, SamplingParams(n_predict=10, eos_token_ids=(stop,)))
    steps = drive(sched, cache)
    first = want.index(stop)
    assert r.output == want[:first + 1] and r.finish_reason == "stop"
    assert sum(len(s.entries[0].tokens) for s in steps) == len(prompt) + first      # the end token never ran
    r2 = sched.add("b", prompt, SamplingParams(n_predict=10, eos_token_ids=(stop,), ignore_eos=True))
    drive(sched, cache)
    assert r2.output == want and r2.finish_reason == "length"


def test_slots_limit_live_requests_and_fifo_admission():
    sched, cache, _ = make(seqs=2, tokens=512)
    reqs = [sched.add(i, [i + 1] * 5, SamplingParams(n_predict=4)) for i in range(5)]
    order = []
    def on_step(st):
        assert len(sched.running) <= 2
        for r in st.requests:
            if r.request_id not in order:
                order.append(r.request_id)
    drive(sched, cache, on_step)
    assert order == [0, 1, 2, 3, 4]
    for r in reqs:
        assert r.output == solo(r.prompt, 4)


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    # 6 pages of 16: two requests of 40 + 40 tokens fit (3 + 3 pages) until one needs a 4th page
    sched, cache, _ = make(tokens=96, seqs=4, budget=64, chunk=64)
    a = sched.add("a", list(range(40)), SamplingParams(n_predict=30))
    b = sched.add("b", list(range(10, 50)), SamplingParams(n_predict=30))
    drive(sched, cache)
    assert sched.num_preemptions >= 1
    assert a.preemptions == 0 and b.preemptions >= 1          # the older request never yields
    assert a.output == solo(a.prompt, 30) and b.output == solo(b.prompt, 30)
    assert cache.free_pages() == [6] and not cache.live_requests()


def test_a_request_too_large_for_the_cache_alone_ends_with_out_of_cache():
    sched, cache, _ = make(tokens=48, seqs=2, ctx=128, chunk=64)
    r = sched.add("a", list(range(30)), SamplingParams(n_predict=60))
    ok = sched.add("b", [5, 6, 7], SamplingParams(n_predict=3))
    drive(sched, cache)
    assert r.finish_reason == "out_of_cache" and len(r.output) >= 17       # 48 - 30 (-1) tokens fitted
    assert ok.output == solo(ok.prompt, 3) and ok.finish_reason == "length"
    assert cache.free_pages() == [3]


def test_abort_frees_everything():
    sched, cache, _ = make()
    sched.add("a", list(range(20)), SamplingParams(n_predict=50))
    sched.add("b", list(range(20)), SamplingParams(n_predict=50))
    st = sched.schedule()
    for e in st.entries:
        cache.commit(e.request_id, len(e.tokens))
    sched.apply(st, [])
    sched.abort("a")
    assert sched.finished["a"].finish_reason == "aborted" and "a" not in cache
    sched.abort("b")
    assert not sched.has_work() and cache.free_pages() == [cache.num_pages]
    cache.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_arrivals_with_few_pages_every_request_finishes_like_its_solo_run(seed):
    rng = random.Random(seed)
    tokens = rng.choice([64, 96, 160])
    sched, cache, opts = make(tokens=tokens, seqs=rng.choice([2, 3, 4]), budget=rng.choice([8, 24, 64]),
                              chunk=rng.choice([4, 16, 64]), ctx=64)
    pending = [(f"r{i}", [rng.randrange(VOCAB) for _ in range(rng.randint(1, 30))], rng.randint(1, 20))
               for i in range(12)]
    reqs = []
    def arrive(_st=None):
        while pending and rng.random() < 0.4:
            rid, prompt, n = pending.pop(0)
            reqs.append(sched.add(rid, prompt, SamplingParams(n_predict=n)))
    arrive()
    while pending or sched.has_work():
        if not sched.has_work():
            rid, prompt, n = pending.pop(0)
            reqs.append(sched.add(rid, prompt, SamplingParams(n_predict=n)))
        drive_one = drive(sched, cache, arrive)
    assert len(reqs) == 12
    for r in reqs:
        assert r.finish_reason == "length", (r.request_id, r.finish_reason)
        assert r.output == solo(r.prompt, min(r.params.n_predict, opts.ctx_size - len(r.prompt)))
    assert cache.free_pages() == [cache.num_pages] and not cache.live_requests()
    cache.check()


def drive_ahead(sched, cache, limit=5000):
    """The engine's loop with one decode step launched ahead (its tokens unknown when it is put together): the
    stand-in 'device' computes a step's tokens only when the step is collected, from the history as it is then."""
    inflight, kinds = None, []
    for _ in range(limit):
        if inflight is None:
            if not sched.has_work():
                break
            inflight = sched.schedule()
            if inflight is None:
                break
            for e in inflight.entries:
                cache.commit(e.request_id, len(e.tokens))
            kinds.append("scheduled")
        st = inflight
        ahead = sched.lookahead(st) if all(len(e.tokens) == 1 for e in st.entries) else None
        if ahead is not None:
            assert [e.tokens for e in ahead.entries] == [[0]] * len(st.entries) and ahead.requests == st.requests
            for e in ahead.entries:
                cache.commit(e.request_id, 1)
            kinds.append("ahead")
        # the device's answer for st: a row whose request has ended gets a token too (nobody reads it)
        sampled = [next_token(req.tokens) if req.state == "running" else -1
                   for req, samp in zip(st.requests, st.samples) if samp]
        sched.apply(st, sampled)
        cache.check()
        if ahead is not None and not any(r.state == "running" for r in ahead.requests):
            ahead = None
        inflight = ahead
    else:
        raise AssertionError("the scheduler did not finish")
    return kinds


def test_lookahead_steps_give_every_request_its_solo_tokens():
    sched, cache, _ = make(tokens=512, seqs=4, budget=64, chunk=16, ctx=128)
    prompts = [[(3 * i + j) % VOCAB for j in range(n)] for i, n in enumerate((5, 20, 33))]
    lens = (9, 14, 6)
    reqs = [sched.add(i, p, SamplingParams(n_predict=n, ignore_eos=True)) for i, (p, n) in enumerate(zip(prompts, lens))]
    kinds = drive_ahead(sched, cache)
    assert kinds.count("ahead") >= 3                      # while all three decoded and none was about to end
    for r, p, n in zip(reqs, prompts, lens):
        assert r.output == solo(p, n) and r.finish_reason == "length"
    assert cache.stats()["live_requests"] == 0 and cache.stats()["pages_in_use"] == [0]


def test_lookahead_row_of_a_request_that_ends_on_an_end_token_is_dropped():
    sched, cache, _ = make(tokens=512, seqs=4, budget=64, chunk=16, ctx=128)
    prompts = [[(5 * i + j) % VOCAB for j in range(n)] for i, n in enumerate((7, 12))]
    free = [solo(p, 12) for p in prompts]
    stop = free[0][4]                                      # request 0 ends at its fifth token, request 1 goes on
    reqs = [sched.add(0, prompts[0], SamplingParams(n_predict=12, eos_token_ids=(stop,))),
            sched.add(1, prompts[1], SamplingParams(n_predict=12, ignore_eos=True))]
    kinds = drive_ahead(sched, cache)
    assert "ahead" in kinds
    assert reqs[0].output == free[0][:free[0].index(stop) + 1] and reqs[0].finish_reason == "stop"
    assert reqs[1].output == free[1]
    assert cache.stats()["live_requests"] == 0 and cache.stats()["pages_in_use"] == [0]


def test_lookahead_is_refused_when_the_next_step_is_not_certain():
    sched, cache, _ = make(tokens=512, seqs=4, budget=64, chunk=16, ctx=128)
    a = sched.add("a", [1, 2, 3], SamplingParams(n_predict=3, ignore_eos=True))
    st = sched.schedule()                                  # the prompt: not a decode step
    assert sched.lookahead(st) is None
    cache.commit("a", 3); sched.apply(st, [next_token(a.tokens)])
    st = sched.schedule()
    cache.commit("a", 1)
    assert sched.lookahead(st) is not None                 # token 2 of 3 follows for sure
    sched.apply(st, [next_token(a.tokens)])
    st = sched.schedule()
    cache.commit("a", 1)
    assert sched.lookahead(st) is None                     # this step's token is the last one
    sched.add("b", [4, 5], SamplingParams(n_predict=4, ignore_eos=True))
    sched.apply(st, [next_token(a.tokens)])
    assert a.finish_reason == "length"
    st = sched.schedule()
    cache.commit("b", 2); sched.apply(st, [7])
    st = sched.schedule(); cache.commit("b", 1)
    sched.add("c", [9], SamplingParams(n_predict=2, ignore_eos=True))
    assert sched.lookahead(st) is None                     # somebody waits: the next step will not be this batch
