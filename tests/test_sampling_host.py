"""Sampling options and the host's random number generator (no GPU)."""
import pytest

import plain_model as plain
from boring_llm_b200.sampling import SamplingParams, XorShift64, penalty_window


def test_generator_matches_the_plain_transcription():
    for seed in (0, 1, 42, 2**40 + 3):
        g, s = XorShift64(seed), plain.seed_rng(seed)
        for _ in range(50):
            u, s = plain.rng_next_f32(s)
            assert g.next_f32() == u
            assert g.state == s


def test_defaults_are_the_reference_defaults():
    p = SamplingParams()
    assert (p.n_predict, p.temperature, p.seed, p.top_k, p.top_p, p.min_p) == (40, 0.0, 0, 0, 1.0, 0.0)
    assert (p.repeat_penalty, p.repeat_last_n) == (1.0, 64)      # src/main.br:563-590
    with pytest.raises(ValueError):
        SamplingParams(min_p=2.0)
    with pytest.raises(ValueError):
        SamplingParams(repeat_penalty=0.0)


def test_penalty_window():
    h = [1, 2, 3, 2, 1, 4]
    assert penalty_window(h, 3) == [2, 1, 4]
    assert penalty_window(h, -1) == [1, 2, 3, 4]
    assert penalty_window(h, 0) == [] and penalty_window([], 5) == []
    assert penalty_window(h, 64) == [1, 2, 3, 4]
