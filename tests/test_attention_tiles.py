"""The launch list of the tcgen05 prefill attention (host side, no GPU)."""
import random

from boring_llm_b200.parts.attention import tc_attention_tiles


def covered(tiles, q_lens):
    rows = {r: [0] * n for r, n in enumerate(q_lens) if n > 1}
    for r, t0 in tiles:
        assert t0 % 128 == 0 and t0 < q_lens[r]
        for t in range(t0, min(t0 + 128, q_lens[r])):
            rows[r][t] += 1
    return all(all(c == 1 for c in v) for v in rows.values())


def test_every_row_is_in_exactly_one_tile():
    rng = random.Random(3)
    for _ in range(200):
        R = rng.randint(1, 6)
        q_lens = [rng.choice([1, 1, 2, 17, 128, 129, 255, 256, 257, 700, 2048]) for _ in range(R)]
        ctx_lens = [n + rng.choice([0, 5, 300, 4000]) for n in q_lens]
        tiles = tc_attention_tiles(q_lens, ctx_lens)
        assert covered(tiles, q_lens), (q_lens, ctx_lens, tiles)
        assert all(q_lens[r] > 1 for r, _ in tiles)


def test_the_tile_with_the_most_keys_is_last_in_the_list():
    q_lens, ctx_lens = [2048, 1, 300], [2048, 77, 5000]
    tiles = tc_attention_tiles(q_lens, ctx_lens)
    keys = [ctx_lens[r] - q_lens[r] + min(t0 + 128, q_lens[r]) for r, t0 in tiles]
    assert len(tiles) == 16 + 3
    assert [-(-k // 128) for k in keys] == sorted(-(-k // 128) for k in keys)
    assert tiles[-1][0] == 2                                         # 5000 keys: launched first


def test_a_plan_for_a_replayed_step_has_sizes_that_its_shape_determines():
    """The attention's step plan (host side). For a step that runs once the lists are exact; for a step that is
    captured and replayed they are padded to multiples of 8 with entries of the request without tokens, the longest
    context of the single-token requests is rounded up to a power of two, and two batches with the same padded lists
    have the same shape (they may share a captured graph) although their contents differ."""
    from boring_llm_b200.parts import attention
    from boring_llm_b200.parts.attention import attention_plan
    q_lens, ctx_lens = [1, 130, 1, 70, 1], [900, 400, 33, 70, 2047]
    exact = attention_plan(q_lens, ctx_lens)
    assert exact.arrays["singles"].tolist() == [0, 2, 4] and exact.host["longest_single"] == 2047
    assert exact.arrays["tiles64"].tolist() == [[1, 0], [1, 64], [1, 128], [3, 0], [3, 64]]
    assert exact.arrays["tiles128"].shape == (0, 2)                                        # 200 prompt tokens: below the threshold
    assert exact.shape == (5, 0, 3, 2047)
    # padded: two fillers behind the batch (indices 5 and 6), entries point at the last
    padded = attention_plan(q_lens + [0, 0], ctx_lens + [1, 1], filler=6)
    assert padded.arrays["singles"].tolist() == [0, 2, 4, 6, 6, 6, 6, 6] and padded.host["longest_single"] == 2048
    assert padded.arrays["tiles64"].tolist() == [[1, 0], [1, 64], [1, 128], [3, 0], [3, 64], [6, 0], [6, 0], [6, 0]]
    assert padded.shape == (8, 0, 8, 2048)
    other = attention_plan([1, 1, 129, 66, 1, 1, 0, 0], [1500, 2, 129, 100, 1025, 7, 1, 1], filler=7)
    assert other.shape == padded.shape and other.arrays["singles"].tolist() != padded.arrays["singles"].tolist()
    # many prompt tokens: the 128-row tiles too, padded at the FRONT (the kernel starts from the end of the list)
    old = attention.PREFILL_TC_MIN_TOKENS
    try:
        attention.PREFILL_TC_MIN_TOKENS = 256
        big = attention_plan([300, 1, 0], [1000, 50, 1], filler=2)
    finally:
        attention.PREFILL_TC_MIN_TOKENS = old
    t128 = big.arrays["tiles128"].tolist()
    assert len(t128) == 8 and t128[:5] == [[2, 0]] * 5 and sorted(t128[5:]) == [[0, 0], [0, 128], [0, 256]]
    assert t128[-1] == [0, 256]                                                            # the tile with the most keys starts first
    for plan in (exact, padded, big):
        assert all(a.dtype.name == "int32" for a in plan.arrays.values())


def test_parts_collect_one_plan_per_key():
    """`collect_plans` walks a model's parts and keeps one plan per key: 24 attention layers share one."""
    import boring_llm_b200 as b
    import helpers
    model = b.build_model(b.Qwen2Config.from_dict(helpers.TINY["B"]))
    plans = model.collect_plans([1, 5], [9, 5])
    assert list(plans) == ["paged attention"] and plans["paged attention"].arrays["singles"].tolist() == [0]


def test_who_takes_a_norm_that_the_product_before_has_begun():
    """`takes_pending_norm(part, rows)`: a part's `takes_pending_norm_at(rows)` decides where it has one, else its
    flag; a part that says nothing (the toy parts of the tests) and no part at all take none. The attention takes one
    from the row count of the products on pairs of SMs on (with fewer rows its norm is part of its own kernel)."""
    from boring_llm_b200.parts.base import takes_pending_norm
    from boring_llm_b200.parts.attention import GQAAttention, QKV_EPILOGUE_MIN_ROWS

    class Silent:
        pass

    class Flag:
        takes_pending_norm = True

    class ByRows:
        takes_pending_norm = True

        def takes_pending_norm_at(self, rows):
            return rows % 2 == 0

    assert not takes_pending_norm(None, 8) and not takes_pending_norm(Silent(), 8)
    assert takes_pending_norm(Flag(), 1) and takes_pending_norm(Flag(), 4096)
    assert takes_pending_norm(ByRows(), 8) and not takes_pending_norm(ByRows(), 9)
    at = GQAAttention.takes_pending_norm_at
    assert not at(None, 8) and not at(None, QKV_EPILOGUE_MIN_ROWS - 1) and at(None, QKV_EPILOGUE_MIN_ROWS) and at(None, 2048)
