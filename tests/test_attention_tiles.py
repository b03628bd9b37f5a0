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
