"""The launch list of the tcgen05 prefill attention (host side, no GPU)."""
import random

from boring_llm_b200.parts.attention import tc_attention_blocks


def covered(blocks, q_lens):
    rows = {r: [0] * n for r, n in enumerate(q_lens) if n > 1}
    for r, t0, limit in blocks:
        assert limit in (128, 256) and t0 % 128 == 0
        for t in range(t0, min(t0 + limit, q_lens[r])):
            rows[r][t] += 1
    return all(all(c == 1 for c in v) for v in rows.values())


def test_every_row_is_in_exactly_one_block():
    rng = random.Random(3)
    for _ in range(200):
        R = rng.randint(1, 6)
        q_lens = [rng.choice([1, 1, 2, 17, 128, 129, 255, 256, 257, 700, 2048]) for _ in range(R)]
        ctx_lens = [n + rng.choice([0, 5, 300, 4000]) for n in q_lens]
        for heads, sms in [(14, 148), (2, 148), (4, 1), (64, 148)]:
            blocks = tc_attention_blocks(q_lens, ctx_lens, heads, sms)
            assert covered(blocks, q_lens), (q_lens, ctx_lens, heads, sms, blocks)
            assert all(q_lens[r] > 1 for r, _, _ in blocks)


def test_pairs_stay_together_when_the_sms_are_filled_and_split_heaviest_first_when_not():
    full = tc_attention_blocks([8192], [8192], 14)
    assert len(full) == 32 and all(rows == 256 for _, _, rows in full)
    few = tc_attention_blocks([2048], [2048], 14)
    assert len(few) * 14 >= 148 > (len(few) - 1) * 14
    singles = [t0 for _, t0, rows in few if rows == 128]
    pairs = [t0 for _, t0, rows in few if rows == 256]
    assert singles and pairs and min(singles) > max(pairs)          # the blocks with the most keys were split
    assert few[-1][1] == max(t0 for _, t0, _ in few) or few[-1][2] == 256   # the costliest block is launched first (last in the list)
