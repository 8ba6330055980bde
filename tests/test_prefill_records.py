"""The work list of the tcgen05 prefill kernel, as the host makes it (no GPU needed)."""
import random

import numpy as np

from tokamak_b200.csrc import ops


def blocks_of(q_start, q_len, kv_len, slots):
    out = {}
    for r in range(len(q_len)):
        if q_len[r] <= 1:
            continue
        for b in range(-(-q_len[r] // ops.PREFILL_TC_ROWS)):
            rows = min(ops.PREFILL_TC_ROWS, q_len[r] - ops.PREFILL_TC_ROWS * b)
            pos0 = kv_len[r] - q_len[r] + ops.PREFILL_TC_ROWS * b
            out[q_start[r] + ops.PREFILL_TC_ROWS * b] = (rows, pos0, slots[r], (pos0 + rows - 1) // ops.PREFILL_TC_KEYS + 1)
    return out


def check(q_len, kv_len, heads, sms):
    q_start = list(np.cumsum([0] + q_len[:-1]))
    slots = list(range(10, 10 + len(q_len)))
    records, n_parts, n_split = ops.prefill_tc_records(q_start, q_len, kv_len, slots, heads=heads, sms=sms)
    assert records.dtype == np.int32 and records.shape[1] == ops.PREFILL_TC_RECORD
    want = blocks_of(q_start, q_len, kv_len, slots)
    lengths = [int(r[5] - r[4]) for r in records]
    assert lengths == sorted(lengths, reverse=True)                 # longest first
    seen, cut, mergers = {}, {}, {}
    for i, (tok0, rows, pos0, slot, kb, ke, part, parts, poff, split, merger, _) in enumerate(records.tolist()):
        assert merger in (0, 1) and (parts > 1 or merger == 0)
        if parts > 1:
            mergers.setdefault(tok0, []).append((i, merger))
        assert (rows, pos0, slot) == want[tok0][:3]
        assert 0 <= kb < ke <= want[tok0][3] and 0 <= part < parts <= ops.PREFILL_TC_MAX_PARTS
        seen.setdefault(tok0, []).append((part, kb, ke, parts))
        if parts > 1:
            assert ke - kb >= ops.PREFILL_TC_MIN_PART
            cut.setdefault(tok0, set()).add((poff, split, parts))
        else:
            assert (poff, split) == (0, 0)
    assert set(seen) == set(want)                                   # every block of tokens is there
    for tok0, parts in seen.items():
        parts.sort()
        assert [p[0] for p in parts] == list(range(parts[0][3]))    # each part once
        assert parts[0][1] == 0 and parts[-1][2] == want[tok0][3]   # the parts cover all key tiles,
        assert all(a[2] == b[1] for a, b in zip(parts, parts[1:]))  # one after the other
    # exactly one part of a cut block adds the parts up: the one listed last
    for rows_of in mergers.values():
        assert [m for _, m in sorted(rows_of)] == [0] * (len(rows_of) - 1) + [1]
    # the cut blocks' scratch ranges [poff, poff + parts) do not overlap, their counters differ
    spans = sorted(next(iter(v)) for v in cut.values())
    assert all(len(v) == 1 for v in cut.values())
    assert all(a[0] + a[2] <= b[0] for a, b in zip(spans, spans[1:]))
    assert sorted(s[1] for s in spans) == list(range(n_split))
    assert n_parts == sum(s[2] for s in spans)
    return records, n_parts, n_split


def test_no_cut_when_there_is_enough_work():
    records, n_parts, n_split = check([2048] * 4, [2048] * 4, heads=32, sms=148)
    assert n_split == 0 and len(records) == 4 * 8


def test_one_portion_against_a_long_context_is_cut():
    records, n_parts, n_split = check([256, 1, 1], [4096, 900, 17], heads=32, sms=148)
    assert (n_split, n_parts) == (1, 4)               # 32 items: four parts each fill 128 of the 148 SMs
    assert max(int(r[5] - r[4]) for r in records) == 16
    records, n_parts, n_split = check([512, 1, 1], [4096, 900, 17], heads=40, sms=148)
    assert n_split == 0                                # 80 items: a second part of each would not fit the round


def test_single_tokens_make_no_items():
    records, n_parts, n_split = check([1, 1], [5, 6], heads=8, sms=148)
    assert records.shape == (0, ops.PREFILL_TC_RECORD) and (n_parts, n_split) == (0, 0)


def test_random_batches():
    rng = random.Random(3)
    for _ in range(200):
        n = rng.randint(1, 6)
        q_len = [rng.choice([1, 2, 100, 256, 257, 700, 3000]) for _ in range(n)]
        kv_len = [q + rng.choice([0, 5, 1000, 20000]) for q in q_len]
        check(q_len, kv_len, heads=rng.choice([1, 8, 40]), sms=rng.choice([1, 148, 1 << 20]))
