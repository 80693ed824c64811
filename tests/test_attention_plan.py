"""The attention work list (host side): every tile's key range is covered exactly once by its
splits, long tiles beside many short ones are cut, even steps are not."""

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from freetoken_b200.engine.attention_plan import (DEAL_MOST_PIECES, FIXED_COST_KEYS, SPLIT_QUANTUM, TC_ONE_TILE_COSTS,
                                                  TC_TWO_TILE_COSTS, build_plan, dealt_makespan, wave_splits)


def ranges_by_tile(plan):
    tiles = {}
    for seg, tok0, ntok, kb, ke, nsplit, split, base in plan.items.tolist():
        tiles.setdefault((seg, tok0, ntok), []).append((split, kb, ke, nsplit, base))
    return tiles


@pytest.mark.parametrize("segs,group,tile,window", [
    ([(1, 1), (1, 130), (17, 17), (5, 69), (2, 64), (33, 200), (1, 65)], 3, 16, None),
    ([(300, 300), (1, 5000), (40, 1000)], 6, 128, None),
    ([(7, 90), (1, 400)], 2, 64, 32),
    ([(1, 40000)], 6, 16, None),
])
def test_splits_cover_each_tile_once(segs, group, tile, window):
    plan = build_plan(segs, group, tile, window, n_kv_heads=2)
    assert plan.n_items == plan.items.shape[0]
    slots = []
    for (seg, tok0, ntok), parts in ranges_by_tile(plan).items():
        q_len, kv_len = segs[seg]
        pos0 = kv_len - q_len
        hi = pos0 + tok0 + ntok
        lo = max(0, pos0 + tok0 - window + 1) if window else 0
        parts.sort()
        assert [p[0] for p in parts] == list(range(len(parts))) and all(p[3] == len(parts) for p in parts)
        assert parts[0][1] == lo and parts[-1][2] == hi
        for (_, _, e0, _, _), (_, b1, _, _, _) in zip(parts, parts[1:]):
            assert e0 == b1 and (b1 - lo) % SPLIT_QUANTUM == 0
        if len(parts) > 1:
            slots += list(range(parts[0][4], parts[0][4] + len(parts)))
    assert sorted(slots) == list(range(plan.n_slots)), "partial slots are used once each"


SEGMENT = st.tuples(st.sampled_from([1, 1, 1, 2, 5, 17, 64, 300, 512, 1300, 2048]),
                    st.sampled_from([0, 0, 3, 64, 500, 3000, 20000, 70000])).map(lambda qp: (qp[0], qp[0] + qp[1]))


@settings(max_examples=150, deadline=None)
@given(segs=st.lists(SEGMENT, min_size=1, max_size=12), group=st.sampled_from([1, 3, 6, 8]),
       tile=st.sampled_from([16, 64, 128, 256]), window=st.sampled_from([None, None, 32, 500]),
       n_kv=st.sampled_from([1, 2, 8]), sm=st.sampled_from([74, 148]), fixed=st.sampled_from([None, None, 1, 2, 5]),
       key_tile=st.sampled_from([None, 0, 128]), priced=st.booleans())
def test_any_step_is_covered_once_by_its_work_list(segs, group, tile, window, n_kv, sm, fixed, key_tile, priced):
    """Whatever the step, the kernel form, the window and the way the pieces are chosen (fixed counts for graph
    replay, the wave rule, the dealing search with or without the kernels' costs): every tile of whole tokens is
    there once, its pieces follow each other from its first visible key to its last without a gap, cuts lie on
    the kernel's quantum, every cut tile has partial slots of its own, and a list for the kernels that deal it
    out themselves is sorted by length."""
    if tile < group:
        tile = 64 if group > 16 else 16
    costs = (TC_TWO_TILE_COSTS if tile == 256 else TC_ONE_TILE_COSTS) if (priced and tile >= 128) else None
    plan = build_plan(segs, group, tile, window, n_kv, sm_count=sm, fixed_splits=fixed, key_tile=key_tile, costs=costs)
    quantum = 128 if (key_tile == 128 or (key_tile is None and tile >= 128)) else SPLIT_QUANTUM
    tpt = 2 * max(1, 128 // group) if tile == 256 else max(1, tile // group)
    want_tiles = {(s, t0, min(tpt, q - t0)) for s, (q, _) in enumerate(segs) for t0 in range(0, q, tpt)}
    by_tile = ranges_by_tile(plan)
    assert set(by_tile) == want_tiles
    used_slots = []
    for (seg, tok0, ntok), parts in by_tile.items():
        q_len, kv_len = segs[seg]
        pos0 = kv_len - q_len
        hi = pos0 + tok0 + ntok
        lo = max(0, pos0 + tok0 - window + 1) if window else 0
        parts.sort()
        assert [p[0] for p in parts] == list(range(len(parts))) and all(p[3] == len(parts) for p in parts)
        assert parts[0][1] == lo and parts[-1][2] == hi
        for (_, kb, ke, _, _), (_, kb2, _, _, _) in zip(parts, parts[1:]):
            assert kb <= ke == kb2 and ((ke - lo) % quantum == 0 or ke == hi)
        if len(parts) > 1:
            assert len({p[4] for p in parts}) == 1
            used_slots += list(range(parts[0][4], parts[0][4] + len(parts)))
    assert len(set(used_slots)) == len(used_slots) and all(0 <= x < plan.n_slots for x in used_slots)
    if quantum == 128:
        lengths = (plan.items[:, 4] - plan.items[:, 3]).tolist()
        assert lengths == sorted(lengths)
    if fixed is not None and fixed > 1:
        assert plan.n_items == fixed * len(want_tiles) and plan.n_slots == plan.n_items  # what a graph was recorded with
    if costs is not None and fixed is None:
        assert plan.est_us is None or plan.est_us > 0


def test_a_long_portion_beside_many_single_tokens_is_cut():
    """63 decoded tokens over 2k contexts beside a 512-token portion over a 100k-token prefix: the long
    tiles are split so that no SM is left alone with one of them; an even prefill is left whole."""
    segs = [(1, 2000 + i) for i in range(63)] + [(512, 100_000)]
    plan = build_plan(segs, 6, 128, None, n_kv_heads=8, sm_count=74)
    long_tiles = [parts for (seg, _, _), parts in ranges_by_tile(plan).items() if seg == 63]
    assert all(len(parts) >= 2 for parts in long_tiles)
    longest = max(ke - kb for parts in long_tiles for _, kb, ke, _, _ in parts)
    total = sum(ke - kb for _, _, _, kb, ke, _, _, _ in plan.items.tolist())
    assert longest <= 0.75 * total * 8 / (2 * 74), "no piece near the fair share of an SM"
    even = build_plan([(2048, 2048)], 6, 128, None, n_kv_heads=8, sm_count=74)
    assert even.n_slots == 0
    batch = build_plan([(1, 2048)] * 64, 6, 16, None, n_kv_heads=8)
    assert batch.n_slots == 0, "64 equal requests fill the GPU as they are"
    one_long = build_plan([(1, 2048)] * 63 + [(1, 100_000)], 6, 16, None, n_kv_heads=8)
    assert one_long.n_slots >= 16, "the one long request is cut"


def test_wave_splits_prefers_full_waves():
    assert wave_splits(64, 296, 16, 2048) in (4, 5)  # 64 tiles on 296 slots: 4 or 5 splits fill a wave
    assert wave_splits(512, 296, 16, 2048) == 1       # already more tiles than slots
    assert wave_splits(8, 296, 1, 128) == 1           # the caller's limit (no piece under 256 keys) holds
    assert wave_splits(8, 296, 16, 2048) == 16        # one request alone: as many pieces as allowed


def test_the_128_row_kernel_gets_pieces_on_tile_boundaries_sorted_by_length():
    # one long portion beside single tokens of other requests, as the 128-row kernel gets it
    segs = [(512, 20000)] + [(1, 100 + 37 * i) for i in range(20)]
    plan = build_plan(segs, 6, 128, None, n_kv_heads=8, sm_count=74)
    spans = [ke - kb for _, _, _, kb, ke, _, _, _ in plan.items.tolist()]
    assert spans == sorted(spans), "the kernel deals the list out from its end: longest pieces last"
    for (seg, tok0, ntok), parts in ranges_by_tile(plan).items():
        parts.sort()
        lo = parts[0][1]
        for (_, _, e0, _, _) in parts[:-1]:
            assert (e0 - lo) % 128 == 0, "a piece ends where a 128-key tile ends"
    # a fixed number of rows (graph replay): as many rows and slots whatever the lengths, dealt by length
    fixed = build_plan([(1, 3000), (1, 500)], 6, 128, None, n_kv_heads=8, fixed_splits=3)
    assert sorted(r[0] for r in fixed.items.tolist()) == [0, 0, 0, 0, 0, 1] and fixed.n_slots == 6
    spans = [r[4] - r[3] for r in fixed.items.tolist()]
    assert spans == sorted(spans)


def test_fixed_plans_deal_their_rows_by_length():
    """Graph-replayed decode steps: the number of item rows and of scratch slots depends on the batch size
    and the split count only, the rows go to the requests in proportion to their lengths, every key is in
    exactly one piece, and equal lengths give the plan they always gave."""
    from freetoken_b200.engine.attention_plan import deal_rows

    assert deal_rows([2048] * 8, 16, 32) == [2] * 8
    assert deal_rows([1000, 20000, 5000, 100], 16, 32) == [1, 12, 2, 1]
    assert deal_rows([10, 10], 6, 2) == [3, 3]          # more rows than the cap allows: still all dealt
    assert deal_rows([5], 4, 32) == [4] and deal_rows([], 4, 32) == []
    rng = np.random.default_rng(0)
    for _ in range(50):
        b, s = int(rng.integers(1, 20)), int(rng.integers(1, 9))
        segs = [(1, int(rng.integers(1, 30000))) for _ in range(b)]
        for key_tile in (0, 128):
            plan = build_plan(segs, 6, 16, None, n_kv_heads=8, fixed_splits=s, key_tile=key_tile)
            assert plan.n_items == b * s
            assert plan.n_slots == (b * s if s > 1 else 0)
            covered = {i: [] for i in range(b)}
            for seg, tok0, ntok, kb, ke, nsplit, split, base in plan.items.tolist():
                assert 1 <= nsplit <= 64 and 0 <= split < nsplit and 0 <= kb <= ke <= segs[seg][1]
                assert nsplit == 1 or base + nsplit <= plan.n_slots
                covered[seg].append((kb, ke, nsplit, base))
            for i, parts in covered.items():
                parts.sort()
                assert len(parts) == parts[0][2] and len({p[3] for p in parts}) == 1
                real = [(a, e) for a, e, _, _ in parts if e > a]
                assert real[0][0] == 0 and real[-1][1] == segs[i][1]
                assert all(real[j][1] == real[j + 1][0] for j in range(len(real) - 1))
            longest = max(ke - kb for _, _, _, kb, ke, _, _, _ in plan.items.tolist())
            fair = sum(kv for _, kv in segs) / (b * s)
            if s > 1 and max(kv for _, kv in segs) / s > 2048:
                assert longest <= 2.2 * fair + 2 * 128 + 256, (segs, s, longest, fair)
    same = build_plan([(1, 2100)] * 8, 6, 16, None, n_kv_heads=8, fixed_splits=2, key_tile=128)
    assert sorted((r[0], r[3], r[4], r[5], r[6]) for r in same.items.tolist()) == sorted(
        (i, kb, ke, 2, j) for i in range(8) for j, (kb, ke) in enumerate([(0, 1152), (1152, 2100)]))


def test_lists_of_a_few_pieces_per_cta_are_cut_so_that_the_dealing_ends_soonest():
    """The tcgen05 kernels run 148 CTAs through the sorted list, to and fro.  A 512-token portion after
    65,024 tokens is 25 tiles x 8 KV heads = 200 equally long pieces: whole they take two rounds, as halves
    three half rounds.  With two query tiles per piece (104 pieces) quarters take three quarter rounds."""
    # the model itself: 200 equal pieces on 148 CTAs, then 400 halves
    assert dealt_makespan([1280.0] * 25, 8, 148, 128) == 2 * 1280
    assert dealt_makespan([640.0] * 50, 8, 148, 128) == 3 * 640
    # sorted, the longest first, to and fro: the CTA with the longest piece gets the shortest of the next round
    assert dealt_makespan([128.0, 256.0, 384.0, 512.0], 1, 2, 128) == 640

    segs = [(512, 65536)]
    one = build_plan(segs, 6, 128, None, 8, sm_count=74, key_tile=128)
    assert set(one.items[:, 5].tolist()) == {2} and one.n_items == 50
    pair = build_plan(segs, 6, 256, None, 8, sm_count=74, key_tile=128)
    assert set(pair.items[:, 5].tolist()) == {4} and pair.n_items == 52
    for plan in (one, pair):  # never more pieces than partial results are set aside for
        assert plan.n_slots * 8 <= DEAL_MOST_PIECES * 148
        for parts in ranges_by_tile(plan).values():
            parts.sort()
            assert parts[0][1] == 0 and all(a[2] == b[1] for a, b in zip(parts, parts[1:]))
            assert all((b - 0) % 128 == 0 for _, b, _, _, _ in parts)
    # what the choice rests on: the busiest CTA's keys, whole against cut
    def busiest(plan):
        return dealt_makespan([FIXED_COST_KEYS + ke - kb for _, _, _, kb, ke, _, _, _ in plan.items.tolist()], 8, 148, 128)
    whole = build_plan(segs, 6, 128, None, 8, sm_count=74, key_tile=128, max_splits=1)
    assert set(whole.items[:, 5].tolist()) == {1}
    assert busiest(one) < 0.8 * busiest(whole)

    # a whole prompt of 2,048 tokens has pieces of every length: dealt to and fro they end together, no cut
    fresh = build_plan([(2048, 2048)], 6, 256, None, 8, sm_count=74, key_tile=128)
    assert set(fresh.items[:, 5].tolist()) == {1}
    # graph-replayed plans keep their fixed number of rows
    fixed = build_plan([(1, 4096)] * 8, 6, 16, None, 8, sm_count=74, key_tile=128, fixed_splits=2)
    assert fixed.n_items == 16


def test_a_step_takes_the_tcgen05_attention_form_whose_work_list_ends_sooner():
    """Long steps choose between one and two query tiles a piece by the estimated time of each form's work list
    (the kernel's measured costs per piece, the dealing played through).  The cases are timings on a B200:
    (tokens of the portion, tokens before it) -> microseconds with one tile a piece, with two."""
    from freetoken_b200.engine.step import StepBuilder

    measured = {(256, 0): (10.8, 14.0), (768, 0): (23.5, 24.7), (1024, 0): (34.2, 32.3), (4096, 0): (291.6, 243.9),
                (256, 4096): (53.8, 62.6), (256, 65536): (538.8, 488.5), (512, 4096): (109.1, 91.7),
                (512, 65024): (1050.8, 895.9), (768, 8192): (190.1, 264.2), (1024, 8192): (281.9, 297.7),
                (1024, 32768): (1044.7, 938.5), (2048, 8192): (592.6, 503.5)}
    for (tokens, past), (one, two) in measured.items():
        builder = StepBuilder(None, [(tokens, past + tokens)], False, 148)
        rows = builder.cheaper_attention_rows(6, None, 8, 128)
        assert rows == (256 if two < one else 128), (tokens, past)
        for form, us in ((128, one), (256, two)):
            plan = builder._drafts[("attention", 6, form, None, 8, 128, False)]
            assert abs(plan.est_us / us - 1) < 0.12, (tokens, past, form, plan.est_us, us)
        # the list of the chosen form is the one the step then uses
        key = builder.attention_plan(6, rows, None, 8, 128)
        assert builder.plans[key].est_us is not None and len(builder.sections) == 1
    # graph-replayed decode steps keep their fixed lists: no estimate, no choice
    fixed = StepBuilder(None, [(1, 4096)] * 8, True, 148)
    assert fixed.plans[fixed.attention_plan(6, 16, None, 8, 128, few_rows=True)].est_us is None


def test_which_attention_kernel_a_step_gets():
    """The rows per CTA (and the few-rows flag) name the kernel: 16 float32 / small bfloat16 tiles, 64
    mma.sync, 128 tcgen05 with one query tile, 256 with two (steps of a thousand tokens and more), 16
    with the flag for decode steps on tcgen05."""
    import torch

    from freetoken_b200.parts.attention import (TC_MIN_TOKENS, TC_PAIR_MIN_TOKENS, attention_kernel_form as form,
                                                attention_tile_rows as rows)

    bf, f32 = torch.bfloat16, torch.float32
    assert rows(f32, False, 6, 4096, 128, 16) == 16 and rows(f32, True, 6, 8, 128, 16) == 16
    assert form(bf, True, 6, 8, 128, 16, None, 4096) == (16, True)   # decode on the tcgen05 kernel, few rows
    assert form(bf, True, 16, 8, 128, 16, None, 4096) == (16, True)
    assert form(bf, True, 24, 8, 128, 16, None, 4096) == (128, False)  # a group too large for its 16 columns
    assert form(bf, True, 6, 8, 64, 16, None, 4096) == (16, False)
    assert form(bf, False, 6, 4096, 128, 16) == (256, False)
    assert rows(bf, True, 6, 8, 64, 16, None, 4096) == 16            # head size it does not take
    assert rows(bf, True, 6, 8, 128, 16, 512, 4096) == 16            # a window
    assert rows(bf, True, 6, 8, 128, 8, None, 4096) == 16            # pages of 8 tokens
    assert rows(bf, False, 6, TC_MIN_TOKENS - 1, 128, 16) == 64
    assert rows(bf, False, 6, TC_MIN_TOKENS, 128, 16) == 128
    assert rows(bf, False, 6, TC_PAIR_MIN_TOKENS, 128, 16) == 256
    # a portion of a long prompt is cut along the keys into enough pieces for two tiles per CTA
    assert rows(bf, False, 6, 512, 128, 16, None, 65536) == 256 and rows(bf, False, 6, 512, 128, 16, None, 8192) == 128
    assert rows(bf, False, 6, 200, 128, 16, None, 65536) == 128
    assert rows(bf, False, 6, 4096, 80, 16) == 64
