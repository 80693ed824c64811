"""Host-side work list for the paged attention kernels.

One step's queries are cut into tiles of whole tokens (a tile holds the ``group`` query
heads of one KV head for ``tokens_per_tile`` consecutive tokens of one segment).  A tile
whose visible key range is long and that would leave SMs idle is split along the keys;
each split writes a partial result (running max, sum, unnormalised output) that a merge
kernel combines in split order.  The reference fixes 8 splits for decode
(python/freetoken/attention/triton.py:90, python/freetoken/kernel/triton/attention.py:352-466)
and never splits prefill; here the count follows the work so that a single long request
still fills the GPU.

A work item is 8 int32: segment, first token of the tile (within the segment), tokens in
the tile, first key, one past the last key, number of splits of the tile, index of this
split, and the tile's first partial slot.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

ITEM_INTS = 8
SPLIT_QUANTUM = 64  # split boundaries are multiples of this many keys (of 128 for the kernel with 128-key tiles)


@dataclass
class AttentionPlan:
    items: np.ndarray  # [W, 8] int32
    n_items: int
    n_slots: int  # partial slots used (0 when nothing is split)
    tokens_per_tile: int
    max_splits: int


FIXED_COST_KEYS = 100  # what a CTA's start-up, write-out and merge cost, in keys' worth of time


def wave_splits(base_ctas: int, slots: int, limit: int, span: int = 2048) -> int:
    """Number of key splits (1..limit) with the shortest estimated time.

    ``base_ctas`` CTAs would run without splitting, ``slots`` CTAs are resident at once, ``span`` keys
    lie in a tile's range.  Time ~ waves x (fixed cost + keys per split): a last, partly filled wave
    costs a whole wave, and every split pays the fixed cost again.  Ties go to fewer splits."""
    best, best_t = 1, None
    for s in range(1, max(1, limit) + 1):
        waves = -(-base_ctas * s // slots)
        t = waves * (FIXED_COST_KEYS + span / s)
        if best_t is None or t < best_t * 0.98:
            best, best_t = s, t
    return best


SPLIT_COST_KEYS = 100  # what writing a piece's partial result and merging it costs on top, in keys' worth of time
DEAL_MOST_CUTS = 16    # the longest tile is tried in up to this many pieces
DEAL_SEARCH_LIMIT = 8  # lists of more than this many pieces per CTA are dealt evenly enough as they are
DEAL_MOST_PIECES = 4   # pieces of cut tiles per CTA that partial results are set aside for


def dealt_makespan(costs: Sequence[float], n_kv_heads: int, ctas: int, key_tile: int) -> float:
    """The busiest CTA's load when the tcgen05 kernels deal a list out: the pieces sorted by length, each
    once per KV head, the longest first, round after round to and fro over ``min(ctas, pieces)`` CTAs.
    ``costs`` are in keys; a piece pays for whole key tiles."""
    c = np.sort(np.asarray(costs, dtype=np.float64))[::-1]
    c = np.ceil(c / key_tile) * key_tile
    c = np.repeat(c, n_kv_heads)
    g = max(1, min(ctas, c.shape[0]))
    rounds = -(-c.shape[0] // g)
    c = np.concatenate([c, np.zeros(rounds * g - c.shape[0])]).reshape(rounds, g)
    c[1::2] = c[1::2, ::-1]
    return float(c.sum(axis=0).max())


def deal_rows(spans: Sequence[int], total: int, cap: int) -> List[int]:
    """``total`` item rows dealt to tiles in proportion to their key spans: every tile at least one, none
    more than ``cap`` (as far as ``total`` allows), the sum exactly ``total``.  Equal spans get equal shares."""
    n = len(spans)
    if n == 0:
        return []
    total = max(total, n)
    weight = [max(1, int(sp)) for sp in spans]
    whole = sum(weight)
    want = [w * total / whole for w in weight]
    got = [max(1, min(cap, int(x))) for x in want]
    # hand out what is left by largest remainder, take back what is too much from the largest shares
    while sum(got) < total:
        open_ = [i for i in range(n) if got[i] < cap]
        if not open_:
            open_ = list(range(n))  # every tile is at the cap: the rest are empty rows on the longest tiles
        i = max(open_, key=lambda j: (want[j] - got[j], weight[j], -j))
        got[i] += 1
    while sum(got) > total:
        i = max((j for j in range(n) if got[j] > 1), key=lambda j: (got[j] - want[j], -weight[j], j))
        got[i] -= 1
    return got


def tokens_per_tile(tile_rows: int, group: int) -> int:
    if tile_rows == 256:  # two tiles of 128 rows, each with whole tokens
        return 2 * max(1, 128 // group)
    return max(1, tile_rows // group)


def build_plan(segments: Sequence[Tuple[int, int]], group: int, tile_rows: int,
               window: Optional[int], n_kv_heads: int, sm_count: int = 148,
               max_splits: int = 32, min_split_keys: int = 256,
               fixed_splits: Optional[int] = None,
               sparse: Optional[Tuple[int, int]] = None, key_tile: Optional[int] = None) -> AttentionPlan:
    """``segments`` holds (q_len, kv_len) per segment, in step order.

    ``fixed_splits`` fixes the number of item rows at that many per tile on average: the rows are dealt
    to the tiles in proportion to their key spans (:func:`deal_rows`; a request of 20,000 tokens beside one
    of 1,000 gets twenty times the pieces, so that the pieces are about equally long; rows a tile cannot
    use get an empty key range).  CUDA-graph replay uses it so that the item count and the number of
    scratch slots of a step never change.

    ``key_tile`` is the number of keys the kernel walks at a time when it is one that runs one CTA per
    SM through the whole list (128 for the tcgen05 kernels; None: 128 for tiles of 128 rows and more,
    else 0): pieces are then multiples of it, the list is sorted by length, and for lists of a few pieces
    per CTA the number of pieces per tile is the one with which the kernel's dealing ends soonest
    (:func:`dealt_makespan`).

    ``sparse = (block_size, topk)`` plans a block-sparse layer: one token per tile (every token has
    its own choice of key blocks) and key ranges that count chosen keys: ``min(topk, visible
    blocks) * block_size`` of them."""
    if key_tile is None:
        key_tile = 128 if tile_rows >= 128 else 0
    tpt = 1 if sparse else tokens_per_tile(tile_rows, group)
    tiles: List[Tuple[int, int, int, int, int]] = []  # seg, tok0, ntok, lo, hi
    for s, (q_len, kv_len) in enumerate(segments):
        pos0 = kv_len - q_len
        for tok0 in range(0, q_len, tpt):
            ntok = min(tpt, q_len - tok0)
            hi = pos0 + tok0 + ntok  # last query's position + 1
            lo = 0
            if window is not None:
                lo = max(0, pos0 + tok0 - window + 1)
            if sparse:
                block, topk = sparse
                lo, hi = 0, min(topk, (pos0 + tok0) // block + 1) * block
            tiles.append((s, tok0, ntok, lo, hi))
    n_tiles = len(tiles)
    target = 2 * sm_count
    # keys of all tiles together, per resident CTA: a tile that is long against that and against the
    # other tiles would keep one SM busy long after the rest is done (a long portion beside many
    # single tokens), so it is cut into pieces of half that share
    all_keys = sum(hi - lo for _, _, _, lo, hi in tiles)
    piece = max(all_keys * n_kv_heads / max(1, target) / 2, float(min_split_keys))
    mean_span = all_keys / max(1, n_tiles)
    rows: List[List[int]] = []
    n_slots = 0
    dealt = None
    if fixed_splits is not None and fixed_splits > 1:
        dealt = deal_rows([hi - lo for _, _, _, lo, hi in tiles], n_tiles * fixed_splits, max(fixed_splits, max_splits))
    quantum = key_tile if key_tile else SPLIT_QUANTUM  # a piece that ends inside a key tile pays for all of it
    wants: List[int] = []
    mosts: List[int] = []
    for ti, (s, tok0, ntok, lo, hi) in enumerate(tiles):
        span = hi - lo
        most = min(max_splits, max(1, span // min_split_keys))
        if fixed_splits is not None:
            want = dealt[ti] if dealt is not None else fixed_splits
        elif n_tiles * n_kv_heads >= target:
            want = 1
            if span > piece and span > 2 * mean_span:
                want = max(1, min(most, int(-(-span // piece))))
        else:
            # splits that fill whole waves of resident CTAs, none shorter than min_split_keys
            if key_tile:  # (no more pieces than the mixers set partial results aside for)
                most = max(1, min(most, DEAL_MOST_PIECES * target // (n_tiles * n_kv_heads)))
            want = wave_splits(n_tiles * n_kv_heads, target, most, span)
        wants.append(want)
        mosts.append(most)

    def cut(span: int, want: int) -> Tuple[int, int]:
        """(keys per piece, pieces) of a tile cut into at most ``want`` pieces of whole quanta."""
        quanta = -(-span // quantum)
        n_real = max(1, min(want, quanta))
        per = -(-quanta // n_real) * quantum
        return per, (max(1, -(-span // per)) if span > 0 else 1)

    if key_tile and fixed_splits is None and n_tiles * n_kv_heads <= DEAL_SEARCH_LIMIT * target:
        # The tcgen05 kernels run one CTA per SM through the sorted list, to and fro; with a few pieces per
        # CTA the last round decides (200 equal pieces on 148 CTAs take two rounds, 400 halves three half
        # rounds).  So: the counts from above against pieces of at most L keys for a few L (a k-th of the
        # longest tile; shorter tiles get fewer pieces), the kernel's dealing played through for each.
        spans = np.asarray([hi - lo for _, _, _, lo, hi in tiles], dtype=np.int64)
        quanta = -(-spans // quantum)
        cap = np.asarray(mosts, dtype=np.int64)

        def played(counts: np.ndarray) -> Optional[float]:
            n = np.maximum(1, np.minimum(counts, quanta))
            per = -(-quanta // n) * quantum          # keys per piece, as cut() has them
            n = np.where(spans > 0, np.maximum(1, -(-spans // per)), 1)
            if int(n[n > 1].sum()) * n_kv_heads > DEAL_MOST_PIECES * target:
                return None  # (the partial results of so many pieces would not fit what the mixers set aside)
            costs = np.repeat(per, n).astype(np.float64)
            last = np.cumsum(n) - 1
            costs[last] = spans - (n - 1) * per      # a tile's last piece is what is left
            costs += FIXED_COST_KEYS + np.repeat(np.where(n > 1, SPLIT_COST_KEYS, 0), n)
            return dealt_makespan(costs, n_kv_heads, target, key_tile)

        best = np.asarray(wants, dtype=np.int64)
        best_t = played(best)
        longest = int(spans.max()) if n_tiles else 0
        seen = None
        for k in range(1, DEAL_MOST_CUTS + 1):
            limit = -(-longest // (k * quantum)) * quantum  # keys per piece
            if limit < min_split_keys:
                break
            counts = np.maximum(1, np.minimum(cap, -(-spans // limit)))
            if seen is not None and np.array_equal(counts, seen):
                continue
            seen = counts
            t = played(counts)
            if t is None:
                break  # (more cuts need more room still)
            if best_t is None or t < best_t * 0.97:
                best, best_t = counts, t
        wants = [int(x) for x in best]

    for ti, (s, tok0, ntok, lo, hi) in enumerate(tiles):
        span = hi - lo
        want = wants[ti]
        per, n_real = cut(span, want)
        n_rows = want if fixed_splits is not None else n_real
        base = n_slots if n_rows > 1 else 0
        for i in range(n_rows):
            b = min(hi, lo + i * per)
            e = min(hi, lo + (i + 1) * per)
            rows.append([s, tok0, ntok, b, e, n_rows, i, base])
        if n_rows > 1 or dealt is not None:  # (fixed plans: the slots are numbered the same whatever the shares)
            n_slots += n_rows
    if key_tile:
        # the tcgen05 kernels deal the list out from its end, to and fro over its CTAs: longest pieces last
        # here (their place in the list means nothing else: partial results are found by base + split)
        rows.sort(key=lambda r: r[4] - r[3])
    items = np.asarray(rows, dtype=np.int32).reshape(-1, ITEM_INTS)
    return AttentionPlan(items=items, n_items=items.shape[0], n_slots=n_slots,
                         tokens_per_tile=tpt, max_splits=max_splits)
