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
    est_us: Optional[float] = None  # the launch's estimated time, where the kernel's costs per piece were given


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


@dataclass(frozen=True)
class PieceCosts:
    """What a piece of work costs a tcgen05 attention kernel, fitted to timings on a B200 (21 portions of 256
    to 4,096 tokens after 0 to 65,536 earlier ones, both forms; the estimates built on these are within 10 % of
    every one of them and name the faster form in every case): microseconds per 128-key tile of a piece, per
    piece, and on top per piece of a tile that is cut along the keys (its partial result is written in 32-bit
    and merged)."""
    us_per_key_tile: float
    fixed_us: float
    split_us: float


TC_ONE_TILE_COSTS = PieceCosts(1.35, 4.0, 3.0)  # 128 query rows a piece
TC_TWO_TILE_COSTS = PieceCosts(2.1, 6.0, 9.0)   # 256 query rows a piece (two tiles on the same keys)
LAUNCH_US = 4.0


def build_plan(segments: Sequence[Tuple[int, int]], group: int, tile_rows: int,
               window: Optional[int], n_kv_heads: int, sm_count: int = 148,
               max_splits: int = 32, min_split_keys: int = 256,
               fixed_splits: Optional[int] = None,
               sparse: Optional[Tuple[int, int]] = None, key_tile: Optional[int] = None,
               costs: Optional[PieceCosts] = None) -> AttentionPlan:
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
    (:func:`dealt_makespan`).  ``costs`` gives that search the kernel's measured costs per piece and the
    plan an estimate of the launch's time (``est_us``), by which a step chooses between kernel forms.

    ``sparse = (block_size, topk)`` plans a block-sparse layer: one token per tile (every token has
    its own choice of key blocks) and key ranges that count chosen keys: ``min(topk, visible
    blocks) * block_size`` of them."""
    if key_tile is None:
        key_tile = 128 if tile_rows >= 128 else 0
    tpt = 1 if sparse else tokens_per_tile(tile_rows, group)
    # tiles: segment, first token, tokens, first key, one past the last key
    seg_q = np.asarray([q for q, _ in segments], dtype=np.int64).reshape(-1)
    seg_kv = np.asarray([kv for _, kv in segments], dtype=np.int64).reshape(-1)
    per_seg = -(-np.maximum(seg_q, 0) // tpt)
    seg = np.repeat(np.arange(seg_q.shape[0], dtype=np.int64), per_seg)
    tok0 = (np.arange(int(per_seg.sum()), dtype=np.int64) - (np.cumsum(per_seg) - per_seg)[seg]) * tpt
    ntok = np.minimum(tpt, seg_q[seg] - tok0)
    pos0 = (seg_kv - seg_q)[seg]
    hi = pos0 + tok0 + ntok  # last query's position + 1
    lo = np.zeros_like(hi)
    if window is not None:
        lo = np.maximum(0, pos0 + tok0 - window + 1)
    if sparse:
        block, topk = sparse
        lo = np.zeros_like(hi)
        hi = np.minimum(topk, (pos0 + tok0) // block + 1) * block
    spans = hi - lo
    n_tiles = int(spans.shape[0])
    target = 2 * sm_count
    quantum = key_tile if key_tile else SPLIT_QUANTUM  # a piece that ends inside a key tile pays for all of it
    quanta = -(-spans // quantum)
    mosts = np.minimum(max_splits, np.maximum(1, spans // min_split_keys))
    dealt = None
    if fixed_splits is not None:
        if fixed_splits > 1:
            dealt = deal_rows(spans.tolist(), n_tiles * fixed_splits, max(fixed_splits, max_splits))
            wants = np.asarray(dealt, dtype=np.int64)
        else:
            wants = np.full(n_tiles, fixed_splits, dtype=np.int64)
    elif n_tiles * n_kv_heads >= target:
        # keys of all tiles together, per resident CTA: a tile that is long against that and against the
        # other tiles would keep one SM busy long after the rest is done (a long portion beside many
        # single tokens), so it is cut into pieces of half that share
        all_keys = int(spans.sum())
        piece = max(all_keys * n_kv_heads / max(1, target) / 2, float(min_split_keys))
        mean_span = all_keys / max(1, n_tiles)
        cut_it = (spans > piece) & (spans > 2 * mean_span)
        wants = np.where(cut_it, np.maximum(1, np.minimum(mosts, np.ceil(spans / piece).astype(np.int64))), 1)
    else:
        # splits that fill whole waves of resident CTAs, none shorter than min_split_keys
        if key_tile and n_tiles:  # (no more pieces than the mixers set partial results aside for)
            mosts = np.maximum(1, np.minimum(mosts, DEAL_MOST_PIECES * target // (n_tiles * n_kv_heads)))
        known = {}
        wants = np.ones(n_tiles, dtype=np.int64)
        for i in range(n_tiles):
            k = (int(mosts[i]), int(spans[i]))
            if k not in known:
                known[k] = wave_splits(n_tiles * n_kv_heads, target, k[0], k[1])
            wants[i] = known[k]

    fixed_keys, split_keys = float(FIXED_COST_KEYS), float(SPLIT_COST_KEYS)
    if costs is not None and key_tile:
        fixed_keys = costs.fixed_us / costs.us_per_key_tile * key_tile
        split_keys = costs.split_us / costs.us_per_key_tile * key_tile

    def pieces_of(counts: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
        """(keys per piece, pieces) of every tile cut into at most ``counts`` pieces of whole quanta."""
        n = np.maximum(1, np.minimum(counts, quanta))
        per = -(-np.maximum(quanta, 1) // n) * quantum
        return per, np.where(spans > 0, np.maximum(1, -(-spans // per)), 1)

    def played(counts: np.ndarray) -> Optional[float]:
        per, n = pieces_of(counts)
        if int(n[n > 1].sum()) * n_kv_heads > DEAL_MOST_PIECES * target:
            return None  # (the partial results of so many pieces would not fit what the mixers set aside)
        piece_keys = np.repeat(per, n).astype(np.float64)
        last = np.cumsum(n) - 1
        piece_keys[last] = spans - (n - 1) * per      # a tile's last piece is what is left
        piece_keys += fixed_keys + np.repeat(np.where(n > 1, split_keys, 0.0), n)
        return dealt_makespan(piece_keys, n_kv_heads, target, key_tile)

    best_t = None
    if key_tile and fixed_splits is None and n_tiles and n_tiles * n_kv_heads <= DEAL_SEARCH_LIMIT * target:
        # The tcgen05 kernels run one CTA per SM through the sorted list, to and fro; with a few pieces per
        # CTA the last round decides (200 equal pieces on 148 CTAs take two rounds, 400 halves three half
        # rounds).  So: the counts from above against pieces of at most L keys for a few L (a k-th of the
        # longest tile; shorter tiles get fewer pieces), the kernel's dealing played through for each.
        best, best_t = wants, played(wants)
        longest = int(spans.max())
        seen = None
        for k in range(1, DEAL_MOST_CUTS + 1):
            limit = -(-longest // (k * quantum)) * quantum  # keys per piece
            if limit < min_split_keys:
                break
            counts = np.maximum(1, np.minimum(mosts, -(-spans // limit)))
            if seen is not None and np.array_equal(counts, seen):
                continue
            seen = counts
            t = played(counts)
            if t is None:
                break  # (more cuts need more room still)
            if best_t is None or t < best_t * 0.97:
                best, best_t = counts, t
        wants = best

    per, n_real = pieces_of(wants)
    n_rows = wants if fixed_splits is not None else n_real
    n_rows = np.maximum(1, n_rows)
    slotted = (n_rows > 1) | (dealt is not None)  # (fixed plans: the slots are numbered the same whatever the shares)
    slot_start = np.cumsum(np.where(slotted, n_rows, 0)) - np.where(slotted, n_rows, 0)
    n_slots = int(np.where(slotted, n_rows, 0).sum())
    tile_of = np.repeat(np.arange(n_tiles), n_rows)
    first = np.cumsum(n_rows) - n_rows
    i = np.arange(int(n_rows.sum())) - first[tile_of]
    b = np.minimum(hi[tile_of], lo[tile_of] + i * per[tile_of])
    e = np.minimum(hi[tile_of], lo[tile_of] + (i + 1) * per[tile_of])
    base = np.where(n_rows[tile_of] > 1, slot_start[tile_of], 0)
    items = np.stack([seg[tile_of], tok0[tile_of], ntok[tile_of], b, e, n_rows[tile_of], i, base], axis=1)
    if key_tile and items.shape[0]:
        # the tcgen05 kernels deal the list out from its end, to and fro over its CTAs: longest pieces last
        # here (their place in the list means nothing else: partial results are found by base + split)
        items = items[np.argsort(e - b, kind="stable")]
    items = np.ascontiguousarray(items, dtype=np.int32).reshape(-1, ITEM_INTS)
    est_us = None
    if costs is not None and key_tile and n_tiles and fixed_splits is None:
        if best_t is None:
            best_t = played(wants)
        if best_t is not None:
            est_us = best_t / key_tile * costs.us_per_key_tile + LAUNCH_US
            if n_slots:  # partial results written and read again in 32-bit (heads of 128), and the merge's launch
                est_us += 4.0 + n_slots * n_kv_heads * min(tile_rows, 256) * 130 * 4 / 4e6
    return AttentionPlan(items=items, n_items=items.shape[0], n_slots=n_slots,
                         tokens_per_tile=tpt, max_splits=max_splits, est_us=est_us)
