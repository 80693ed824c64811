"""Each CUDA kernel alone against its plain PyTorch reference (tests/kernel_refs.py), in float32
and bfloat16, at sizes other than the engine's tiny configurations: widths and vocabularies that
are no power of two, head sizes in steps of 16, odd numbers of heads and groups, pages of several
sizes, fresh pages filled with NaN so that a read of an unwritten slot shows."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import kernel_refs as ref
from freetoken_b200.engine.attention_plan import build_plan
from freetoken_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)


def attn_tol(dtype):
    """Attention outputs: the probabilities are rounded to bfloat16 before P.V (as the reference
    does, python/freetoken/kernel/triton/attention.py:252,573), an error of up to 2^-9 per
    probability times values of size up to ~4, plus the rounding of the output itself."""
    return tol(dtype) if dtype == torch.float32 else dict(rtol=2e-2, atol=1.5e-2)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    n = 1
    for d in shape:
        n *= d
    if n > 50_000_000:  # (gigabytes of expert weights: drawn on the device, the CPU takes a quarter of a minute)
        g = torch.Generator(device=DEV).manual_seed(seed + sum(shape))
        return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H,T", [(331, 112, 9), (1000, 3072, 33), (77, 50, 5)])
def test_embedding_gather(dtype, V, H, T):
    table = rnd(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    out = torch.empty(T, H, dtype=torch.float32, device=DEV)
    want = torch.empty_like(out)
    ops.embedding_gather(table, ids, out)
    ref.embedding_gather(table, ids, want)
    assert torch.equal(out, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,T,gemma", [(112, 7, True), (3072, 19, True), (50, 3, False), (6144, 4, False)])
def test_add_rmsnorm(dtype, H, T, gemma):
    x = rnd(T, H, dtype=dtype)
    res = rnd(T, H, seed=1)
    w = rnd(H, scale=0.1, seed=2)
    for mode in ("add", "residual_only", "x_only", "rows"):
        r1, r2 = res.clone(), res.clone()
        rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV) if mode == "rows" else None
        n = 3 if mode == "rows" else T
        out = torch.empty(n, H, dtype=dtype, device=DEV)
        want = torch.empty_like(out)
        o32 = torch.empty(n, H, dtype=torch.float32, device=DEV)
        w32 = torch.empty_like(o32)
        xa = None if mode == "residual_only" else x
        ra, rb = (None, None) if mode == "x_only" else (r1, r2)
        ops.add_rmsnorm(xa, ra, w, 1e-5, gemma, out, out_f32=o32, rows=rows)
        ref.add_rmsnorm(xa, rb, w, 1e-5, gemma, want, out_f32=w32, rows=rows)
        torch.testing.assert_close(out.float(), want.float(), **tol(dtype))
        torch.testing.assert_close(o32, out.float(), rtol=0, atol=0)
        if mode == "add":
            torch.testing.assert_close(r1, r2, rtol=1e-6, atol=1e-6)
        elif ra is not None:
            assert torch.equal(r1, res)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,T,k", [(3072, 8, 8), (100, 5, 3), (520, 33, 1), (48, 2, 4)])
def test_add_rmsnorm_routes_is_combine_then_norm(dtype, H, T, k):
    """The sum over routes taken inside the norm kernel: the same bits as the two kernels one after
    the other, for all rows and for chosen rows, with and without a shared expert's rows."""
    R = T * k
    y = rnd(R, H, dtype=dtype)
    pos = torch.randperm(R, generator=torch.Generator().manual_seed(4)).to(torch.int32).to(DEV)
    pos[0] = -1  # a route that went to no expert adds nothing
    shared = rnd(T, H, dtype=dtype, seed=6)
    w = rnd(H, scale=0.1, seed=2)
    res = rnd(T, H, seed=1)
    for sh in (None, shared):
        for rows in (None, torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)):
            n = T if rows is None else 2
            r1, r2 = res.clone(), res.clone()
            out, want = torch.empty(n, H, dtype=dtype, device=DEV), torch.empty(n, H, dtype=dtype, device=DEV)
            o32, w32 = torch.empty(n, H, device=DEV), torch.empty(n, H, device=DEV)
            ops.add_rmsnorm_routes(y, pos, k, sh, r1, w, 1e-5, True, out, out_f32=o32, rows=rows)
            delta = torch.empty(T, H, dtype=dtype, device=DEV)
            ops.moe_combine(y, pos, T, k, sh, delta)
            ops.add_rmsnorm(delta, r2, w, 1e-5, True, want, out_f32=w32, rows=rows)
            assert torch.equal(out, want) and torch.equal(o32, w32) and torch.equal(r1, r2)
            if rows is not None:
                assert torch.equal(r1, res)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["silu", "swigluoai"])
def test_act_and_mul(dtype, act):
    gu = rnd(13, 2 * 72, dtype=dtype, scale=4.0)
    out = torch.empty(13, 72, dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    ops.act_and_mul(gu, out, act, 1.702, 7.0)
    ref.act_and_mul(gu, want, act, 1.702, 7.0)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


def test_cast_and_table_update():
    x = rnd(1000)
    y = torch.empty(1000, dtype=torch.bfloat16, device=DEV)
    ops.cast(x, y)
    assert torch.equal(y, x.to(torch.bfloat16))
    z = torch.empty(1000, dtype=torch.float32, device=DEV)
    ops.cast(y, z)
    assert torch.equal(z, y.float())
    table = torch.zeros(4, 10, dtype=torch.int32, device=DEV)
    ups = torch.tensor([[3, 7], [-1, -1], [39, 2], [11, 5]], dtype=torch.int32, device=DEV)
    ops.table_update(table, ups, 4)
    want = torch.zeros(40, dtype=torch.int32)
    want[3], want[39], want[11] = 7, 2, 5
    assert torch.equal(table.view(-1).cpu(), want)


def make_rope(max_pos, rd, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float) / rd))
    f = torch.einsum("i,j->ij", torch.arange(max_pos, dtype=torch.float), inv)
    return torch.cat((f.cos(), f.sin()), -1).contiguous().to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,rd,P,gemma,norm", [
    (7, 1, 48, 24, 4, True, True), (6, 3, 32, 32, 8, False, False), (48, 8, 128, 64, 16, True, True),
    (5, 5, 80, 16, 3, True, True), (2, 2, 256, 128, 16, False, True), (5, 3, 64, 16, 5, True, True),
    (7, 3, 128, 0, 4, True, True), (5, 1, 128, 128, 8, False, True), (3, 2, 64, 64, 4, True, False)])
@pytest.mark.parametrize("T", [21, 150])
def test_norm_rope_store(dtype, Hq, Hkv, D, rd, P, gemma, norm, T):
    pages = -(-T // P) + 9
    x = rnd(T, (Hq + 2 * Hkv) * D, dtype=dtype)
    pos = torch.randint(0, 100, (T,), dtype=torch.int32, device=DEV)
    table = make_rope(100, rd) if rd else None
    slots = torch.randperm(pages * P)[:T].to(torch.int32).to(DEV)
    slots[5] = -1
    qw = rnd(D, scale=0.1, seed=3) if norm else None
    kw = rnd(D, scale=0.1, seed=4) if norm else None
    got, want = [], []
    for fn, store in ((ops.norm_rope_store, got), (ref.norm_rope_store, want)):
        q = torch.zeros(T, Hq, D, dtype=dtype, device=DEV)
        ks = torch.full((pages, Hkv, P, D), float("nan"), dtype=dtype, device=DEV)
        vs = torch.full((pages, Hkv, P, D), float("nan"), dtype=dtype, device=DEV)
        fn(x, D, rd, pos, table, 1e-6, gemma, [
            dict(first_head=0, n_heads=Hq, norm_weight=qw, rotate=True, dense_out=q),
            dict(first_head=Hq, n_heads=Hkv, norm_weight=kw, rotate=True, slab=ks, slot_map=slots),
            dict(first_head=Hq + Hkv, n_heads=Hkv, norm_weight=None, rotate=False, slab=vs, slot_map=slots)])
        store.extend([q, ks, vs])
    for a, b in zip(got, want):
        assert torch.equal(torch.isnan(a), torch.isnan(b))
        torch.testing.assert_close(torch.nan_to_num(a.float()), torch.nan_to_num(b.float()), **tol(dtype))


def run_attention(dtype, Hq, Hkv, D, P, segs, window, fixed_splits=None, force_split=False, seed=0, tile=None,
                  spoil_reference=None, few_rows=False, plan_kw=None):
    """segs: list of (q_len, kv_len).  Builds a shuffled page layout with NaN in every unwritten
    slot, runs kernel and reference, returns both outputs."""
    G = Hq // Hkv
    tile = tile or (64 if dtype == torch.bfloat16 else 16)
    width = max(-(-kv // P) for _, kv in segs) + 1
    n_pages = sum(-(-kv // P) for _, kv in segs) + 3
    g = torch.Generator().manual_seed(seed)
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(len(segs) + 1, width, dtype=torch.int32)
    ks = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype)
    vs = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype)
    seg_info, q_start = [], 0
    rows = list(range(len(segs), 0, -1))  # block-table rows in reverse order
    for (q_len, kv_len), row in zip(segs, rows):
        for b in range(-(-kv_len // P)):
            page = perm.pop()
            bt[row, b] = page
            n = min(P, kv_len - b * P)
            ks[page, :, :n] = torch.randn(Hkv, n, D, generator=g).to(dtype)
            vs[page, :, :n] = torch.randn(Hkv, n, D, generator=g).to(dtype)
        seg_info.append([q_start, q_len, kv_len, row])
        q_start += q_len
    T = q_start
    q = torch.randn(T, Hq, D, generator=g).to(dtype).to(DEV)
    ks, vs, bt = ks.to(DEV), vs.to(DEV), bt.to(DEV)
    seg = torch.tensor(seg_info, dtype=torch.int32, device=DEV)
    kw = dict(sm_count=148)
    if force_split:
        kw = dict(sm_count=4096, min_split_keys=32)
    if few_rows:
        kw["key_tile"] = 128
    kw.update(plan_kw or {})
    plan = build_plan(segs, G, tile, window, Hkv, fixed_splits=fixed_splits, **kw)
    items = torch.from_numpy(plan.items).to(DEV)
    part_o = part_ml = None
    if plan.n_slots:
        part_o = torch.full((plan.n_slots, Hkv, tile, D), float("nan"), dtype=torch.float32, device=DEV)
        part_ml = torch.full((plan.n_slots, Hkv, tile, 2), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full((T, Hq, D), float("nan"), dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    scale = D ** -0.5
    ops.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, part_o, part_ml, out, tile,
                        scale, window, few_rows=few_rows)
    if spoil_reference is not None:  # (segment, position): the reference is made blind to that key
        si, kpos = spoil_reference
        page = int(bt[rows[si], kpos // P])
        ks, vs = ks.clone(), vs.clone()
        qs = q[seg_info[si][0]: seg_info[si][0] + seg_info[si][1]].float().view(-1, Hkv, G, D).mean((0, 2))
        ks[page, :, kpos % P] = (-30.0 * qs / qs.norm(dim=-1, keepdim=True)).to(dtype)  # score far below the rest
        vs[page, :, kpos % P] = 0
    ref.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, None, None, want, tile, scale,
                        window)
    return out, want, plan


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,P", [(7, 1, 48, 4), (6, 3, 32, 8), (12, 2, 128, 16), (4, 4, 80, 5),
                                        (2, 1, 256, 16), (3, 3, 16, 1), (16, 2, 64, 32)])
def test_attention_mixed_batch(dtype, Hq, Hkv, D, P):
    segs = [(1, 1), (1, 130), (17, 17), (5, 69), (2, 64), (33, 200), (1, 65)]
    out, want, _ = run_attention(dtype, Hq, Hkv, D, P, segs, None)
    assert not torch.isnan(out).any()
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))


@pytest.mark.parametrize("tile", [128, 256])
@pytest.mark.parametrize("Hq,Hkv,P", [(12, 2, 16), (48, 8, 16), (5, 5, 32), (7, 1, 64), (16, 1, 16), (3, 1, 48)])
def test_attention_tensor_core_kernel(Hq, Hkv, P, tile):
    """The tcgen05 kernels (tiles of 128 query rows, one or two to a CTA, head size 128) on a mixed batch: whole prompts,
    portions with earlier keys, single tokens, lengths on and off the edges of its 128-key tiles and
    16-key boxes; every unwritten cache slot holds NaN."""
    assert ops.attention_tc_fits(128, P, Hq // Hkv)
    assert not ops.attention_tc_fits(64, P, Hq // Hkv) and not ops.attention_tc_fits(128, 8, 1)
    segs = [(300, 300), (1, 1), (128, 128), (17, 273), (1, 130), (129, 257), (40, 40), (2, 64), (250, 1000), (1, 129)]
    out, want, _ = run_attention(torch.bfloat16, Hq, Hkv, 128, P, segs, None, tile=tile)
    assert not torch.isnan(out).any()
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))
    assert ops.read_status() == 0


@pytest.mark.parametrize("tile", [128, 256])
def test_attention_tensor_core_kernel_split_keys(tile):
    """One long request alone: its tiles are split along the keys and merged."""
    segs = [(140, 3000)]
    out, want, plan = run_attention(torch.bfloat16, 12, 2, 128, 16, segs, None, force_split=True, tile=tile)
    assert plan.n_slots > 0
    assert not torch.isnan(out).any()
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))
    assert ops.read_status() == 0


@pytest.mark.parametrize("tile", [128, 256])
def test_attention_tensor_core_kernel_portion_of_a_long_prompt_beside_single_tokens(tile):
    """A 300-token portion after 19,700 earlier tokens beside decoding requests, with the work list as the
    engine makes it for these kernels (one CTA per SM, pieces on key-tile edges): the long tiles are cut along
    the keys into the number of pieces with which the kernel's dealing ends soonest, the short ones are not."""
    segs = [(300, 20000), (1, 700), (1, 128), (1, 1999), (1, 1)]
    G = 6
    plan = build_plan(segs, G, tile, None, 2, sm_count=74, key_tile=128)
    cut = {tuple(r[:3]): r[5] for r in plan.items.tolist()}
    assert all(n > 1 for (seg, _, _), n in cut.items() if seg == 0) and all(n == 1 for (seg, _, _), n in cut.items() if seg > 0)
    out, want, used = run_attention(torch.bfloat16, 12, 2, 128, 16, segs, None, tile=tile, plan_kw=dict(sm_count=74, key_tile=128))
    assert used.n_items == plan.n_items and used.n_slots == plan.n_slots > 0
    assert not torch.isnan(out).any()
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))
    assert ops.read_status() == 0


def test_attention_tensor_core_kernel_finds_a_far_key():
    """One key among two thousand carries the whole weight: scale one query and that key so that its
    score stands out; the output must be that key's value row."""
    torch.manual_seed(3)
    Hq, Hkv, D, P, n = 6, 1, 128, 16, 2048
    segs = [(n, n)]
    G = Hq // Hkv
    pages = n // P + 1
    ks = torch.randn(pages, Hkv, P, D).mul(0.1)
    vs = torch.randn(pages, Hkv, P, D)
    q = torch.randn(n, Hq, D).mul(0.1)
    far, tok = 37, 1900
    direction = torch.randn(D)
    direction = direction / direction.norm()
    ks[1 + far // P, 0, far % P] = direction * 30
    q[tok, :] = direction * 30
    bt = torch.arange(1, pages, dtype=torch.int32).view(1, -1).to(DEV)
    seg = torch.tensor([[0, n, n, 0]], dtype=torch.int32, device=DEV)
    plan = build_plan(segs, G, 128, None, Hkv)
    items = torch.from_numpy(plan.items).to(DEV)
    q, ks, vs = q.to(torch.bfloat16).to(DEV), ks.to(torch.bfloat16).to(DEV), vs.to(torch.bfloat16).to(DEV)
    out = torch.empty_like(q)
    po = pm = None
    if plan.n_slots:  # one request alone on the GPU: its tiles are split along the keys
        po = torch.empty(plan.n_slots, Hkv, 128, D, dtype=torch.float32, device=DEV)
        pm = torch.empty(plan.n_slots, Hkv, 128, 2, dtype=torch.float32, device=DEV)
    ops.paged_attention(q, ks, vs, bt, seg, 1, items, plan.n_items, po, pm, out, 128, D ** -0.5, None)
    want = vs[1 + far // P, 0, far % P].float()
    for h in range(Hq):
        torch.testing.assert_close(out[tok, h].float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("fixed", [None, 5])
def test_attention_split_keys(dtype, fixed):
    segs = [(1, 1000), (1, 3), (2, 517), (1, 64)]
    out, want, plan = run_attention(dtype, 12, 2, 64, 16, segs, None, fixed_splits=fixed, force_split=True)
    assert plan.n_slots > 0
    assert not torch.isnan(out).any()
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))


@pytest.mark.parametrize("Hq,Hkv,D,P", [(12, 2, 128, 16), (7, 1, 48, 4), (16, 1, 64, 8), (3, 3, 16, 1), (8, 4, 256, 32),
                                        (48, 8, 128, 16)])
@pytest.mark.parametrize("fixed", [None, 1, 4, 16])
@pytest.mark.parametrize("window", [None, 50])
def test_attention_decode_tiles(Hq, Hkv, D, P, fixed, window):
    """Steps of single decoded tokens use 16-row tiles in bfloat16 (keys split between the warps)."""
    segs = [(1, 1), (1, 130), (1, 17), (1, 700), (1, 64), (1, 65), (1, 1999), (1, 63)]
    out, want, plan = run_attention(torch.bfloat16, Hq, Hkv, D, P, segs, window, fixed_splits=fixed, tile=16,
                                    force_split=fixed is None)
    assert not torch.isnan(out.float()).any()
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))


@pytest.mark.parametrize("Hq,Hkv,P", [(12, 2, 16), (48, 8, 16), (5, 5, 32), (7, 1, 64), (16, 1, 16), (3, 1, 48), (10, 2, 16)])
@pytest.mark.parametrize("fixed", [None, 1, 4, 16])
def test_attention_tensor_core_decode_kernel(Hq, Hkv, P, fixed):
    """The tcgen05 kernel in its form for tiles of at most 16 rows (one softmax warp, head size 128) on
    single tokens and short portions: lengths on and off the edges of its 128-key tiles and 16-key
    boxes, whole, in fixed numbers of pieces (some of them empty) and in forced pieces; every unwritten
    cache slot holds NaN."""
    G = Hq // Hkv
    assert ops.attention_tc_few_fits(128, P, G)
    assert not ops.attention_tc_few_fits(64, P, G) and not ops.attention_tc_few_fits(128, 8, 1)
    assert not ops.attention_tc_few_fits(128, 16, 17)
    segs = [(1, 1), (1, 130), (1, 17), (1, 700), (1, 128), (1, 129), (1, 1999), (1, 127), (1, 256), (1, 1024)]
    if fixed is None:  # portions of a few tokens beside them: several tokens to a tile, or tiles of its own
        segs += [(2, 64), (3, 300), (5, 5), (4, 1000)]
    out, want, plan = run_attention(torch.bfloat16, Hq, Hkv, 128, P, segs, None, fixed_splits=fixed,
                                    tile=16, force_split=fixed is None, few_rows=True)
    assert fixed == 1 or plan.n_slots > 0
    assert not torch.isnan(out.float()).any()
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))
    assert ops.read_status() == 0
    names = list(ops.variant_counts())
    assert any("at most 16 rows" in n for n in names), names


def test_attention_tensor_core_decode_kernel_many_rounds():
    """More pieces than SMs, so that every CTA works through several: the roles run on into the next
    piece; twice in a row, so that the arrival counters of the first launch serve the second."""
    segs = [(1, 300 + 37 * i) for i in range(48)]
    for _ in range(2):
        out, want, plan = run_attention(torch.bfloat16, 48, 8, 128, 16, segs, None, fixed_splits=2, tile=16,
                                        few_rows=True)
        assert plan.n_items * 8 > 2 * 148
        assert not torch.isnan(out.float()).any()
        torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))
    assert ops.read_status() == 0


def test_attention_tensor_core_decode_kernel_finds_a_far_key():
    """One key among four thousand carries the whole weight, in a tile that is split along the keys: the
    running maximum moves there, the accumulator is rescaled, and the merge weighs the pieces."""
    torch.manual_seed(5)
    Hq, Hkv, D, P, n = 12, 2, 128, 16, 4096
    G = Hq // Hkv
    pages = n // P + 1
    for far in (37, 2100, 4095):
        ks = torch.randn(pages, Hkv, P, D).mul(0.1)
        vs = torch.randn(pages, Hkv, P, D)
        q = torch.randn(1, Hq, D).mul(0.1)
        direction = torch.randn(D)
        direction = direction / direction.norm()
        ks[1 + far // P, :, far % P] = direction * 30
        q[0, :] = direction * 30
        bt = torch.arange(1, pages, dtype=torch.int32).view(1, -1).to(DEV)
        seg = torch.tensor([[0, 1, n, 0]], dtype=torch.int32, device=DEV)
        rows = 16
        plan = build_plan([(1, n)], G, rows, None, Hkv, fixed_splits=4, key_tile=128)
        items = torch.from_numpy(plan.items).to(DEV)
        qd, kd, vd = q.to(torch.bfloat16).to(DEV), ks.to(torch.bfloat16).to(DEV), vs.to(torch.bfloat16).to(DEV)
        out = torch.empty_like(qd)
        po = torch.empty(plan.n_slots, Hkv, rows, D, dtype=torch.float32, device=DEV)
        pm = torch.empty(plan.n_slots, Hkv, rows, 2, dtype=torch.float32, device=DEV)
        ops.paged_attention(qd, kd, vd, bt, seg, 1, items, plan.n_items, po, pm, out, rows, D ** -0.5, None,
                            few_rows=True)
        for h in range(Hq):
            want = vd[1 + far // P, h // G, far % P].float()
            torch.testing.assert_close(out[0, h].float(), want, rtol=2e-2, atol=2e-2)
    assert ops.read_status() == 0


def sparse_problem(dtype, Hq, Hkv, D, P, segs, block, seed=0):
    """Paged keys, values and index keys of a few requests (NaN in every unwritten slot)."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-kv // P) for _, kv in segs) + 2
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(len(segs), max(-(-kv // P) for _, kv in segs), dtype=torch.int32)
    ks = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype)
    vs = torch.full((n_pages, Hkv, P, D), float("nan"), dtype=dtype)
    iks = torch.full((n_pages, 1, P, D), float("nan"), dtype=dtype)
    info, q0 = [], 0
    for row, (q_len, kv_len) in enumerate(segs):
        for b in range(-(-kv_len // P)):
            page = perm.pop()
            bt[row, b] = page
            n = min(P, kv_len - b * P)
            ks[page, :, :n] = torch.randn(Hkv, n, D, generator=g).to(dtype)
            vs[page, :, :n] = torch.randn(Hkv, n, D, generator=g).to(dtype)
            iks[page, :, :n] = torch.randn(1, n, D, generator=g).to(dtype)
        info.append([q0, q_len, kv_len, row])
        q0 += q_len
    q = torch.randn(q0, Hq, D, generator=g).to(dtype)
    iq = torch.randn(q0, Hkv, D, generator=g).to(dtype)
    seg = torch.tensor(info, dtype=torch.int32)
    return [t.to(DEV) for t in (q, iq, ks, vs, iks, bt, seg)], q0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,P,block,topk,local,init", [(4, 2, 16, 4, 8, 3, 1, 0), (12, 2, 128, 16, 128, 4, 1, 0),
                                                               (6, 3, 32, 8, 16, 5, 2, 1), (7, 1, 48, 4, 8, 2, 1, 0)])
def test_block_sparse_selection_and_attention(dtype, Hq, Hkv, D, P, block, topk, local, init):
    segs = [(1, 1), (1, 9 * block + 3), (5, 5), (9, 4 * block + 2), (1, block), (2, block + 1)]
    (q, iq, ks, vs, iks, bt, seg), T = sparse_problem(dtype, Hq, Hkv, D, P, segs, block)
    max_blocks = max(kv for _, kv in segs) // block + 1
    sel = torch.full((T, Hkv, topk), -7, dtype=torch.int32, device=DEV)
    want_sel = torch.full_like(sel, -7)
    ops.sparse_select(iq, iks, bt, seg, len(segs), block, local, init, max_blocks, sel)
    ref.sparse_select(iq, iks, bt, seg, len(segs), block, local, init, max_blocks, want_sel)
    assert torch.equal(sel, want_sel)
    # the local block is always there, the list ascends, and short sequences take every block
    assert (sel[0, :, 0] == 0).all() and (sel[0, :, 1:] == -1).all()
    plan = build_plan(segs, Hq // Hkv, 16, None, Hkv, sm_count=4096, min_split_keys=32, sparse=(block, topk))
    items = torch.from_numpy(plan.items).to(DEV)
    po = pm = None
    if plan.n_slots:
        po = torch.full((plan.n_slots, Hkv, 16, D), float("nan"), dtype=torch.float32, device=DEV)
        pm = torch.full((plan.n_slots, Hkv, 16, 2), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full((T, Hq, D), float("nan"), dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    ops.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, po, pm, out, 16, D ** -0.5, None,
                        sel=sel, block_size=block)
    ref.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, None, None, want, 16, D ** -0.5, None,
                        sel=sel, block_size=block)
    assert not torch.isnan(out.float()).any()
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    # while nothing is dropped the result is dense attention
    dense = torch.empty_like(out)
    ref.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, None, None, dense, 16, D ** -0.5, None)
    short = [i for i, (ql, kv) in enumerate(segs) if kv <= topk * block]
    for i in short:
        q0, ql = int(seg[i, 0]), int(seg[i, 1])
        torch.testing.assert_close(out[q0:q0 + ql].float(), dense[q0:q0 + ql].float(), **attn_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 64, 100])
def test_attention_window(dtype, window):
    segs = [(1, 150), (40, 40), (9, 120)]
    out, want, _ = run_attention(dtype, 6, 3, 32, 8, segs, window)
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_far_key_stands_out(dtype):
    """One key far back gets a large score: every query must put almost all its weight there,
    so a kernel that drops or misplaces a far page cannot pass."""
    Hq, Hkv, D, P = 4, 2, 64, 16
    segs = [(1, 700), (3, 515)]
    G = Hq // Hkv
    tile = 64 if dtype == torch.bfloat16 else 16
    out, want, _ = run_attention(dtype, Hq, Hkv, D, P, segs, None, force_split=True, seed=5)
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(dtype))
    # now make position 3 of segment 0 dominate and check the output equals its value row
    g = torch.Generator().manual_seed(9)
    kv = 700
    ks = torch.randn(50, Hkv, P, D, generator=g).to(dtype).to(DEV) * 0.1
    vs = torch.randn(50, Hkv, P, D, generator=g).to(dtype).to(DEV)
    bt = torch.arange(1, 46, dtype=torch.int32).view(1, -1).to(DEV)
    q = torch.randn(1, Hq, D, generator=g).to(dtype).to(DEV)
    for h in range(Hkv):
        ks[1, h, 3] = (q[0, h * G].float() * 8).to(dtype)  # page 1 holds positions 0..15
    seg = torch.tensor([[0, 1, kv, 0]], dtype=torch.int32, device=DEV)
    plan = build_plan([(1, kv)], G, tile, None, Hkv, sm_count=4096, min_split_keys=32)
    items = torch.from_numpy(plan.items).to(DEV)
    po = torch.empty(max(plan.n_slots, 1), Hkv, tile, D, dtype=torch.float32, device=DEV)
    pm = torch.empty(max(plan.n_slots, 1), Hkv, tile, 2, dtype=torch.float32, device=DEV)
    out = torch.empty(1, Hq, D, dtype=dtype, device=DEV)
    ops.paged_attention(q, ks, vs, bt, seg, 1, items, plan.n_items, po, pm, out, tile, D ** -0.5, None)
    for h in range(Hkv):
        torch.testing.assert_close(out[0, h * G].float(), vs[1, h, 3].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(8192, 3072), (3072, 6144), (100, 72), (7, 8), (1000, 520), (33, 24576)])
def test_few_token_product_streams_the_weights(T, N, K, monkeypatch):
    """``ops.linear`` sends products of few bfloat16 rows to this library's own kernel (by default of one row;
    here of up to four, which the kernel takes as well); other sizes go to the library."""
    x = rnd(T, K, dtype=torch.bfloat16)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05)
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    name = "few-token product: weights streamed by warps"
    before = ops.variant_counts().get(name, 0)
    ops.linear(x, w, out)
    assert ops.variant_counts().get(name, 0) - before == (1 if T <= ops.SMALL_LINEAR_MAX_TOKENS else 0)
    monkeypatch.setattr(ops, "SMALL_LINEAR_MAX_TOKENS", 4)
    before = ops.variant_counts().get(name, 0)
    ops.linear(x, w, out)
    took = ops.variant_counts().get(name, 0) - before
    assert took == (1 if ops.small_linear_fits(T, N, K) else 0)
    if not ops.small_linear_fits(T, N, K):  # three and four rows of 24,576 do not fit its shared memory: the library's
        assert K == 24576 and T > 2
        return
    want = x.float() @ w.float().T
    # (sums of thousands of terms near zero: the bound is on the size of the row's results, not of each)
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-3 * float(want.abs().mean() + 1))
    assert not ops.small_linear_fits(5, N, K) and not ops.small_linear_fits(1, N, 12)


@pytest.mark.parametrize("act", ["silu", "swigluoai"])
@pytest.mark.parametrize("T,k,E,H,I", [(1, 8, 256, 3072, 1536), (4, 8, 256, 3072, 1536), (3, 2, 5, 64, 40), (2, 3, 7, 520, 8),
                                       (4, 4, 4, 48, 104)])
def test_few_token_expert_products(T, k, E, H, I, act):
    """The routed few-token kernels against the plain statement, routes in token order, several routes to
    one expert, and a route that names no expert (its rows are zero)."""
    g = torch.Generator().manual_seed(T * 100 + E)
    h = rnd(T, H, dtype=torch.bfloat16)
    w1 = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.05)
    w2 = rnd(E, H, I, dtype=torch.bfloat16, scale=0.05)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] if k <= E else torch.randint(0, E, (k,), generator=g)
                       for _ in range(T)]).to(torch.int32)
    if T > 1:
        ids[1, 0] = ids[0, 0]  # two tokens at one expert
    if T > 2:
        ids[2, k - 1] = -1
    ids = ids.to(DEV)
    wts = torch.rand(T, k, device=DEV) + 0.5
    assert ops.moe_small_fits(T, H, I, k) and not ops.moe_small_fits(5, H, I, k) and not ops.moe_small_fits(1, H + 4, I, k)
    a = torch.full((T * k, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    y = torch.full((T * k, H), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.moe_small_gate_up(h, ids, w1, act, 1.702, 7.0, a)
    a_in = rnd(T * k, I, dtype=torch.bfloat16, seed=5)
    ops.moe_small_down(a_in, ids, wts, w2, y)
    want_a, want_y = torch.zeros(T * k, I, device=DEV), torch.zeros(T * k, H, device=DEV)
    for r in range(T * k):
        e = int(ids.view(-1)[r])
        if e < 0:
            continue
        gu = (h[r // k].float() @ w1[e].float().T).to(torch.bfloat16).float()
        want_a[r] = ref.gated(gu[:I], gu[I:], act, 1.702, 7.0) if hasattr(ref, "gated") else _gated(gu[:I], gu[I:], act)
        want_y[r] = (a_in[r].float() @ w2[e].float().T) * wts.view(-1)[r]
    assert not torch.isnan(a.float()).any() and not torch.isnan(y.float()).any()
    # (gate and up are rounded to bfloat16 before the activation: a last-bit difference there is amplified by (u + 1))
    torch.testing.assert_close(a.float(), want_a, rtol=3e-2, atol=4e-3)
    torch.testing.assert_close(y.float(), want_y, **tol(torch.bfloat16))


def _gated(g, u, act, alpha=1.702, limit=7.0):
    if act == "silu":
        return g * torch.sigmoid(g) * u
    g = g.clamp(max=limit)
    u = u.clamp(-limit, limit)
    return g * torch.sigmoid(alpha * g) * (u + 1)


# ---------------------------------------------------------------------------------------------
# Negative controls: the tolerances above must be able to fail.  Each bfloat16 kernel's output is
# compared, with the same bound as its test, against a reference that was given a slightly wrong
# problem (one key of one request missing; one row counted to the neighbouring expert): the
# comparison has to raise.
@pytest.mark.parametrize("tile", [16, 64, 128, 256])
def test_attention_bound_notices_one_missing_key(tile):
    segs = [(40, 40), (1, 36)] if tile != 16 else [(1, 40), (1, 36)]
    Hq, Hkv, D, P = 12, 2, 128, 16
    out, want, _ = run_attention(torch.bfloat16, Hq, Hkv, D, P, segs, None, tile=tile)
    torch.testing.assert_close(out.float(), want.float(), **attn_tol(torch.bfloat16))
    # the same problem, but the reference does not see key 20 of the first request (its score is made
    # hopeless by turning the key against every query, its value is zeroed)
    out2, wrong, _ = run_attention(torch.bfloat16, Hq, Hkv, D, P, segs, None, tile=tile, spoil_reference=(0, 20))
    assert torch.equal(out, out2)
    with pytest.raises(AssertionError):
        torch.testing.assert_close(out.float(), wrong.float(), **attn_tol(torch.bfloat16))
    # (a small fault, not a gross one: the rows of the other request are untouched, and in the spoilt
    # request the typical output moves by a few hundredths)
    diff = (want.float() - wrong.float()).abs()
    n_first = 40 if tile != 16 else 1
    assert diff[n_first:].max() == 0 and diff[:n_first].median() < 0.05


@pytest.mark.parametrize("tc", [True, False])
def test_expert_product_bounds_notice_one_row_at_the_wrong_expert(tc):
    E, H, I = 8, 256, 128
    counts = [5, 0, 9, 3, 40, 1, 0, 6]
    R = sum(counts)
    off = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32, device=DEV)
    wrong_off = off.clone()
    wrong_off[3] += 1  # the first row of expert 3 is counted to expert 2
    x = rnd(R, H, dtype=torch.bfloat16)
    w1 = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.1)
    w2 = rnd(E, H, I, dtype=torch.bfloat16, scale=0.1)
    routes = torch.randperm(R).to(torch.int32).to(DEV)
    wts = torch.rand(R, device=DEV) + 0.5
    ops.set_moe_tensor_cores(tc)
    try:
        a, y = torch.empty(R, I, dtype=torch.bfloat16, device=DEV), torch.empty(R, H, dtype=torch.bfloat16, device=DEV)
        ops.moe_gemm1_act(x, w1, off, "silu", 1.702, 7.0, a)
        a_in = rnd(R, I, dtype=torch.bfloat16, seed=3)
        ops.moe_gemm2(a_in, w2, off, routes, wts, y)
    finally:
        ops.set_moe_tensor_cores(True)
    for offsets, ok in ((off, True), (wrong_off, False)):
        a2, y2 = torch.empty_like(a), torch.empty_like(y)
        ref.moe_gemm1_act(x, w1, offsets, "silu", 1.702, 7.0, a2)
        ref.moe_gemm2(a_in, w2, offsets, routes, wts, y2)
        for got, want in ((a, a2), (y, y2)):
            if ok:
                torch.testing.assert_close(got.float(), want.float(), **tol(torch.bfloat16))
            else:
                with pytest.raises(AssertionError):
                    torch.testing.assert_close(got.float(), want.float(), **tol(torch.bfloat16))
                assert ((got.float() - want.float()).abs().amax(-1) > 0.1).sum() == 1  # exactly that row


@pytest.mark.parametrize("scoring,bias", [("sigmoid", True), ("sigmoid", False), ("softmax", False), ("softmax", True)])
@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (37, 256, 8), (5, 6, 3), (64, 100, 100), (3, 1, 1)])
def test_router_topk(scoring, bias, T, E, k):
    logits = rnd(T, E, scale=2.0)
    logits[0, : min(E, 4)] = 0.5  # ties: the lower index must win
    b = rnd(E, scale=0.01, seed=7) if bias else None
    ids = torch.empty(T, k, dtype=torch.int32, device=DEV)
    w = torch.empty(T, k, dtype=torch.float32, device=DEV)
    ids2, w2 = torch.empty_like(ids), torch.empty_like(w)
    ops.router_topk(logits, b, k, scoring, 2.0, ids, w)
    ref.router_topk(logits, b, k, scoring, 2.0, ids2, w2)
    assert torch.equal(ids, ids2)
    torch.testing.assert_close(w, w2, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("T,N,K,dtype", [(8, 96, 192, torch.bfloat16), (1, 64, 64, torch.bfloat16), (8, 192, 96, torch.bfloat16),
                                         (20, 96, 192, torch.bfloat16), (5, 96, 192, torch.float32)])
def test_linear_pads_few_rows_inside_its_buffers(T, N, K, dtype):
    """Few bfloat16 rows against a long weight are multiplied as 16 rows of the same buffers: the rows
    past T may hold anything (NaN here) and what lies behind the output rows is only overwritten where
    the buffer has room; without room the product is taken as it is."""
    w = rnd(N, K, dtype=dtype, scale=K ** -0.5, seed=3)
    xbuf = torch.full((64, K), float("nan"), dtype=dtype, device=DEV)
    obuf = torch.zeros(64, N, dtype=dtype, device=DEV)
    xbuf[:T] = rnd(T, K, dtype=dtype)
    ops.linear(xbuf[:T], w, obuf[:T])
    want = xbuf[:T].float() @ w.float().T
    torch.testing.assert_close(obuf[:T].float(), want, **tol(dtype))
    assert not torch.isnan(obuf[:T]).any() and (obuf[max(16, T):] == 0).all()
    tight_x, tight_o = xbuf[:T].clone(), torch.empty(T, N, dtype=dtype, device=DEV)  # no room to pad
    ops.linear(tight_x, w, tight_o)
    torch.testing.assert_close(tight_o.float(), want, **tol(dtype))


@pytest.mark.parametrize("E,H,I,R", [(12, 1664, 1536, 4000), (24, 640, 1600, 2500), (100, 256, 128, 40000),
                                     (40, 1152, 1088, 1900)])
def test_moe_products_by_pairs_of_ctas_equal_single_ctas(E, H, I, R):
    """Token tiles of 256 (in the last case 128) rows, hundreds of tiles: the expert products run on pairs of CTAs
    (cta_group::2: 256 weight rows a tile, each CTA loads half of the tokens).  Every output element is the same sum in the
    same order as in the one-CTA form, so the results are equal bit for bit; experts with a few rows, with
    exactly 256, with 257 and with none are among them, and widths of an odd number of feature tiles."""
    g = torch.Generator().manual_seed(E)
    ids = torch.randint(0, E, (R,), generator=g)
    ids[: R // 3] = 3        # a crowded expert: several token tiles
    ids[ids == 5] = 6        # an expert without rows
    ids[R // 3: R // 3 + 256] = 7
    ids[ids == 8] = 9
    ids[R // 3 + 256: R // 3 + 256 + 257] = 8
    counts = torch.bincount(ids, minlength=E)
    off = torch.tensor([0] + counts.cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    x = rnd(R, H, dtype=torch.bfloat16)
    w1 = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.05)
    w2 = rnd(E, H, I, dtype=torch.bfloat16, scale=0.05)
    a_in = rnd(R, I, dtype=torch.bfloat16, seed=9)
    routes = torch.randperm(R).to(torch.int32).to(DEV)
    wts = torch.rand(R, device=DEV) + 0.5
    outs = []
    for pairs in (True, False):
        ops.set_moe_pairs(pairs)
        ops.variant_counts(reset=True)
        a = torch.full((R, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        y = torch.full((R, H), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.moe_gemm1_act(x, w1, off, "swigluoai", 1.702, 7.0, a)
        ops.moe_gemm2(a_in, w2, off, routes, wts, y)
        ran = ops.variant_counts()
        tile = 128 if R // E < 80 else 256  # (the last case has 128-token tiles)
        assert bool(ran.get(f"expert gate/up product: tcgen05, {tile} tokens a tile, pairs of CTAs")) == pairs, ran
        if (H + 127) // 128 * E * (256 // tile) > 296:  # (enough tiles of the down product for the deep form)
            assert bool(ran.get(f"expert down product: tcgen05, {tile} tokens a tile, pairs of CTAs")) == pairs, ran
        outs.append((a, y))
    ops.set_moe_pairs(True)
    assert ops.read_status() == 0
    assert not torch.isnan(outs[0][0]).any() and not torch.isnan(outs[0][1]).any()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("scoring,bias", [("sigmoid", True), ("softmax", False)])
@pytest.mark.parametrize("T,H,E,k", [(1, 64, 8, 2), (8, 3072, 256, 8), (13, 100, 7, 3), (32, 520, 33, 5), (9, 36, 301, 1),
                                     (1, 3072, 256, 8), (3, 64, 256, 8), (5, 128, 200, 6), (6, 96, 64, 64), (12, 256, 100, 4),
                                     (7, 64, 40, 40)])
def test_moe_route_in_one_launch(scoring, bias, T, H, E, k):
    """Logits, choice and sort in one launch against the three separate statements; run several
    times so that the arrival counter is seen to come back to zero."""
    assert ops.moe_route_fits(T, H, E, k) and not ops.moe_route_fits(33, H, E, k) and not ops.moe_route_fits(T, H + 2, E, k)
    x = rnd(T, H, scale=1.0)
    w = rnd(E, H, scale=H ** -0.5, seed=5)
    if T > 2:
        x[2] = x[1]  # equal tokens make equal choices, whatever their place in the batch
    b = rnd(E, scale=0.01, seed=7) if bias else None
    ref_logits = (x.double() @ w.double().T).float()
    ids2 = torch.empty(T, k, dtype=torch.int32, device=DEV)
    w2 = torch.empty(T, k, dtype=torch.float32, device=DEV)
    for rep in range(3):
        logits = torch.full((T, E), float("nan"), device=DEV)
        ids = torch.full((T, k), -1, dtype=torch.int32, device=DEV)
        wts = torch.empty(T, k, dtype=torch.float32, device=DEV)
        counts = torch.empty(E, dtype=torch.int32, device=DEV)
        off = torch.empty(E + 1, dtype=torch.int32, device=DEV)
        routes = torch.empty(T * k, dtype=torch.int32, device=DEV)
        pos = torch.empty(T * k, dtype=torch.int32, device=DEV)
        ops.moe_route(x, w, b, k, scoring, 2.5, logits, ids, wts, counts, off, routes, pos)
        torch.testing.assert_close(logits, ref_logits, rtol=1e-5, atol=1e-5)
        ref.router_topk(logits, b, k, scoring, 2.5, ids2, w2)  # the choice, given the kernel's own logits
        assert torch.equal(ids, ids2)
        torch.testing.assert_close(wts, w2, rtol=1e-5, atol=1e-7)
        c2, o2, r2, p2 = torch.empty_like(counts), torch.empty_like(off), torch.empty_like(routes), torch.empty_like(pos)
        ref.moe_permute(ids, E, c2, o2, r2, p2)
        for got, want in ((counts, c2), (off, o2), (routes, r2), (pos, p2)):
            assert torch.equal(got, want)
        if T > 2:
            assert torch.equal(logits[1], logits[2]) and torch.equal(ids[1], ids[2])
    alone = torch.empty(1, E, device=DEV)
    ops.moe_route(x[-1:].contiguous(), w, b, k, scoring, 2.5, alone, ids[:1].clone(), wts[:1].clone(), counts, off,
                  routes[:k].clone(), pos[:k].clone())
    assert torch.equal(alone[0], logits[-1]), "a token's logits must not depend on the batch"


@pytest.mark.parametrize("T,k,E", [(1, 2, 8), (50, 4, 16), (300, 8, 256), (7, 3, 6), (2, 1, 40), (2048, 8, 256),
                                   (3001, 3, 7), (700, 5, 1100)])
def test_moe_permute_gather_combine(T, k, E):
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    if T > 4:
        ids[:4] = ids[0]  # several tokens to the same experts
    outs = []
    for fn in (ops.moe_permute, ref.moe_permute):
        counts = torch.empty(E, dtype=torch.int32, device=DEV)
        off = torch.empty(E + 1, dtype=torch.int32, device=DEV)
        routes = torch.empty(T * k, dtype=torch.int32, device=DEV)
        pos = torch.empty(T * k, dtype=torch.int32, device=DEV)
        fn(ids, E, counts, off, routes, pos)
        outs.append((counts, off, routes, pos))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    counts, off, routes, pos = outs[0]
    for dtype in DTYPES:
        h = rnd(T, 56, dtype=dtype)
        x, x2 = torch.empty(T * k, 56, dtype=dtype, device=DEV), torch.empty(T * k, 56, dtype=dtype, device=DEV)
        ops.moe_gather(h, routes, k, x)
        ref.moe_gather(h, routes, k, x2)
        assert torch.equal(x, x2)
        y = rnd(T * k, 56, dtype=dtype, seed=3)
        sh = rnd(T, 56, dtype=dtype, seed=4)
        for shared in (None, sh):
            o, o2 = torch.empty(T, 56, dtype=dtype, device=DEV), torch.empty(T, 56, dtype=dtype, device=DEV)
            ops.moe_combine(y, pos, T, k, shared, o)
            ref.moe_combine(y, pos, T, k, shared, o2)
            torch.testing.assert_close(o.float(), o2.float(), **tol(dtype))


@pytest.mark.parametrize("T,k,E", [(9, 4, 16), (2048, 8, 256), (3001, 3, 7)])
def test_moe_permute_with_routes_to_no_expert(T, k, E):
    """Ids outside [0, E) get no row: their position is -1 and the rows nobody claimed hold -1
    (both the short-step and the long-step kernels)."""
    g = torch.Generator().manual_seed(T)
    ids = torch.randint(0, E, (T, k), generator=g).to(torch.int32)
    ids[T // 2, 0] = -1
    ids[T - 1, k - 1] = E
    ids[0, 0] = E + 5
    flat = ids.reshape(-1)
    valid = (flat >= 0) & (flat < E)
    order = torch.argsort(torch.where(valid, flat, torch.full_like(flat, E)), stable=True)
    n_valid = int(valid.sum())
    want_routes = torch.cat([order[:n_valid].to(torch.int32), torch.full((flat.numel() - n_valid,), -1, dtype=torch.int32)])
    want_pos = torch.full((flat.numel(),), -1, dtype=torch.int32)
    want_pos[order[:n_valid]] = torch.arange(n_valid, dtype=torch.int32)
    want_counts = torch.bincount(flat[valid].long(), minlength=E).to(torch.int32)
    counts = torch.empty(E, dtype=torch.int32, device=DEV)
    off = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    routes = torch.empty(T * k, dtype=torch.int32, device=DEV)
    pos = torch.empty(T * k, dtype=torch.int32, device=DEV)
    ops.moe_permute(ids.to(DEV), E, counts, off, routes, pos)
    assert torch.equal(counts.cpu(), want_counts)
    assert torch.equal(off.cpu()[1:], torch.cumsum(want_counts, 0).to(torch.int32)) and off[0].item() == 0
    assert torch.equal(routes.cpu(), want_routes)
    assert torch.equal(pos.cpu(), want_pos)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,H,I,counts", [
    (6, 112, 40, [0, 5, 1, 0, 33, 2]), (4, 96, 48, [64, 0, 0, 1]), (8, 64, 32, [3] * 8),
    (3, 200, 72, [130, 1, 70]), (5, 128, 256, [0, 0, 0, 0, 9])])
@pytest.mark.parametrize("act", ["silu", "swigluoai"])
def test_moe_grouped_gemms(dtype, E, H, I, counts, act):
    R = sum(counts)
    off = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32, device=DEV)
    x = rnd(R, H, dtype=dtype)
    w1 = rnd(E, 2 * I, H, dtype=dtype, scale=0.1)
    w2 = rnd(E, H, I, dtype=dtype, scale=0.1)
    a, a2 = torch.empty(R, I, dtype=dtype, device=DEV), torch.empty(R, I, dtype=dtype, device=DEV)
    ops.moe_gemm1_act(x, w1, off, act, 1.702, 7.0, a)
    ref.moe_gemm1_act(x, w1, off, act, 1.702, 7.0, a2)
    torch.testing.assert_close(a.float(), a2.float(), **tol(dtype))
    routes = torch.randperm(R).to(torch.int32).to(DEV)
    wts = torch.rand(R, device=DEV) + 0.5
    y, y2 = torch.empty(R, H, dtype=dtype, device=DEV), torch.empty(R, H, dtype=dtype, device=DEV)
    ops.moe_gemm2(a2, w2, off, routes, wts, y)
    ref.moe_gemm2(a2, w2, off, routes, wts, y2)
    torch.testing.assert_close(y.float(), y2.float(), **tol(dtype))


@pytest.mark.parametrize("E,H,I,R,k", [(256, 3072, 1536, 64, 8), (256, 3072, 1536, 2048, 8), (32, 512, 256, 700, 4),
                                       (8, 64, 32, 9, 2), (16, 1024, 1000, 300, 2),
                                       (12, 1664, 1536, 4000, 2), (24, 640, 1600, 2500, 2), (40, 1152, 1088, 1900, 2)])
def test_moe_tensor_core_gemms_match_cuda_core_gemms(E, H, I, R, k):
    """The tcgen05 kernels against the CUDA-core kernels on the same inputs (and, for the small
    cases, against the plain reference), at decode-like and prefill-like row counts, including
    experts without rows and experts with more rows than one token tile.  The last three have hundreds
    of rows per expert and hundreds of tiles: token tiles of 256 and 128 rows in the deep-pipeline form,
    where a CTA multiplies two feature tiles with each token tile (widths of 13 x 128, 25 x 64, 17 x 64
    and 9 x 128 features: an odd number of feature tiles, so the last pair has one)."""
    g = torch.Generator().manual_seed(R)
    ids = torch.randint(0, E, (R,), generator=g)
    if R > 100:
        ids[: R // 3] = 3  # one crowded expert: several token tiles
    counts = torch.bincount(ids, minlength=E)
    off = torch.tensor([0] + counts.cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    x = rnd(R, H, dtype=torch.bfloat16)
    w1 = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.05)
    w2 = rnd(E, H, I, dtype=torch.bfloat16, scale=0.05)
    routes = torch.randperm(R).to(torch.int32).to(DEV)
    wts = torch.rand(R, device=DEV) + 0.5
    outs = []
    a_in = rnd(R, I, dtype=torch.bfloat16, seed=9)  # both kernels get the same input for the second product
    for tc in (True, False):
        ops.set_moe_tensor_cores(tc)
        a = torch.full((R, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        y = torch.full((R, H), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.moe_gemm1_act(x, w1, off, "swigluoai", 1.702, 7.0, a)
        ops.moe_gemm2(a_in, w2, off, routes, wts, y)
        outs.append((a, y))
    ops.set_moe_tensor_cores(True)
    assert ops.read_status() == 0
    (a_tc, y_tc), (a_cc, y_cc) = outs
    assert not torch.isnan(a_tc).any() and not torch.isnan(y_tc).any()
    # second product: same inputs, the kernels differ only in the order of the 32-bit sums
    torch.testing.assert_close(y_tc.float(), y_cc.float(), **tol(torch.bfloat16))
    # first product: gate and up are rounded to bfloat16 before the activation, and (u + 1) can
    # cancel, so a one-ulp difference in u is amplified.  Both kernels are held to the bound that
    # rounding g and u (2^-8 relative each) and the result can cause around the 32-bit value.
    g32 = torch.empty(R, I, device=DEV)
    u32 = torch.empty(R, I, device=DEV)
    offs = off.tolist()
    for e in range(E):
        lo, hi = offs[e], offs[e + 1]
        if hi > lo:
            gu = x[lo:hi].float() @ w1[e].float().T
            g32[lo:hi], u32[lo:hi] = gu[:, :I], gu[:, I:]
    alpha, limit, eps = 1.702, 7.0, 2.0 ** -8
    gc, uc = g32.clamp(max=limit), u32.clamp(-limit, limit)
    sig = torch.sigmoid(alpha * gc)
    exact = gc * sig * (uc + 1)
    d_g = (sig * (1 + alpha * gc * (1 - sig)) * (uc + 1)).abs()
    d_u = (gc * sig).abs()
    bound = eps * (g32.abs() * d_g + u32.abs() * d_u + exact.abs()) + 1e-3
    for got in (a_tc, a_cc):
        assert ((got.float() - exact).abs() <= bound).all()


@pytest.mark.parametrize("scoring,bias", [("sigmoid", True), ("softmax", False)])
@pytest.mark.parametrize("T,H,E,k", [(300, 3072, 256, 8), (70, 520, 33, 5), (40, 96, 301, 2)])
def test_router_logits_from_three_bfloat16_products(scoring, bias, T, H, E, k):
    """Long bfloat16 steps: the float32 router weights split into three bfloat16 pieces whose sum is the
    weight exactly, three tensor-core products with 32-bit accumulators, and the choice kernel adding the
    pieces.  The products are the exact ones; what differs from the float32 matrix product is the rounding
    of the partial sums (the tensor cores' 32-bit accumulators cut off where the CUDA cores round), so the
    distance to the float64 product is held to 1.5e-6 of sum |x||w| (measured: 6.4e-7 at a width of 3,072
    against 1.2e-7 for the library's float32 product; 1.8e-4 is the bound of a 32-bit sum of that length).
    The choice is the one the reference statement makes from the summed logits."""
    from freetoken_b200.parts.moe import split_in_three

    w = rnd(E, H, scale=H ** -0.5, seed=5)
    w[0, 0] = 1.0 + 2.0 ** -23   # needs all three pieces
    w[1, 1] = -3.0e-30           # tiny
    pieces = split_in_three(w)
    assert pieces is not None and pieces.shape == (3 * E, H) and pieces.dtype == torch.bfloat16
    assert torch.equal((pieces[:E].float() + pieces[E:2 * E].float()) + pieces[2 * E:].float(), w)
    assert split_in_three(torch.full((2, 8), float("inf"), device=DEV)) is None
    x = rnd(T, H, dtype=torch.bfloat16, scale=1.0)
    got3 = torch.mm(x, pieces.t(), out_dtype=torch.float32)
    logits = (got3[:, :E] + got3[:, E:2 * E]) + got3[:, 2 * E:]
    exact = x.double() @ w.double().T
    plain = x.float() @ w.t()
    scale_ = (x.double().abs() @ w.double().abs().T)  # what the rounding errors are relative to
    err_split = ((logits.double() - exact).abs() / scale_).max().item()
    err_plain = ((plain.double() - exact).abs() / scale_).max().item()
    assert err_split < 1.5e-6 and err_split < 16 * err_plain + 1e-7, (err_split, err_plain)
    b = rnd(E, scale=0.01, seed=7) if bias else None
    ids, wts = torch.empty(T, k, dtype=torch.int32, device=DEV), torch.empty(T, k, device=DEV)
    ids2, w2 = torch.empty_like(ids), torch.empty_like(wts)
    ops.router_topk(got3.contiguous(), b, k, scoring, 2.5, ids, wts, n_parts=3)
    ref.router_topk(logits, b, k, scoring, 2.5, ids2, w2)
    assert torch.equal(ids, ids2)
    torch.testing.assert_close(wts, w2, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("E,H,I,T,k", [(256, 3072, 1536, 8, 8), (256, 3072, 1536, 500, 8), (32, 512, 256, 120, 4),
                                       (8, 64, 32, 5, 2), (6, 200, 48, 30, 3), (16, 1000, 112, 120, 2), (4, 128, 64, 1, 4)])
def test_moe_gate_up_product_gathers_its_rows(E, H, I, T, k):
    """The gate/up kernel reading each expert's rows from the tokens in their own order (two warps copy
    them into the swizzled tile) against the same kernel on rows copied into expert order first: the
    same products in the same order, so the results are equal bit for bit (the other tests hold that kernel
    to the references).  Decode-like and prefill-like
    row counts (token tiles of 16 and 32 rows), a crowded expert, widths that end inside a 64-element piece of k."""
    assert ops.moe_gemm1_gather_fits(torch.bfloat16, H, I, E, T * k)
    assert not ops.moe_gemm1_gather_fits(torch.float32, H, I, E, T * k)
    assert not ops.moe_gemm1_gather_fits(torch.bfloat16, H + 4, I, E, T * k)
    assert not ops.moe_gemm1_gather_fits(torch.bfloat16, H, I, E, 100 * E)  # token tiles of more than 32 rows
    g = torch.Generator().manual_seed(T + k)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    if T > 100:
        ids[: T // 2, 0] = 3  # one crowded expert: several token tiles
        ids[: T // 2, 1:] = torch.stack([torch.randperm(E - 4, generator=g)[: k - 1] + 4 for _ in range(T // 2)]).to(torch.int32)
    ids = ids.to(DEV)
    counts = torch.empty(E, dtype=torch.int32, device=DEV)
    off = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    routes = torch.empty(T * k, dtype=torch.int32, device=DEV)
    pos = torch.empty(T * k, dtype=torch.int32, device=DEV)
    ops.moe_permute(ids, E, counts, off, routes, pos)
    h = rnd(T, H, dtype=torch.bfloat16)
    w1 = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.05)
    x = torch.empty(T * k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_gather(h, routes, k, x)
    want = torch.full((T * k, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    got = torch.full((T * k, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.moe_gemm1_act(x, w1, off, "swigluoai", 1.702, 7.0, want)
    for _ in range(2):  # twice: the stages' barriers start from where the launch before left nothing
        got.fill_(float("nan"))
        ops.moe_gemm1_act_gather(h, routes, k, w1, off, "swigluoai", 1.702, 7.0, got)
        assert not torch.isnan(got).any()
        assert torch.equal(got, want)
    assert ops.read_status() == 0
    assert any("gate/up" in n for n in ops.variant_counts())


@pytest.mark.parametrize("V", [256, 331, 50000, 200064, 16390])
def test_sample(V):
    R = 9
    logits = rnd(R, V, scale=3.0)
    logits[0, 7] = logits[0, 3] = logits[0].max() + 1  # tie: index 3 wins
    temp = torch.tensor([0.0, 0.8, 1.0, 0.5, 1.3, 0.0, 1.0, 1.0, 2.0], device=DEV)
    top_k = torch.tensor([0, 0, 5, 0, 40, 0, 1, 0, 3], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.9, 0.7, 1.0, 1.0, 0.3, 0.95], device=DEV)
    for trial in range(6):
        u = torch.rand(R, generator=torch.Generator().manual_seed(trial)).to(DEV)
        out = torch.empty(R, dtype=torch.int32, device=DEV)
        want = torch.empty_like(out)
        ops.sample(logits, temp, top_k, top_p, u, out)
        ref.sample(logits, temp, top_k, top_p, u, want)
        assert out[0].item() == 3
        assert torch.equal(out, want), (trial, out, want)


@pytest.mark.parametrize("R,V", [(70, 9001), (3, 200064), (300, 520)])
def test_sample_greedy_rows_in_chunks(R, V):
    """Rows cut into chunks over several blocks: the argmax with the lowest index on a tie, run twice so
    that the arrival counters are seen to come back to zero."""
    logits = rnd(R, V, scale=2.0)
    top = logits.max() + 1
    logits[1, V - 1] = top
    logits[1, V // 2] = top  # the tie lies in two different chunks
    zeros = torch.zeros(R, device=DEV)
    for _ in range(2):
        out = torch.empty(R, dtype=torch.int32, device=DEV)
        ops.sample(logits, zeros, torch.zeros(R, dtype=torch.int32, device=DEV), torch.ones(R, device=DEV), zeros, out)
        assert torch.equal(out.long(), torch.argmax(logits, dim=-1))
        assert out[1].item() == V // 2


def test_kernels_refuse_what_they_cannot_do():
    from freetoken_b200.errors import KernelError

    q = torch.zeros(1, 2, 24, device=DEV)  # head size 24 is no multiple of 16
    slab = torch.zeros(2, 2, 4, 24, device=DEV)
    with pytest.raises(KernelError):
        ops.paged_attention(q, slab, slab, torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                            torch.zeros(1, 4, dtype=torch.int32, device=DEV), 1,
                            torch.zeros(1, 8, dtype=torch.int32, device=DEV), 1, None, None,
                            torch.zeros_like(q), 16, 1.0, None)
    with pytest.raises(KernelError):  # tensors on the CPU never reach a kernel
        ops.cast(torch.zeros(4), torch.zeros(4, dtype=torch.bfloat16))
