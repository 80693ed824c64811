"""The attention entry point that allocates nothing (freetoken_b200/csrc/no_alloc.h).

Some users of the library cannot call cudaMalloc while a step runs: a host that gave the whole
GPU to its own pools at start-up, a caller that cannot afford the device-wide synchronisation an
allocation implies, or a plain C / ctypes user with no tensor library to make a scratch buffer.
For them ``ftk_paged_attention_static_scratch`` keeps the scratch of split attention tiles in a
fixed array inside the library.  This test calls it through its exported C symbol, twice in a row
with different inputs (the array keeps the first call's contents), and compares each result with
the ordinary entry point, which is given scratch tensors; it also checks that a work list too big
for the array is refused.  The file sorts last so that a run that stops at the first failure has
already run every other test.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from freetoken_b200.engine.attention_plan import build_plan
from freetoken_b200.kernels import library, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def problem(dtype, seed, segs, Hq=12, Hkv=2, D=64, P=16, tile=None):
    g = torch.Generator().manual_seed(seed)
    G = Hq // Hkv
    tile = tile or (64 if dtype == torch.bfloat16 else 16)
    n_pages = sum(-(-kv // P) for _, kv in segs) + 2
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(len(segs), max(-(-kv // P) for _, kv in segs), dtype=torch.int32)
    ks = torch.randn(n_pages, Hkv, P, D, generator=g).to(dtype)
    vs = torch.randn(n_pages, Hkv, P, D, generator=g).to(dtype)
    info, q0 = [], 0
    for row, (q_len, kv_len) in enumerate(segs):
        for b in range(-(-kv_len // P)):
            bt[row, b] = perm.pop()
        info.append([q0, q_len, kv_len, row])
        q0 += q_len
    q = torch.randn(q0, Hq, D, generator=g).to(dtype)
    plan = build_plan(segs, G, tile, None, Hkv, sm_count=4096, min_split_keys=32)
    assert plan.n_slots > 0
    return dict(q=q.to(DEV), ks=ks.to(DEV), vs=vs.to(DEV), bt=bt.to(DEV),
                seg=torch.tensor(info, dtype=torch.int32, device=DEV), n_segs=len(segs), plan=plan,
                items=torch.from_numpy(plan.items).to(DEV), tile=tile, G=G, Hq=Hq, Hkv=Hkv, D=D, P=P,
                n_pages=n_pages)


def ordinary(pr):
    plan = pr["plan"]
    po = torch.empty(plan.n_slots, pr["Hkv"], pr["tile"], pr["D"], dtype=torch.float32, device=DEV)
    pm = torch.empty(plan.n_slots, pr["Hkv"], pr["tile"], 2, dtype=torch.float32, device=DEV)
    out = torch.empty_like(pr["q"])
    ops.paged_attention(pr["q"], pr["ks"], pr["vs"], pr["bt"], pr["seg"], pr["n_segs"], pr["items"], plan.n_items,
                        po, pm, out, pr["tile"], pr["D"] ** -0.5, None)
    return out


def static_scratch(lib, pr):
    plan = pr["plan"]
    out = torch.empty_like(pr["q"])
    host_items = np.ascontiguousarray(plan.items, dtype=np.int32)
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = lib.ftk_paged_attention_static_scratch
    fn.restype = i32
    fn.argtypes = [vp, vp, vp, i32, vp, i32, vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32, i32, vp]
    rc = fn(pr["q"].data_ptr(), pr["ks"].data_ptr(), pr["vs"].data_ptr(),
            ops.F32 if pr["q"].dtype == torch.float32 else ops.BF16,
            pr["bt"].data_ptr(), pr["bt"].shape[1], pr["seg"].data_ptr(), pr["n_segs"],
            host_items.ctypes.data, pr["items"].data_ptr(), plan.n_items, out.data_ptr(),
            pr["Hq"], pr["Hkv"], pr["D"], pr["P"], pr["n_pages"], pr["tile"], pr["D"] ** -0.5, 0,
            torch.cuda.current_stream().cuda_stream)
    return rc, out


@pytest.mark.parametrize("dtype,tile", [(torch.float32, 16), (torch.bfloat16, 64), (torch.bfloat16, 16)])
def test_static_scratch_matches_the_ordinary_entry_point_twice_in_a_row(dtype, tile):
    """16-row bfloat16 tiles are the decode kernel, whose splits are merged by the split that arrives last
    (single tokens only); 64-row tiles and float32 use the separate merge."""
    lib = library.load()
    tol = dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=1.5e-2)
    single = dtype == torch.bfloat16 and tile == 16
    first = problem(dtype, 1, [(1, 900), (1 if single else 2, 300), (1, 64)], tile=tile)
    second = problem(dtype, 2, [(1, 450), (1, 777), (1 if single else 3, 129), (1, 20)], tile=tile)
    for pr in (first, second):  # the second call finds the first call's partial results in the array
        want = ordinary(pr)
        rc, got = static_scratch(lib, pr)
        assert rc == 0, lib.ftk_last_error().decode()
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), **tol)


def test_static_scratch_refuses_what_does_not_fit():
    lib = library.load()
    pr = problem(torch.float32, 3, [(1, 300)], Hq=8, Hkv=8, D=256)
    # a work list for 40 long requests needs far more than 16 MiB of partial results; the call is
    # refused before anything is launched, so the small tensors above are never touched
    pr["plan"] = build_plan([(1, 4000)] * 40, 1, 16, None, 8, sm_count=4096, min_split_keys=32)
    pr["items"] = torch.from_numpy(pr["plan"].items).to(DEV)
    assert pr["plan"].n_slots * 8 * 16 * (256 + 2) * 4 > (16 << 20)
    rc, _ = static_scratch(lib, pr)
    assert rc != 0
    assert b"static array holds" in lib.ftk_last_error()
    # a work list whose numbers make no sense is refused too, before any size is computed from it
    bad = pr["plan"].items.copy()
    bad[0, 5], bad[0, 7] = 3, -5
    pr["plan"].items[:] = bad
    rc, _ = static_scratch(lib, pr)
    assert rc != 0 and b"split" in lib.ftk_last_error()
