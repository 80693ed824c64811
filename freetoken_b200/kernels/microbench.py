"""Times one kernel at a time at given sizes and reports it against its roofline.

    python -m freetoken_b200.kernels.microbench moe --experts 256 --tokens 8 [--hidden 3072 --inter 1536 --top-k 8]
    python -m freetoken_b200.kernels.microbench attention --batch 8 --context 2048
    python -m freetoken_b200.kernels.microbench attention --prefill 2048
    python -m freetoken_b200.kernels.microbench sample --rows 8 --vocab 200064
    python -m freetoken_b200.kernels.microbench few --tokens 1
    python -m freetoken_b200.kernels.microbench sparse --batch 8 --context 32768
    python -m freetoken_b200.kernels.microbench sparse --prefill 2048 --context 32768

Each case allocates its inputs once (larger than L2 where the real workload is), warms up, then
times ``--iters`` launches with CUDA events and prints one JSON line: time, the bytes the kernel has
to move (or its flops), and the fraction of the HBM or tensor peak that this is.  ``--profile`` brackets
a few launches with cudaProfilerStart/Stop for ``ncu --profile-from-start off`` on a small case.
The reference reports per-kernel bandwidth the same way (python/freetoken/benchmark/perf.py:60-74).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from ..engine.attention_plan import TC_ONE_TILE_COSTS, TC_TWO_TILE_COSTS, build_plan, wave_splits
from . import ops

HBM_GBS = 6650.0  # used when no measured peaks are on file
BF16_TFLOPS = 1590.0
_PEAKS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "MEASURED_PEAKS.json")
if os.path.isfile(_PEAKS):  # the copy rate and library product rate measured on this machine's GPUs
    try:
        with open(_PEAKS) as _f:
            _m = json.load(_f)
        HBM_GBS = float(_m.get("hbm_gbs", HBM_GBS))
        BF16_TFLOPS = float(_m.get("bf16_tflops", BF16_TFLOPS))
    except (OSError, ValueError):
        pass


def _time(fn, iters: int, warmup: int, profile: bool) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if profile:
        torch.cuda.profiler.start()
        for _ in range(min(iters, 3)):
            fn()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return float("nan")
    # the launches are replayed from a CUDA graph so that the figure is device time, not the
    # Python call overhead of issuing them
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e3  # microseconds


def bench_moe(a) -> dict:
    dev = "cuda"
    ops.set_moe_pairs(not getattr(a, "no_pairs", False))
    E, H, I, k, T = a.experts, a.hidden, a.inter, a.top_k, a.tokens
    g = torch.Generator(device=dev).manual_seed(0)
    w1 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    routes = torch.empty(T * k, dtype=torch.int32, device=dev)
    pos = torch.empty(T * k, dtype=torch.int32, device=dev)
    ops.moe_permute(ids, E, counts, off, routes, pos)
    h = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    x = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    ops.moe_gather(h, routes, k, x)
    act = torch.empty(T * k, I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    wts = torch.rand(T * k, device=dev)
    distinct = int((counts > 0).sum())
    out = {}
    for name, fn, wbytes, flops in (
            ("gemm1", lambda: ops.moe_gemm1_act(x, w1, off, "silu", 1.702, 7.0, act), distinct * 2 * I * H * 2,
             2 * T * k * 2 * I * H),
            ("gemm1_gather", (lambda: ops.moe_gemm1_act_gather(h, routes, k, w1, off, "silu", 1.702, 7.0, act))
             if ops.moe_gemm1_gather_fits(torch.bfloat16, H, I, E, T * k) else None,
             distinct * 2 * I * H * 2, 2 * T * k * 2 * I * H),
            ("gemm2", lambda: ops.moe_gemm2(act, w2, off, routes, wts, y), distinct * H * I * 2, 2 * T * k * H * I)):
        if (a.only and a.only != name) or fn is None:
            continue
        us = _time(fn, a.iters, a.warmup, a.profile)
        out[name] = {"us": round(us, 2), "weight_bytes": wbytes, "gbs": round(wbytes / us / 1e3, 1),
                     "hbm_frac": round(wbytes / us / 1e3 / HBM_GBS, 3),
                     "tflops": round(flops / us / 1e6, 1), "tensor_frac": round(flops / us / 1e6 / BF16_TFLOPS, 3)}
    out["distinct_experts"] = distinct
    out["status"] = ops.read_status()
    return out


def bench_attention(a) -> dict:
    dev = "cuda"
    Hq, Hkv, D, P = a.q_heads, a.kv_heads, a.head_dim, a.page_size
    G = Hq // Hkv
    if a.prefill:
        segs = [(a.prefill, a.past + a.prefill)]  # a portion of a prompt after --past earlier tokens
    else:
        segs = [(1, a.context)] * a.batch
    n_pages = sum(-(-kv // P) for _, kv in segs) + 1
    g = torch.Generator(device=dev).manual_seed(0)
    ks = torch.empty(n_pages, Hkv, P, D, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    vs = torch.empty(n_pages, Hkv, P, D, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    width = max(-(-kv // P) for _, kv in segs)
    bt = torch.zeros(len(segs), width, dtype=torch.int32)
    info, q0, page = [], 0, 1
    for row, (ql, kv) in enumerate(segs):
        n = -(-kv // P)
        bt[row, :n] = torch.arange(page, page + n)
        page += n
        info.append([q0, ql, kv, row])
        q0 += ql
    bt = bt.to(dev)
    seg = torch.tensor(info, dtype=torch.int32, device=dev)
    q = torch.randn(q0, Hq, D, device=dev, generator=g).to(torch.bfloat16)
    fixed = None
    tile = 128 if (a.prefill >= 128 and not a.no_tc and ops.attention_tc_fits(D, P, G)) else 64
    if tile == 128 and a.pair:
        tile = 256  # two query tiles per CTA
    few_rows = False
    if not a.prefill:
        few_rows = a.few_rows and ops.attention_tc_few_fits(D, P, G)
        tc = few_rows or (a.tc and ops.attention_tc_fits(D, P, G))
        fixed = wave_splits(len(segs) * Hkv, 148 if tc else 2 * 148, 16, a.context) if a.splits is None else a.splits
        tile = 16 if few_rows else 128 if tc else (16 if G <= 16 else 64)
    tensor_core = few_rows or tile >= 128  # (one CTA per SM: the engine plans these for half as many CTA slots)
    costs = None
    if tile >= 128 and fixed is None:  # as the engine plans these kernels' work lists
        costs = TC_TWO_TILE_COSTS if tile == 256 else TC_ONE_TILE_COSTS
    plan = build_plan(segs, G, tile, None, Hkv, sm_count=74 if tensor_core else 148, fixed_splits=fixed,
                      key_tile=128 if tensor_core else 0, costs=costs)
    items = torch.from_numpy(plan.items).to(dev)
    po = pm = None
    if plan.n_slots:
        po = torch.empty(plan.n_slots, Hkv, tile, D, dtype=torch.float32, device=dev)
        pm = torch.empty(plan.n_slots, Hkv, tile, 2, dtype=torch.float32, device=dev)
    out = torch.empty_like(q)
    us = _time(lambda: ops.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, po, pm, out, tile,
                                           D ** -0.5, None, few_rows=few_rows), a.iters, a.warmup, a.profile)
    kv_bytes = sum(kv for _, kv in segs) * Hkv * D * 2 * 2
    flops = sum(4 * (ql * kv - ql * (ql - 1) // 2) * Hq * D for ql, kv in segs)
    return {"us": round(us, 2), "items": plan.n_items, "est_us": None if plan.est_us is None else round(plan.est_us, 1),
            "kv_bytes": kv_bytes, "gbs": round(kv_bytes / us / 1e3, 1),
            "hbm_frac": round(kv_bytes / us / 1e3 / HBM_GBS, 3), "tflops": round(flops / us / 1e6, 1),
            "tensor_frac": round(flops / us / 1e6 / BF16_TFLOPS, 3)}


def bench_few(a) -> dict:
    """The few-token kernels (``csrc/gemv.cu``) at the headline sizes: the qkv and output projections of
    ``--tokens`` tokens, and the routed gate/up and down products of their routes.  Six copies of the dense
    weights and other experts every launch, so that every launch reads its weights from memory."""
    dev = "cuda"
    H, I, E, k, T = a.hidden, a.inter, a.experts, a.top_k, a.tokens
    q_dim, kv_dim, copies = a.q_heads * a.head_dim, a.kv_heads * a.head_dim, 6
    g = torch.Generator(device=dev).manual_seed(0)
    wq = torch.empty(copies, q_dim + 2 * kv_dim, H, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    wo = torch.empty(copies, H, q_dim, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    w1 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    xo = torch.randn(T, q_dim, device=dev, generator=g).to(torch.bfloat16)
    qkv = torch.empty(T, q_dim + 2 * kv_dim, dtype=torch.bfloat16, device=dev)
    o = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    ids = [torch.stack([(torch.randperm(E, device=dev, generator=g)[:k]) for _ in range(T)]).to(torch.int32)
           for _ in range(copies)]
    wts = torch.rand(T, k, device=dev)
    act = torch.empty(T * k, I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    turn = [0]

    def nxt():
        turn[0] = (turn[0] + 1) % copies
        return turn[0]

    cases = (
        ("qkv", lambda: ops.small_linear(x, wq[nxt()], qkv), (q_dim + 2 * kv_dim) * H * 2),
        ("out_proj", lambda: ops.small_linear(xo, wo[nxt()], o), H * q_dim * 2),
        ("gate_up", lambda: ops.moe_small_gate_up(x, ids[nxt()], w1, "silu", 1.702, 7.0, act), T * k * 2 * I * H * 2),
        ("down", lambda: ops.moe_small_down(act, ids[nxt()], wts, w2, y), T * k * H * I * 2))
    out = {}
    for name, fn, nbytes in cases:
        if a.only and a.only != name:
            continue
        us = _time(fn, a.iters, a.warmup, a.profile)
        out[name] = {"us": round(us, 2), "weight_bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1),
                     "hbm_frac": round(nbytes / us / 1e3 / HBM_GBS, 3)}
    return out


def bench_sparse(a) -> dict:
    """The block-sparse layer kind at its real geometry (the reference's M3: blocks of 128 keys, 16 chosen
    blocks, 64 query heads on 4 KV heads of 128, one shared index key of 128 per token): block selection
    (index scores, forced blocks, top-k) and attention over the chosen blocks, for single tokens of
    ``--batch`` requests at ``--context`` tokens, or for a ``--prefill`` portion at the end of one request of
    ``--context`` tokens.  Bytes: the visible index keys once per request and step; the chosen keys and values
    per token and KV head."""
    dev = "cuda"
    Hq, Hkv, D, P, Di = a.q_heads, a.kv_heads, a.head_dim, a.page_size, a.head_dim
    block, topk = a.block, a.topk
    segs = [(a.prefill, a.context)] if a.prefill else [(1, a.context)] * a.batch
    n_pages = sum(-(-kv // P) for _, kv in segs) + 1
    g = torch.Generator(device=dev).manual_seed(0)
    ks = torch.empty(n_pages, Hkv, P, D, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    vs = torch.empty(n_pages, Hkv, P, D, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    iks = torch.empty(n_pages, 1, P, Di, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=g)
    width = max(-(-kv // P) for _, kv in segs)
    bt = torch.zeros(len(segs), width, dtype=torch.int32)
    info, q0, page = [], 0, 1
    for row, (ql, kv) in enumerate(segs):
        n = -(-kv // P)
        bt[row, :n] = torch.arange(page, page + n)
        page += n
        info.append([q0, ql, kv, row])
        q0 += ql
    bt, T = bt.to(dev), q0
    seg = torch.tensor(info, dtype=torch.int32, device=dev)
    q = torch.randn(T, Hq, D, device=dev, generator=g).to(torch.bfloat16)
    iq = torch.randn(T, Hkv, Di, device=dev, generator=g).to(torch.bfloat16)
    sel = torch.empty(T, Hkv, topk, dtype=torch.int32, device=dev)
    max_blocks = -(-a.context // block)
    out = {}
    scores = None
    if not a.no_tc and ops.sparse_score_fits(Hkv, Di, block):
        scores = torch.empty(T, Hkv, max_blocks, dtype=torch.float32, device=dev)
    us = _time(lambda: ops.sparse_select(iq, iks, bt, seg, len(segs), block, a.local, a.init, max_blocks, sel, scores,
                                         live_blocks=-(-a.context // block)),
               a.iters, a.warmup, a.profile)
    index_bytes = sum(kv for _, kv in segs) * Di * 2
    flops = sum(2 * (ql * kv - ql * (ql - 1) // 2) * Hkv * Di for ql, kv in segs)
    out["select"] = {"us": round(us, 2), "index_key_bytes": index_bytes, "gbs": round(index_bytes / us / 1e3, 1),
                     "hbm_frac": round(index_bytes / us / 1e3 / HBM_GBS, 3), "tflops": round(flops / us / 1e6, 2)}
    plan = build_plan(segs, Hq // Hkv, 16, None, Hkv, sparse=(block, topk))
    items = torch.from_numpy(plan.items).to(dev)
    po = pm = None
    if plan.n_slots:
        po = torch.empty(plan.n_slots, Hkv, 16, D, dtype=torch.float32, device=dev)
        pm = torch.empty(plan.n_slots, Hkv, 16, 2, dtype=torch.float32, device=dev)
    o = torch.empty_like(q)
    us = _time(lambda: ops.paged_attention(q, ks, vs, bt, seg, len(segs), items, plan.n_items, po, pm, o, 16, D ** -0.5,
                                           None, sel=sel, block_size=block), a.iters, a.warmup, a.profile)
    kv_bytes = sum(min(topk * block, kv - ql + t + 1) for ql, kv in segs for t in range(ql)) * Hkv * D * 2 * 2
    out["attend"] = {"us": round(us, 2), "items": plan.n_items, "kv_bytes": kv_bytes, "gbs": round(kv_bytes / us / 1e3, 1),
                     "hbm_frac": round(kv_bytes / us / 1e3 / HBM_GBS, 3)}
    return out


def bench_sample(a) -> dict:
    dev = "cuda"
    logits = torch.randn(a.rows, a.vocab, device=dev)
    temp = torch.full((a.rows,), a.temperature, device=dev)
    top_k = torch.zeros(a.rows, dtype=torch.int32, device=dev)
    top_p = torch.ones(a.rows, device=dev)
    u = torch.rand(a.rows, device=dev)
    out = torch.empty(a.rows, dtype=torch.int32, device=dev)
    us = _time(lambda: ops.sample(logits, temp, top_k, top_p, u, out), a.iters, a.warmup, a.profile)
    nbytes = a.rows * a.vocab * 4
    return {"us": round(us, 2), "bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="microbench")
    sub = ap.add_subparsers(dest="case", required=True)
    for name in ("moe", "attention", "sample", "sparse", "few"):
        p = sub.add_parser(name)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--warmup", type=int, default=5)
        p.add_argument("--profile", action="store_true")
        if name == "moe":
            p.add_argument("--experts", type=int, default=256)
            p.add_argument("--tokens", type=int, default=8)
            p.add_argument("--hidden", type=int, default=3072)
            p.add_argument("--inter", type=int, default=1536)
            p.add_argument("--top-k", type=int, default=8)
            p.add_argument("--only", choices=["gemm1", "gemm2"], default=None)
            p.add_argument("--no-pairs", action="store_true",
                           help="128- and 256-token tiles on the one-CTA form of the tcgen05 kernel instead of pairs of CTAs")
        elif name == "attention":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--context", type=int, default=2048)
            p.add_argument("--prefill", type=int, default=0)
            p.add_argument("--past", type=int, default=0, help="tokens of the request before the --prefill portion")
            p.add_argument("--q-heads", type=int, default=48)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--page-size", type=int, default=16)
            p.add_argument("--splits", type=int, default=None)
            p.add_argument("--no-tc", action="store_true", help="prefill on the mma.sync kernel instead of tcgen05")
            p.add_argument("--tc", action="store_true", help="decode on the tcgen05 kernel with 128-row query tiles")
            p.add_argument("--few-rows", action="store_true",
                           help="decode on the tcgen05 kernel in its form for tiles of at most 16 rows")
            p.add_argument("--pair", action="store_true", help="prefill on the tcgen05 kernel with two query tiles per CTA")
        elif name == "few":
            p.add_argument("--tokens", type=int, default=1)
            p.add_argument("--hidden", type=int, default=3072)
            p.add_argument("--inter", type=int, default=1536)
            p.add_argument("--experts", type=int, default=256)
            p.add_argument("--top-k", type=int, default=8)
            p.add_argument("--q-heads", type=int, default=48)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--only", choices=["qkv", "out_proj", "gate_up", "down"], default=None)
        elif name == "sparse":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--context", type=int, default=32768)
            p.add_argument("--prefill", type=int, default=0)
            p.add_argument("--q-heads", type=int, default=64)
            p.add_argument("--kv-heads", type=int, default=4)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--page-size", type=int, default=16)
            p.add_argument("--block", type=int, default=128)
            p.add_argument("--topk", type=int, default=16)
            p.add_argument("--local", type=int, default=1)
            p.add_argument("--init", type=int, default=0)
            p.add_argument("--no-tc", action="store_true", help="block scores by a CTA per token and head instead of mma.sync")
        else:
            p.add_argument("--rows", type=int, default=8)
            p.add_argument("--vocab", type=int, default=200064)
            p.add_argument("--temperature", type=float, default=0.0)
    a = ap.parse_args(argv)
    res = {"moe": bench_moe, "attention": bench_attention, "sample": bench_sample, "sparse": bench_sparse, "few": bench_few}[a.case](a)
    print(json.dumps({"case": a.case, **{k: v for k, v in vars(a).items() if k != "case"}, "result": res}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
