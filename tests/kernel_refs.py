"""Plain PyTorch statement of every op in ``freetoken_b200.kernels.ops``, argument for argument.

Two uses: the ``-m gpu`` tests compare each CUDA kernel with its function here (computed in
float32 on the same inputs), and the CPU tests run the engine's step, cache and scheduler
logic with these functions standing in for the kernels (``install``), so that the host-side
code can be checked without a GPU.  Nothing in ``freetoken_b200`` imports this file.

Rounding: a function computes in float32 and rounds once into the dtype of its output.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch


def embedding_gather(table, ids, out):
    out.copy_(table[ids.long()].float())


def add_rmsnorm(x, residual, weight, eps, gemma, out, out_f32=None, rows=None):
    if rows is not None:
        idx = rows.long()
        z = residual[idx].float() if residual is not None else 0
        if x is not None:
            z = z + x[idx].float()
    else:
        z = residual.float() if residual is not None else 0
        if x is not None:
            z = z + x.float()
        if residual is not None and x is not None:
            residual.copy_(z)
    w = weight.float() + 1.0 if gemma else weight.float()
    inv = torch.rsqrt((z * z).sum(-1, keepdim=True) / z.shape[-1] + eps)
    y = (z * inv * w).to(out.dtype)
    out.view(y.shape).copy_(y)
    if out_f32 is not None:
        out_f32.view(y.shape).copy_(y.float())


def add_rmsnorm_routes(y, route_pos, top_k, shared, residual, weight, eps, gemma, out, out_f32=None, rows=None):
    T = residual.shape[0]
    delta = torch.empty(T, y.shape[1], dtype=y.dtype, device=y.device)
    moe_combine(y, route_pos, T, top_k, shared, delta)
    add_rmsnorm(delta, residual, weight, eps, gemma, out, out_f32=out_f32, rows=rows)


def act_and_mul(gate_up, out, act, alpha, limit):
    I = gate_up.shape[1] // 2
    g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    if act == "silu":
        y = g * torch.sigmoid(g) * u
    else:
        g = torch.clamp(g, max=limit)
        u = torch.clamp(u, min=-limit, max=limit)
        y = g * torch.sigmoid(alpha * g) * (u + 1.0)
    out.copy_(y.to(out.dtype))


def cast(src, dst):
    dst.view(-1).copy_(src.reshape(-1).to(dst.dtype))


def copy_tokens(dst, pairs, src, n, vocab):
    for d, s_ in pairs.view(-1, 2)[:n].tolist():
        if d >= 0 and s_ >= 0:
            v = int(src[s_])
            dst[d] = v if 0 <= v < vocab else 0


def table_update(table, updates, n_updates):
    u = updates.view(-1, 2)[:n_updates]
    ok = u[:, 0] >= 0
    table.view(-1)[u[ok, 0].long()] = u[ok, 1]


def norm_rope_store(x, head_dim, rotary_dim, positions, rope_table, eps, gemma, sections):
    T = x.shape[0]
    xs = x.view(T, -1, head_dim).float()
    half = rotary_dim // 2
    if rotary_dim:
        cs = rope_table[positions.long()]
        cos, sin = cs[:, None, :half], cs[:, None, half:]
    for s in sections:
        u = xs[:, s["first_head"]: s["first_head"] + s["n_heads"]]
        w = s.get("norm_weight")
        if w is not None:
            scale = w.float() + 1.0 if gemma else w.float()
            u = u * torch.rsqrt((u * u).sum(-1, keepdim=True) / head_dim + eps) * scale
        if s.get("rotate") and rotary_dim:
            a, b, rest = u[..., :half], u[..., half:rotary_dim], u[..., rotary_dim:]
            u = torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)
        if s.get("dense_out") is not None:
            s["dense_out"].view(T, s["n_heads"], head_dim).copy_(u.to(x.dtype))
        else:
            slab, slots = s["slab"], s["slot_map"][:T].long()
            P = slab.shape[2]
            ok = slots >= 0
            page, off = slots[ok] // P, slots[ok] % P
            slab[page, :, off, :] = u[ok].to(slab.dtype)


def paged_attention(q, k_slab, v_slab, block_table, seg_info, n_segs, items, n_items, part_o, part_ml,
                    out, tile_rows, scale, window, sel=None, block_size=0, few_rows=False):
    """Per query token, softmax over the visible keys gathered through the block table; the
    work list and the scratch are ignored (they only steer how the kernel splits the work).
    With ``sel`` a query reads only the keys of its chosen blocks."""
    T, Hq, D = q.shape
    P = k_slab.shape[2]
    Hkv = k_slab.shape[1]
    G = Hq // Hkv
    info = seg_info.view(-1, 4)[:n_segs].tolist()
    for q_start, q_len, kv_len, row in info:
        pos = torch.arange(kv_len, device=q.device)
        pages = block_table[row, (pos // P).long()].long()
        K = k_slab[pages, :, (pos % P).long(), :].float()  # [kv, Hkv, D]
        V = v_slab[pages, :, (pos % P).long(), :].float()
        for t in range(q_len):
            p_q = kv_len - q_len + t
            lo = 0 if not window else max(0, p_q - window + 1)
            qq = q[q_start + t].float().view(-1, G, D)  # [Hkv, G, D]
            if sel is None:
                kk, vv = K[lo:p_q + 1], V[lo:p_q + 1]
                s = torch.einsum("hgd,khd->hgk", qq, kk) * scale
                p = torch.softmax(s, dim=-1)
                o = torch.einsum("hgk,khd->hgd", p, vv)
            else:
                o = torch.zeros(Hkv, G, D, device=q.device)
                for h in range(Hkv):
                    blocks = [int(b) for b in sel[q_start + t, h].tolist() if b >= 0]
                    idx = torch.cat([torch.arange(b * block_size, min((b + 1) * block_size, p_q + 1))
                                     for b in blocks]).to(q.device)
                    s = (qq[h] @ K[idx, h].T) * scale
                    o[h] = torch.softmax(s, dim=-1) @ V[idx, h]
            out[q_start + t] = o.reshape(Hq, D).to(out.dtype)


def sparse_score_fits(n_heads, dim, block_size):
    return False


def sparse_select(iq, ik_slab, block_table, seg_info, n_segs, block_size, local_blocks, init_blocks, max_blocks, sel,
                  scores=None, live_blocks=0):
    T, Hi, Di = iq.shape
    P = ik_slab.shape[2]
    topk = sel.shape[2]
    sel[:T] = -1
    for q_start, q_len, kv_len, row in seg_info.view(-1, 4)[:n_segs].tolist():
        pos = torch.arange(kv_len, device=iq.device)
        pages = block_table[row, (pos // P).long()].long()
        IK = ik_slab[pages, 0, (pos % P).long(), :].float()  # [kv, Di]
        for t in range(q_len):
            p_q = kv_len - q_len + t
            nb = p_q // block_size + 1
            scores = iq[q_start + t].float() @ IK[: p_q + 1].T  # [Hi, p_q + 1]
            pad = nb * block_size - (p_q + 1)
            if pad:
                scores = torch.nn.functional.pad(scores, (0, pad), value=float("-inf"))
            bs = scores.view(Hi, nb, block_size).amax(-1)
            bs = torch.where(torch.isnan(bs), torch.full_like(bs, -1e30), bs)
            if init_blocks:
                bs[:, : min(init_blocks, nb)] = 1e30
            if local_blocks:
                bs[:, max(0, nb - local_blocks):] = 1e29
            order = torch.argsort(bs, dim=-1, descending=True, stable=True)[:, : min(topk, nb)]
            chosen = torch.sort(order, dim=-1).values
            sel[q_start + t, :, : chosen.shape[1]] = chosen.to(torch.int32)


def router_topk(logits, bias, top_k, scoring, scale, ids, weights, n_parts=1):
    l = logits.float()
    if n_parts > 1:
        parts = l.view(l.shape[0], n_parts, -1)
        l = parts[:, 0]
        for q in range(1, n_parts):
            l = l + parts[:, q]
    s = torch.sigmoid(l) if scoring == "sigmoid" else torch.softmax(l, dim=-1)
    c = s + bias.float() if bias is not None else s
    idx = torch.argsort(c, dim=-1, descending=True, stable=True)[:, :top_k]
    w = s.gather(-1, idx)
    w = w / (w.sum(-1, keepdim=True) + (1e-20 if scoring == "sigmoid" else 0.0))
    ids.copy_(idx.to(torch.int32))
    weights.copy_(w * scale)


def moe_permute(topk_ids, n_experts, expert_counts, expert_offsets, sorted_routes, route_pos):
    flat = topk_ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=n_experts)
    expert_counts.copy_(counts.to(torch.int32))
    expert_offsets[0] = 0
    expert_offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    sorted_routes.copy_(order.to(torch.int32))
    route_pos[order] = torch.arange(flat.numel(), dtype=torch.int32, device=flat.device)


def linear(x, w, out):
    out.copy_((x.float() @ w.float().T).to(out.dtype))


def moe_gemm1_gather_fits(dtype, hidden, inter, n_experts, n_routes):
    return False  # the CPU tests copy the rows first


def attention_tc_fits(head_dim, page_size, group):
    return False  # the CPU tests plan for the other kernels


def attention_tc_few_fits(head_dim, page_size, group):
    return False


def moe_small_fits(n_tokens, hidden, inter, top_k):
    return False  # the few-token kernels are a second route to the same result; the CPU stand-ins take the general one


def moe_route_fits(n_tokens, hidden, n_experts, top_k):
    return 1 <= n_tokens <= 32 and hidden % 4 == 0


def moe_route(x, gate_w, bias, top_k, scoring, scale, logits, ids, weights, expert_counts, expert_offsets,
              sorted_routes, route_pos):
    logits.copy_(x.float() @ gate_w.float().T)
    router_topk(logits, bias, top_k, scoring, scale, ids, weights)
    moe_permute(ids, gate_w.shape[0], expert_counts, expert_offsets, sorted_routes, route_pos)


def moe_gather(h, sorted_routes, top_k, out):
    out.copy_(h[(sorted_routes.long() // top_k)])


def moe_gemm1_act(x_sorted, w1, expert_offsets, act, alpha, limit, out):
    off = expert_offsets.tolist()
    for e in range(w1.shape[0]):
        a, b = off[e], off[e + 1]
        if b > a:
            gu = x_sorted[a:b].float() @ w1[e].float().T
            gu = gu.to(x_sorted.dtype)  # the serving path stores the product before the activation
            act_and_mul(gu, out[a:b], act, alpha, limit)


def moe_gemm2(a, w2, expert_offsets, sorted_routes, topk_weights, out):
    off = expert_offsets.tolist()
    wr = topk_weights.reshape(-1)[sorted_routes.long()].float()
    for e in range(w2.shape[0]):
        lo, hi = off[e], off[e + 1]
        if hi > lo:
            y = (a[lo:hi].float() @ w2[e].float().T) * wr[lo:hi, None]
            out[lo:hi] = y.to(out.dtype)


def moe_combine(y, route_pos, n_tokens, top_k, shared, out):
    pos = route_pos.view(n_tokens, top_k).long()
    acc = torch.zeros(n_tokens, y.shape[1], dtype=torch.float32, device=y.device)
    for j in range(top_k):
        acc = acc + y[pos[:, j]].float()
    if shared is not None:
        acc = acc + shared.float()
    out.copy_(acc.to(out.dtype))


def sample(logits, temperature, top_k, top_p, u, out):
    R, V = logits.shape
    for r in range(R):
        t = float(temperature[r])
        row = logits[r].float()
        if t <= 0:
            out[r] = int(torch.argmax(row))
            continue
        p = torch.softmax(row / max(t, 1e-6), dim=-1)
        k = int(top_k[r])
        if 0 < k < V:
            kth = torch.topk(p, k).values[-1]
            p = torch.where(p >= kth, p, torch.zeros_like(p))
        tp = float(top_p[r])
        if tp < 1.0:
            vals = torch.sort(p, descending=True).values.double()
            csum = torch.cumsum(vals, 0)
            n = int((csum < tp * float(csum[-1])).sum())
            th = vals[min(n, V - 1)].float()
            p = torch.where(p >= th, p, torch.zeros_like(p))
        csum = torch.cumsum(p.double(), 0)
        target = float(u[r]) * float(csum[-1])
        idx = int((csum <= target).sum())
        nz = torch.nonzero(p > 0).view(-1)
        idx = min(idx, int(nz[-1]))
        out[r] = idx


ALL = ["sparse_score_fits", "moe_small_fits", "copy_tokens", "sparse_select", "embedding_gather", "add_rmsnorm", "add_rmsnorm_routes", "act_and_mul", "cast", "table_update", "norm_rope_store",
       "paged_attention", "router_topk", "moe_permute", "moe_route", "moe_route_fits", "linear", "attention_tc_fits", "attention_tc_few_fits", "moe_gemm1_gather_fits", "moe_gather", "moe_gemm1_act", "moe_gemm2",
       "moe_combine", "sample"]


def install(monkeypatch) -> None:
    """Make ``freetoken_b200.kernels.ops`` run these functions (CPU tests of the host logic)."""
    from freetoken_b200.kernels import ops

    for name in ALL:
        monkeypatch.setattr(ops, name, globals()[name])
