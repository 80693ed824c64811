"""Runs the pieces of the reference that run on a CPU, compares the plain implementation with
them, and writes their small outputs to ``tests/golden/golden.json``.

The reference's whole-model forward cannot run without a GPU, and importing its layers needs
the ``flashlib`` package, which is not installed; a three-line stand-in for
``flashlib.kernels.slot_cache`` is written to a temporary folder so that the rest imports.
What does run here, and is recorded:

``rope``, ``router``
    ``RotaryEmbedding._cos_sin_cache`` (python/freetoken/layers/rotary.py:49-59) and
    ``MiniMaxM3SparseMoeBlock._route`` (python/freetoken/models/minimax_m3/moe.py:71-81).
``sparse``, ``paged_attention``, ``fused_experts``
    The reference's own pure-PyTorch oracles, taken out of its test files by name (the files
    themselves skip without a GPU): ``ref_block_scores`` / ``ref_select`` / ``ref_sparse_attend``
    (tests/kernels/test_minimax_m3_sparse.py:43-113), ``_reference_paged_attention``
    (tests/kernels/test_triton_attention.py:9-46), ``_reference_fused_experts_decode``
    (tests/moe/test_fused_moe.py:14-39).
``norm``, ``rope_apply``, ``activation``, ``paged_attention.kernel``
    The reference's Triton kernels under Triton's CPU interpreter (``TRITON_INTERPRET=1``):
    ``gemma_rmsnorm`` / ``rmsnorm`` / ``gemma_fused_add_rmsnorm``
    (python/freetoken/kernel/triton/norm.py:42-112), ``_rope_tiled`` (rope.py:28-91),
    ``_act_and_mul_kernel`` (activation.py:67-112) and ``_paged_attention_kernel``
    (attention.py:45-145).  Wrappers that insist on CUDA tensors are bypassed by launching the
    kernel itself with the wrapper's arguments.  One change is made: the interpreter cannot run
    inline PTX, so ``_fast_ex2`` (``ex2.approx.f32``) is replaced by ``tl.exp2``; the formula
    around it is the reference's.
``state_dict``
    ``create_model`` on the meta device for the first five layers (three dense, two block-sparse
    MoE) of the real-M3-shaped config of tests/models/test_minimax_m3.py:27-79, with the resident
    quantisation switched off: names, shapes, dtypes.
``config``
    ``parse_config`` on that config in both key shapes (raw and native).
``chunked_prefill``
    The page-accounting drive of tests/scheduler/test_scheduler_chunked_prefill.py:49-90 on the
    reference's own managers (cache type ``naive``, the one without prefix reuse): free pages
    after every iteration.

Run from the repository root with the reference mounted:

    python tests/golden/make_golden.py /path/to/reference

It asserts that the plain implementation agrees with each of them and stores seeds and the
reference's outputs, which ``tests/test_plain.py`` (and, for the cache manager and the config
reader, ``tests/test_golden_host.py``) compares against without needing the reference.
"""

from __future__ import annotations

import ast
import json
import os
import sys
import tempfile
import types

os.environ["TRITON_INTERPRET"] = "1"  # before triton is imported

import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from plain import m3_plain  # noqa: E402


@triton.jit
def exact_ex2(x):  # stands in for the reference's inline ``ex2.approx.f32``, which the interpreter cannot run
    return tl.exp2(x)


def functions_of(path: str, names) -> dict:
    """The named top-level functions and classes of a Python file, executed on their own (the
    reference's test modules skip at import without a GPU)."""
    with open(path) as f:
        tree = ast.parse(f.read())
    keep = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    missing = set(names) - {n.name for n in keep}
    assert not missing, f"{path}: {missing} not found"
    head = ast.parse("from __future__ import annotations\nimport torch\n")
    ns: dict = {}
    exec(compile(ast.Module(head.body + keep, []), path, "exec"), ns)
    return ns


def lst(t: torch.Tensor):
    return t.detach().float().cpu().tolist()


def rand(gen, *shape, scale=1.0):
    return torch.randn(*shape, generator=gen) * scale


def chopped(t: torch.Tensor) -> torch.Tensor:
    """float32 -> bfloat16 as Triton's CPU interpreter does it: the low 16 bits are dropped (the GPU
    rounds to nearest even).  Used where an interpreted kernel stores bfloat16, so that the comparison
    is about the arithmetic before the store."""
    return (t.float().contiguous().view(torch.int32) & ~0xFFFF).view(torch.float32)


def plain_cfg(**kw):
    base = dict(act="silu", alpha=1.702, limit=7.0, top_k=2, scale=1.0, scoring="sigmoid", bias=True, n_shared=0)
    base.update(kw)
    return types.SimpleNamespace(**base)


# --------------------------------------------------------------------------- sections
def rope_and_router(golden):
    from freetoken.layers.rotary import RotaryEmbedding
    from freetoken.models.minimax_m3.moe import MiniMaxM3SparseMoeBlock

    golden["rope"], golden["router"] = [], []
    for head, rd, theta, n in [(64, 64, 10000.0, 40), (128, 64, 5e6, 33), (64, 16, 1e6, 50)]:
        table = RotaryEmbedding(head, rd, n, theta)._cos_sin_cache
        cos, sin = m3_plain.rope_table(rd, theta, n, torch.float32)
        assert torch.equal(torch.cat((cos, sin), -1), table), "rope table differs"
        golden["rope"].append({"rotary_dim": rd, "theta": theta, "positions": n,
                               "rows": {str(p): table[p].tolist() for p in (0, 1, n - 1)}})
    for seed, (T, H, E, k, scale) in enumerate([(9, 48, 8, 2, 1.0), (5, 32, 16, 4, 2.0), (7, 64, 6, 3, 2.0)]):
        g = torch.Generator().manual_seed(seed)
        h = torch.randn(T, H, generator=g)
        w = torch.randn(E, H, generator=g) * 0.1
        b = torch.randn(E, generator=g) * 0.01
        me = types.SimpleNamespace(gate=types.SimpleNamespace(weight=w), e_score_correction_bias=b,
                                   top_k=k, norm_topk_prob=True, routed_scaling_factor=scale)
        wts, ids = MiniMaxM3SparseMoeBlock._route(me, h)
        cfg = types.SimpleNamespace(scoring="sigmoid", top_k=k, scale=scale)
        pw, pi = m3_plain.router(h, w, b, cfg)
        assert torch.equal(pi.to(torch.int32), ids), "router choice differs"
        torch.testing.assert_close(pw, wts, rtol=1e-6, atol=1e-7)
        golden["router"].append({"seed": seed, "T": T, "H": H, "E": E, "k": k, "scale": scale,
                                 "ids": ids.tolist(), "weights": wts.tolist()})


def sparse_inputs(seed, T, Hi, group, D):
    g = torch.Generator().manual_seed(seed)
    iq, ik = rand(g, T, Hi, D), rand(g, T, D)
    q, k, v = rand(g, T, Hi * group, D), rand(g, T, Hi, D), rand(g, T, Hi, D)
    return iq, ik, q, k, v


def sparse_oracles(golden, ref):
    """Block scores, selection and attention over the chosen blocks: blocks of 128 as the reference
    pins them, 300 positions (three blocks, the last one ragged)."""
    ns = functions_of(os.path.join(ref, "tests/kernels/test_minimax_m3_sparse.py"),
                      ["ref_block_scores", "ref_select", "ref_sparse_attend"])
    from freetoken.kernel.triton.minimax_m3_sparse import SPARSE_BLOCK_SIZE as BLK

    ns["BLK"] = BLK
    golden["sparse"] = []
    for seed, (T, Hi, group, D, topk, init, local) in enumerate([(300, 2, 2, 16, 2, 0, 1), (290, 1, 3, 8, 1, 1, 1),
                                                                 (400, 2, 1, 16, 2, 1, 2)]):
        iq, ik, q, k, v = sparse_inputs(100 + seed, T, Hi, group, D)
        q_pos = torch.arange(T)
        scores = ns["ref_block_scores"](iq, ik, q_pos)
        sel = ns["ref_select"](scores, q_pos, topk, init, local)
        out = ns["ref_sparse_attend"](q, k, v, sel, q_pos, D ** -0.5)
        allowed = m3_plain.sparse_block_selection(iq, ik, BLK, topk, local, init)
        mine = m3_plain.causal_attention(q, k, v, group, None, allowed)
        pos = torch.arange(T)
        for h in range(Hi):
            for t in range(T):
                want = torch.zeros(T, dtype=torch.bool)
                for b in sel[h][t]:
                    want[b * BLK: (b + 1) * BLK] = True
                assert torch.equal(allowed[h, t] & (pos <= t), want & (pos <= t)), (seed, h, t)
        torch.testing.assert_close(mine, out, rtol=1e-5, atol=1e-6)
        tokens = [0, 1, 127, 128, 129, 255, 256, 257, T - 1]
        golden["sparse"].append({
            "seed": 100 + seed, "T": T, "Hi": Hi, "group": group, "D": D, "block": BLK, "topk": topk, "init": init,
            "local": local, "tokens": tokens,
            "scores": [[[float(x) if x != float("-inf") else None for x in scores[h, t]] for t in tokens]
                       for h in range(Hi)],
            "selection": [[sorted(sel[h][t]) for t in tokens] for h in range(Hi)],
            "out": lst(out[tokens])})


def paged_inputs(seed, lens, q_lens, Hq, Hkv, D):
    g = torch.Generator().manual_seed(seed)
    total = sum(lens)
    perm = torch.randperm(total + 7, generator=g)[:total]  # logical order -> scattered slots
    k_cache, v_cache = rand(g, total + 7, Hkv, D), rand(g, total + 7, Hkv, D)
    indptr = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    q_to_req, q_pos = [], []
    for r, (n, ql) in enumerate(zip(lens, q_lens)):
        q_to_req += [r] * ql
        q_pos += list(range(n - ql, n))
    q = rand(g, len(q_pos), Hq, D)
    return q, k_cache, v_cache, indptr, perm.to(torch.int32), torch.tensor(q_to_req, dtype=torch.int32), \
        torch.tensor(q_pos, dtype=torch.int32)


def plain_paged(q, k_cache, v_cache, indptr, indices, q_to_req, q_pos, group, window=None):
    """The plain attention on each request's keys gathered in order; the queries are its last rows."""
    out = torch.empty_like(q)
    for r in range(indptr.numel() - 1):
        slots = indices[int(indptr[r]): int(indptr[r + 1])].long()
        K, V = k_cache[slots], v_cache[slots]
        rows = (q_to_req == r).nonzero().view(-1)
        n = K.shape[0]
        full_q = torch.zeros(n, q.shape[1], q.shape[2])
        full_q[q_pos[rows].long()] = q[rows]
        allowed = None
        if window is not None:
            p = torch.arange(n)
            allowed = (p[None, :] + window > p[:, None]).expand(K.shape[1], n, n)
        o = m3_plain.causal_attention(full_q, K, V, group, None, allowed)
        out[rows] = o[q_pos[rows].long()]
    return out


def paged_attention_oracle(golden, ref):
    ns = functions_of(os.path.join(ref, "tests/kernels/test_triton_attention.py"), ["_reference_paged_attention"])
    from freetoken.kernel.triton import attention as tattn

    golden["paged_attention"] = []
    for seed, (lens, q_lens, Hq, Hkv, D, window) in enumerate([([9, 33, 5], [9, 1, 3], 4, 2, 16, None),
                                                               ([40, 17], [2, 17], 6, 2, 8, None),
                                                               ([50, 21], [5, 1], 2, 2, 16, 12)]):
        args = paged_inputs(200 + seed, lens, q_lens, Hq, Hkv, D)
        q, k_cache, v_cache, indptr, indices, q_to_req, q_pos = args
        scale = D ** -0.5
        out = ns["_reference_paged_attention"](*args, scale, window)
        mine = plain_paged(*args, Hq // Hkv, window)
        torch.testing.assert_close(mine, out, rtol=1e-5, atol=1e-6)
        # the reference's kernel itself, in the interpreter, with its wrapper's arguments (attention.py:918-946)
        o = torch.empty_like(q)
        tattn._paged_attention_kernel[(q.shape[0], Hq)](
            q, k_cache, v_cache, o, indptr, indices, q_to_req, q_pos, scale, q,
            q.stride(0), q.stride(1), k_cache.stride(0), k_cache.stride(1), v_cache.stride(0), v_cache.stride(1),
            o.stride(0), o.stride(1), GROUP=Hq // Hkv, D=D, BLOCK_D=triton.next_power_of_2(D), BLOCK_N=32,
            SLIDING_WINDOW=window or 0, HAS_SINKS=False, num_warps=4, num_stages=2)
        torch.testing.assert_close(o, out, rtol=1e-5, atol=1e-6)
        golden["paged_attention"].append({"seed": 200 + seed, "lens": lens, "q_lens": q_lens, "Hq": Hq, "Hkv": Hkv,
                                          "D": D, "window": window, "out": lst(out), "kernel": lst(o)})


def fused_experts_oracle(golden, ref):
    ns = functions_of(os.path.join(ref, "tests/moe/test_fused_moe.py"),
                      ["_activation_and_mul", "_reference_fused_experts_decode"])
    golden["fused_experts"] = []
    for seed, (T, H, I, E, k) in enumerate([(5, 24, 12, 6, 2), (3, 16, 20, 4, 3)]):
        g = torch.Generator().manual_seed(300 + seed)
        h, w1, w2 = rand(g, T, H), rand(g, E, 2 * I, H, scale=0.3), rand(g, E, H, I, scale=0.3)
        wts = torch.rand(T, k, generator=g)
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
        out = ns["_reference_fused_experts_decode"](h, w1, w2, wts, ids, "silu")
        W = {}
        for e in range(E):
            W[f"experts.{e}.w1.weight"], W[f"experts.{e}.w3.weight"] = w1[e, :I], w1[e, I:]
            W[f"experts.{e}.w2.weight"] = w2[e]
        mine = m3_plain.routed_experts(h, ids, wts, W, "", plain_cfg(act="silu"), None)
        torch.testing.assert_close(mine, out, rtol=1e-5, atol=1e-6)
        golden["fused_experts"].append({"seed": 300 + seed, "T": T, "H": H, "I": I, "E": E, "k": k, "out": lst(out)})


def triton_norms(golden):
    from freetoken.kernel.triton import norm as tnorm

    golden["norm"] = []
    for seed, (rows, H, eps, gemma, dtype) in enumerate([(5, 48, 1e-6, True, "float32"), (4, 40, 1e-5, False, "float32"),
                                                         (6, 64, 1e-6, True, "bfloat16")]):
        g = torch.Generator().manual_seed(400 + seed)
        dt = getattr(torch, dtype)
        x, r, w = rand(g, rows, H).to(dt), rand(g, rows, H).to(dt), rand(g, H, scale=0.1).to(dt)
        fn = tnorm.gemma_rmsnorm if gemma else tnorm.rmsnorm
        y = fn(x, w, eps, out=torch.empty(rows, H))  # 32-bit output: the kernel's arithmetic, unrounded
        mine = m3_plain.rms_norm(x.float(), w.float(), eps, gemma)
        torch.testing.assert_close(mine, y, rtol=1e-6, atol=1e-7)
        # per-head form: a [tokens, heads, head_dim] view of a wider buffer, normed over head_dim
        wide = rand(g, rows, 3 * H).to(dt)
        heads = wide.view(rows, 3 * H // 8, 8)[:, :4]
        wh = rand(g, 8, scale=0.1).to(dt)
        yh = fn(heads, wh, eps, out=torch.empty(rows, 4, 8))
        mh = m3_plain.rms_norm(heads.float(), wh.float(), eps, gemma)
        torch.testing.assert_close(mh, yh, rtol=1e-6, atol=1e-7)
        # residual sum fused in: the residual is stored rounded, the norm sees the unrounded sum
        x2, r2 = x.clone(), r.clone()
        (tnorm.gemma_fused_add_rmsnorm if gemma else tnorm.fused_add_rmsnorm)(x2, r2, w, eps)
        z = x.float() + r.float()
        mz = m3_plain.rms_norm(z, w.float(), eps, gemma)
        if dtype == "bfloat16":
            assert torch.equal(chopped(z), r2.float())
            close = (chopped(mz) - x2.float()).abs() <= 2.0 ** -7 * x2.float().abs()  # one bfloat16 step
            assert close.all(), "fused add + norm differs"
            # and it is the unrounded sum that is normed: norming the stored residual gives other values
            other = chopped(m3_plain.rms_norm(r2.float(), w.float(), eps, gemma))
            assert (chopped(mz) == x2.float()).float().mean() > 0.97 > (other == x2.float()).float().mean()
        else:
            torch.testing.assert_close(z, r2, rtol=0, atol=0)
            torch.testing.assert_close(mz, x2, rtol=1e-6, atol=1e-7)
        golden["norm"].append({"seed": 400 + seed, "rows": rows, "H": H, "eps": eps, "gemma": gemma, "dtype": dtype,
                               "y": lst(y), "per_head": lst(yh), "fused_residual": lst(r2), "fused_y": lst(x2)})


def triton_rope(golden):
    from freetoken.kernel.triton import rope as trope
    from freetoken.layers.rotary import RotaryEmbedding

    golden["rope_apply"] = []
    for seed, (T, Hq, Hk, D, rd, theta, dtype) in enumerate([(7, 4, 2, 16, 8, 1e4, "float32"),
                                                             (5, 3, 1, 32, 32, 1e6, "float32"),
                                                             (6, 2, 2, 64, 16, 5e6, "bfloat16")]):
        g = torch.Generator().manual_seed(500 + seed)
        dt = getattr(torch, dtype)
        q, k = rand(g, T, Hq * D).to(dt), rand(g, T, Hk * D).to(dt)
        pos = torch.randint(0, 90, (T,), generator=g, dtype=torch.int32)
        cache = RotaryEmbedding(64, rd, 90, theta)._cos_sin_cache
        q2, k2 = q.clone(), k.clone()
        qv, kv = q2.view(T, Hq, D), k2.view(T, Hk, D)
        half = rd // 2
        grid = (triton.cdiv(T, 16), max(Hq, Hk))  # the wrapper's launch (rope.py:122-141)
        trope._rope_tiled[grid](qv, kv, pos, cache, qv.stride(0), qv.stride(1), qv.stride(2), kv.stride(0),
                                kv.stride(1), kv.stride(2), T, Hq, Hk, rd, half, HAS_K=True, INTERLEAVE=False,
                                BLOCK_DHALF=triton.next_power_of_2(half), BLOCK_SEQ=16, BLOCK_HEAD=1, num_warps=4,
                                num_stages=1)
        cos, sin = m3_plain.rope_table(rd, theta, 90, torch.float32)
        mq = m3_plain.apply_rope(q.float().view(T, Hq, D), cos[pos.long()], sin[pos.long()], rd)
        mk = m3_plain.apply_rope(k.float().view(T, Hk, D), cos[pos.long()], sin[pos.long()], rd)
        if dtype == "bfloat16":  # (the interpreter chops where the GPU rounds; allow the last bit of the sum)
            for mine, got in ((mq, qv), (mk, kv)):
                assert ((chopped(mine) - got.float()).abs() <= 2.0 ** -7 * got.float().abs()).all()
                assert (chopped(mine) == got.float()).float().mean() > 0.97
        else:
            torch.testing.assert_close(mq, qv, rtol=1e-6, atol=1e-7)
            torch.testing.assert_close(mk, kv, rtol=1e-6, atol=1e-7)
        golden["rope_apply"].append({"seed": 500 + seed, "T": T, "Hq": Hq, "Hk": Hk, "D": D, "rotary_dim": rd,
                                     "theta": theta, "dtype": dtype, "q": lst(qv), "k": lst(kv)})


def triton_activation(golden):
    from freetoken.kernel.triton import activation as tact

    tact._fast_ex2 = exact_ex2
    golden["activation"] = []
    for seed, (rows, d, act, alpha, limit, dtype) in enumerate([(5, 24, "swigluoai", 1.702, 7.0, "float32"),
                                                                (4, 40, "silu", 0.0, 0.0, "float32"),
                                                                (6, 16, "swigluoai", 1.702, 2.0, "bfloat16")]):
        g = torch.Generator().manual_seed(600 + seed)
        dt = getattr(torch, dtype)
        x = rand(g, rows, 2 * d, scale=4.0).to(dt)
        out = torch.empty(rows, d)  # 32-bit output also for bfloat16 inputs: the arithmetic, unrounded
        kind = tact.SWIGLUOAI if act == "swigluoai" else tact.SILU
        tact._act_and_mul_kernel[(rows, 1)](out, x, d, alpha, limit, ACT=kind, ENABLE_PDL=False,
                                            BLOCK_D=triton.next_power_of_2(d), num_warps=4, num_stages=3)
        mine = m3_plain.activation(x[:, :d].float(), x[:, d:].float(), act, alpha, limit)
        torch.testing.assert_close(mine, out, rtol=2e-6, atol=1e-6)
        golden["activation"].append({"seed": 600 + seed, "rows": rows, "d": d, "act": act, "alpha": alpha,
                                     "limit": limit, "dtype": dtype, "out": lst(out)})


def config_and_state_dict(golden, ref):
    ns = functions_of(os.path.join(ref, "tests/models/test_minimax_m3.py"), ["_Cfg", "_hf_config", "_hf_config_native"])
    from freetoken.distributed.info import set_tp_info
    from freetoken.layers.rotary import set_rope_device
    from freetoken.models import create_model
    from freetoken.models.minimax_m3.config import parse_config

    def as_dict(cfg):
        out = dict(vars(cfg))
        out["text_config"] = dict(vars(cfg.text_config))
        return out

    def facts(mc):
        a = mc.m3_args
        return {"num_layers": mc.num_layers, "hidden_size": mc.hidden_size, "num_qo_heads": mc.num_qo_heads,
                "num_kv_heads": mc.num_kv_heads, "head_dim": mc.head_dim, "vocab_size": mc.vocab_size,
                "rotary_dim": mc.rotary_config.rotary_dim, "rope_theta": mc.rotary_config.base,
                "max_position": mc.rotary_config.max_position, "rms_norm_eps": mc.rms_norm_eps,
                "hidden_act": mc.hidden_act, "swiglu_alpha": mc.hidden_act_alpha, "swiglu_limit": mc.swiglu_limit,
                "num_experts": mc.num_experts, "num_experts_per_tok": mc.num_experts_per_tok,
                "moe_intermediate_size": mc.moe_intermediate_size, "dense_intermediate_size": mc.intermediate_size,
                "shared_intermediate_size": mc.shared_expert_intermediate_size, "n_shared_experts": mc.n_shared_experts,
                "routed_scaling_factor": mc.routed_scaling_factor, "tie_word_embeddings": mc.tie_word_embeddings,
                "moe_layer_ids": list(a.moe_layer_ids), "sparse_layer_ids": list(a.sparse_layer_ids),
                "index_dim": a.index_dim, "num_index_heads": a.num_index_heads, "topk_blocks": a.topk_blocks,
                "block_size": a.block_size, "init_blocks": a.init_blocks, "local_blocks": a.local_blocks}

    for k in ("FREETOKEN_M3_MAX_LAYERS", "FREETOKEN_M3_SPARSE"):
        os.environ.pop(k, None)
    raw_cfg, native_cfg = ns["_hf_config"](), ns["_hf_config_native"]()
    raw_facts, native_facts = facts(parse_config(raw_cfg)), facts(parse_config(native_cfg))
    assert raw_facts == native_facts
    golden["config"] = {"raw": as_dict(raw_cfg), "native": as_dict(native_cfg), "parsed": raw_facts}

    # the first five layers on the meta device, in the serving dtype, without resident quantisation
    os.environ["FREETOKEN_M3_ATTN_MXFP8"] = "0"
    os.environ["FREETOKEN_M3_MLP_MXFP8"] = "0"
    set_tp_info(0, 1)
    set_rope_device(torch.device("cpu"))
    small = ns["_hf_config"](5)
    small.text_config.max_position_embeddings = 4096  # (only sizes the rope table, which is no weight)
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device("meta"):
            model = create_model(parse_config(small))
        sd = {k: [list(v.shape), str(v.dtype).replace("torch.", "")] for k, v in model.state_dict().items()}
    finally:
        torch.set_default_dtype(torch.float32)
    golden["state_dict"] = {"config": as_dict(small), "tensors": sd}


def chunked_prefill_drive(golden, ref):
    """The reference's managers driven as its regression test drives them, with the cache type that
    keeps nothing after a request (the counterpart of this engine's cache): pages free after each
    iteration of the overlapped loop."""
    from freetoken.core import Context, SamplingParams, get_global_ctx, set_global_ctx
    from freetoken.scheduler.cache import CacheManager
    from freetoken.scheduler.decode import DecodeManager
    from freetoken.scheduler.prefill import ChunkedReq, PrefillManager
    from freetoken.scheduler.table import TableManager
    from freetoken.scheduler.utils import PendingReq

    CHUNK, WIDTH, MAX_RUNNING, PAGES = 8, 64, 4, 64
    try:
        get_global_ctx()
    except AssertionError:
        set_global_ctx(Context(page_size=1))
    golden["chunked_prefill"] = []
    for n_chunks, max_tokens in [(4, 4), (3, 9)]:
        pt = torch.zeros((MAX_RUNNING + 1, WIDTH), dtype=torch.int32)
        cm = CacheManager(num_pages=PAGES, page_size=1, page_table=pt, type="naive")
        tm = TableManager(max_running_reqs=MAX_RUNNING, page_table=pt)
        pm = PrefillManager(cm, tm, DecodeManager(page_size=1))
        pm.pending_list = [PendingReq(uid=7, input_ids=torch.arange(n_chunks * CHUNK, dtype=torch.int32),
                                      sampling_params=SamplingParams(max_tokens=max_tokens))]
        trail, last_batch, final_req = [], None, None
        while pm.runnable or last_batch is not None:
            batch = pm.schedule_next_batch(CHUNK)
            scheduled = 0 if batch is None else sum(r.extend_len for r in batch.reqs)
            if batch is not None:
                cm.allocate_paged(batch.reqs)
                for r in batch.reqs:
                    r.complete_one()
            if last_batch is not None:
                for r in last_batch.reqs:
                    if not isinstance(r, ChunkedReq):
                        cm.cache_req(r, finished=False)
                        final_req = r
            last_batch = batch
            trail.append({"scheduled": scheduled, "free": len(cm.free_slots)})
        cm.cache_req(final_req, finished=True)
        tm.free(final_req.table_idx)
        cm.check_integrity()
        golden["chunked_prefill"].append({"chunks": n_chunks, "chunk": CHUNK, "pages": PAGES, "max_tokens": max_tokens,
                                          "trail": trail, "free_at_end": len(cm.free_slots)})


def main(reference_root: str) -> None:
    stub = tempfile.mkdtemp()
    os.makedirs(os.path.join(stub, "flashlib", "kernels"))
    open(os.path.join(stub, "flashlib", "__init__.py"), "w").close()
    open(os.path.join(stub, "flashlib", "kernels", "__init__.py"), "w").close()
    with open(os.path.join(stub, "flashlib", "kernels", "slot_cache.py"), "w") as f:
        f.write("N_STATS = 8\nclass Stat: ...\ndef lru_ensure(*a, **k): raise NotImplementedError\n")
    sys.path.insert(0, stub)
    sys.path.insert(0, os.path.join(reference_root, "python"))

    golden: dict = {}
    rope_and_router(golden)
    sparse_oracles(golden, reference_root)
    paged_attention_oracle(golden, reference_root)
    fused_experts_oracle(golden, reference_root)
    triton_norms(golden)
    triton_rope(golden)
    triton_activation(golden)
    config_and_state_dict(golden, reference_root)
    chunked_prefill_drive(golden, reference_root)
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(golden, f)
    print("the plain implementation agrees with the reference's CPU-runnable pieces: " + ", ".join(golden))
    print(f"golden.json written ({os.path.getsize(os.path.join(HERE, 'golden.json')) // 1024} KB)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
