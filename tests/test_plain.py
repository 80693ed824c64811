"""The plain implementation itself: internal consistency, and agreement with the outputs of the
reference's CPU-runnable pieces recorded in tests/golden/golden.json (its rope table and router, its
own PyTorch oracles for block-sparse attention, paged attention and fused experts, and its Triton
norm, rope, activation and paged-attention kernels run under Triton's CPU interpreter;
tests/golden/make_golden.py says how each was produced)."""

import json
import os
import types

import pytest
import torch

from helpers import model_folder, tokens_for
from plain import m3_plain
from plain.m3_plain import PlainM3
from helpers import NEAR_TIE
from tiny_configs import ALL, TINY_D


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_causal_and_deterministic(name, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    m = PlainM3(folder)
    toks = tokens_for(m.cfg.vocab, 30, 2)
    full = m.logits(toks)
    assert full.shape == (30, m.cfg.vocab)
    torch.testing.assert_close(m.logits(toks[:17]), full[:17], rtol=1e-5, atol=1e-6)
    m64 = PlainM3(folder, dtype=torch.float64)
    torch.testing.assert_close(m64.logits(toks).float(), full, rtol=1e-4, atol=1e-5)
    mb = PlainM3(folder, rounding="bfloat16")
    sure = m.router_margins(toks) > NEAR_TIE  # elsewhere rounding may pick another expert
    assert sure.float().mean() > 0.5
    assert (mb.logits(toks) - full)[sure].abs().max() < 0.03


def test_sparse_attention_equals_dense_when_every_block_is_chosen(tmp_path_factory):
    """Reference property: tests/kernels/test_minimax_m3_sparse.py:279-311."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "D", TINY_D)
    m = PlainM3(folder)
    toks = tokens_for(m.cfg.vocab, 40, 3)
    short = m.logits(toks[:24])  # 3 blocks of 8, topk 3: nothing is dropped
    m.cfg.sparse_layers = [False] * m.cfg.layers
    dense = m.logits(toks)
    torch.testing.assert_close(short, dense[:24], rtol=1e-5, atol=1e-6)
    m.cfg.sparse_layers = [False, True, True]
    long = m.logits(toks)
    assert (long[30:] - dense[30:]).abs().max() > 1e-4  # beyond topk * block the selection bites


def test_block_selection_rules():
    T, block = 40, 8
    iq = torch.zeros(T, 1, 4)
    ik = torch.zeros(T, 4)
    iq[:, 0, 0] = 1.0
    ik[3, 0] = 5.0   # block 0 scores high
    ik[20, 0] = 3.0  # block 2 next
    allowed = m3_plain.sparse_block_selection(iq, ik, block, topk=2, local=1, init=0)
    # query 39: local block 4 is forced, then the best of the rest is block 0
    assert allowed[0, 39, 32:40].all() and allowed[0, 39, 0:8].all() and not allowed[0, 39, 8:32].any()
    # query 5 sees one block only
    assert allowed[0, 5, 0:8].all() and not allowed[0, 5, 8:].any()


def test_golden_rope_and_router():
    with open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")) as f:
        golden = json.load(f)
    for g in golden["rope"]:
        cos, sin = m3_plain.rope_table(g["rotary_dim"], g["theta"], g["positions"], torch.float32)
        table = torch.cat((cos, sin), -1)
        for p, row in g["rows"].items():
            assert torch.equal(table[int(p)], torch.tensor(row))
    for g in golden["router"]:
        gen = torch.Generator().manual_seed(g["seed"])
        h = torch.randn(g["T"], g["H"], generator=gen)
        w = torch.randn(g["E"], g["H"], generator=gen) * 0.1
        b = torch.randn(g["E"], generator=gen) * 0.01
        cfg = types.SimpleNamespace(scoring="sigmoid", top_k=g["k"], scale=g["scale"])
        wts, ids = m3_plain.router(h, w, b, cfg)
        assert ids.tolist() == g["ids"]
        torch.testing.assert_close(wts, torch.tensor(g["weights"]), rtol=1e-6, atol=1e-7)


def test_sampling_reference():
    logits = torch.tensor([0.0, 2.0, 1.0, 2.0, -1.0])
    assert m3_plain.sample_reference(logits, 1.0, 1, 1.0, 0.9) == 1  # top-1 keeps the tie's values
    assert m3_plain.sample_reference(logits, 1.0, -1, 1.0, 0.0) == 0
    assert m3_plain.sample_reference(logits, 1.0, -1, 1.0, 0.999999) == 4
    draws = {m3_plain.sample_reference(logits, 1.0, -1, 0.5, u / 10) for u in range(10)}
    assert draws <= {1, 3}


# ------------------------------------------------------------------------------------------------
# The reference's own oracles and interpreted kernels (inputs are re-made from the recorded seeds with
# the same draws as tests/golden/make_golden.py).
def _golden():
    with open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")) as f:
        return json.load(f)


def _rand(gen, *shape, scale=1.0):
    return torch.randn(*shape, generator=gen) * scale


def _chopped(t):
    """float32 -> bfloat16 by dropping the low 16 bits, as Triton's CPU interpreter stores bfloat16."""
    return (t.float().contiguous().view(torch.int32) & ~0xFFFF).view(torch.float32)


def _cfg(**kw):
    base = dict(act="silu", alpha=1.702, limit=7.0, top_k=2, scale=1.0, scoring="sigmoid", bias=True, n_shared=0)
    base.update(kw)
    return types.SimpleNamespace(**base)


def test_golden_block_sparse_selection_and_attention():
    """ref_block_scores / ref_select / ref_sparse_attend of the reference's tests, blocks of 128."""
    for g in _golden()["sparse"]:
        gen = torch.Generator().manual_seed(g["seed"])
        T, Hi, group, D, BLK = g["T"], g["Hi"], g["group"], g["D"], g["block"]
        iq, ik = _rand(gen, T, Hi, D), _rand(gen, T, D)
        q, k, v = _rand(gen, T, Hi * group, D), _rand(gen, T, Hi, D), _rand(gen, T, Hi, D)
        margins = []
        allowed = m3_plain.sparse_block_selection(iq, ik, BLK, g["topk"], g["local"], g["init"], margins)
        bscore = [x[1] for x in margins if x[0] == "scores"][0]
        for h in range(Hi):
            for i, t in enumerate(g["tokens"]):
                want = torch.tensor([float("-inf") if x is None else x for x in g["scores"][h][i]])
                torch.testing.assert_close(bscore[h, t], want, rtol=1e-5, atol=1e-6)
                chosen = sorted({int(p) // BLK for p in allowed[h, t].nonzero().view(-1) if int(p) <= t})
                assert chosen == g["selection"][h][i], (g["seed"], h, t)
        out = m3_plain.causal_attention(q, k, v, group, None, allowed)
        torch.testing.assert_close(out[g["tokens"]], torch.tensor(g["out"]), rtol=1e-5, atol=1e-6)


def test_golden_paged_attention():
    """_reference_paged_attention of the reference's tests and its Triton kernel (interpreted): keys in
    scattered slots, several requests, queries at the end of their requests, one case with a window."""
    for g in _golden()["paged_attention"]:
        gen = torch.Generator().manual_seed(g["seed"])
        lens, q_lens, Hq, Hkv, D = g["lens"], g["q_lens"], g["Hq"], g["Hkv"], g["D"]
        total = sum(lens)
        perm = torch.randperm(total + 7, generator=gen)[:total]
        k_cache, v_cache = _rand(gen, total + 7, Hkv, D), _rand(gen, total + 7, Hkv, D)
        n_q = sum(q_lens)
        q = _rand(gen, n_q, Hq, D)
        got, row, start = torch.empty(n_q, Hq, D), 0, 0
        for n, ql in zip(lens, q_lens):
            slots = perm[start:start + n]
            K, V = k_cache[slots], v_cache[slots]
            full_q = torch.zeros(n, Hq, D)
            full_q[n - ql:] = q[row:row + ql]
            allowed = None
            if g["window"] is not None:
                p = torch.arange(n)
                allowed = (p[None, :] + g["window"] > p[:, None]).expand(Hkv, n, n)
            got[row:row + ql] = m3_plain.causal_attention(full_q, K, V, Hq // Hkv, None, allowed)[n - ql:]
            row, start = row + ql, start + n
        torch.testing.assert_close(got, torch.tensor(g["out"]), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got, torch.tensor(g["kernel"]), rtol=1e-5, atol=1e-6)


def test_golden_fused_experts():
    """_reference_fused_experts_decode of the reference's tests: gate_up rows gate then up, the route
    weight on the second product, the sum over routes."""
    for g in _golden()["fused_experts"]:
        gen = torch.Generator().manual_seed(g["seed"])
        T, H, I, E, k = g["T"], g["H"], g["I"], g["E"], g["k"]
        h, w1, w2 = _rand(gen, T, H), _rand(gen, E, 2 * I, H, scale=0.3), _rand(gen, E, H, I, scale=0.3)
        wts = torch.rand(T, k, generator=gen)
        ids = torch.stack([torch.randperm(E, generator=gen)[:k] for _ in range(T)])
        W = {}
        for e in range(E):
            W[f"experts.{e}.w1.weight"], W[f"experts.{e}.w3.weight"] = w1[e, :I], w1[e, I:]
            W[f"experts.{e}.w2.weight"] = w2[e]
        mine = m3_plain.routed_experts(h, ids, wts, W, "", _cfg(act="silu"), None)
        torch.testing.assert_close(mine, torch.tensor(g["out"]), rtol=1e-5, atol=1e-6)


def test_golden_norms():
    """The reference's Triton RMSNorm kernels (interpreted): Gemma and plain form, whole rows and
    per-head rows of a wider buffer, and the fused residual sum, where the stored residual is rounded
    but the norm is taken of the unrounded sum."""
    for g in _golden()["norm"]:
        gen = torch.Generator().manual_seed(g["seed"])
        rows, H, eps, gemma = g["rows"], g["H"], g["eps"], g["gemma"]
        dt = getattr(torch, g["dtype"])
        x, r, w = _rand(gen, rows, H).to(dt), _rand(gen, rows, H).to(dt), _rand(gen, H, scale=0.1).to(dt)
        torch.testing.assert_close(m3_plain.rms_norm(x.float(), w.float(), eps, gemma), torch.tensor(g["y"]),
                                   rtol=1e-6, atol=1e-7)
        wide = _rand(gen, rows, 3 * H).to(dt)
        heads = wide.view(rows, 3 * H // 8, 8)[:, :4]
        wh = _rand(gen, 8, scale=0.1).to(dt)
        torch.testing.assert_close(m3_plain.rms_norm(heads.float(), wh.float(), eps, gemma),
                                   torch.tensor(g["per_head"]), rtol=1e-6, atol=1e-7)
        z = x.float() + r.float()
        mz = m3_plain.rms_norm(z, w.float(), eps, gemma)
        fused_y, fused_r = torch.tensor(g["fused_y"]), torch.tensor(g["fused_residual"])
        if g["dtype"] == "bfloat16":
            assert torch.equal(_chopped(z), fused_r)
            assert ((_chopped(mz) - fused_y).abs() <= 2.0 ** -7 * fused_y.abs()).all()
            from_stored = _chopped(m3_plain.rms_norm(fused_r, w.float(), eps, gemma))
            assert (_chopped(mz) == fused_y).float().mean() > 0.97 > (from_stored == fused_y).float().mean()
        else:
            assert torch.equal(z, fused_r)
            torch.testing.assert_close(mz, fused_y, rtol=1e-6, atol=1e-7)


def test_golden_rope_application():
    """The reference's Triton rope kernel (interpreted) on q and k at scattered positions: partial and
    full rotary widths, NeoX pairing, dims past the rotary width untouched."""
    for g in _golden()["rope_apply"]:
        gen = torch.Generator().manual_seed(g["seed"])
        T, Hq, Hk, D, rd = g["T"], g["Hq"], g["Hk"], g["D"], g["rotary_dim"]
        dt = getattr(torch, g["dtype"])
        q, k = _rand(gen, T, Hq * D).to(dt), _rand(gen, T, Hk * D).to(dt)
        pos = torch.randint(0, 90, (T,), generator=gen, dtype=torch.int32).long()
        cos, sin = m3_plain.rope_table(rd, g["theta"], 90, torch.float32)
        for src, heads, want in ((q, Hq, g["q"]), (k, Hk, g["k"])):
            u = src.float().view(T, heads, D)
            mine, want = m3_plain.apply_rope(u, cos[pos], sin[pos], rd), torch.tensor(want)
            if g["dtype"] == "bfloat16":
                assert ((_chopped(mine) - want).abs() <= 2.0 ** -7 * want.abs()).all()
                assert (_chopped(mine) == want).float().mean() > 0.97
            else:
                torch.testing.assert_close(mine, want, rtol=1e-6, atol=1e-7)
            assert torch.equal(want[..., rd:], u[..., rd:])  # dims past the rotary width pass through


def test_golden_activations():
    """The reference's Triton activation kernel (interpreted, exact exp2 in place of ex2.approx): silu and
    the clamped swigluoai with its (up + 1), on values beyond the clamp."""
    for g in _golden()["activation"]:
        gen = torch.Generator().manual_seed(g["seed"])
        d = g["d"]
        x = _rand(gen, g["rows"], 2 * d, scale=4.0).to(getattr(torch, g["dtype"])).float()
        mine = m3_plain.activation(x[:, :d], x[:, d:], g["act"], g["alpha"], g["limit"])
        torch.testing.assert_close(mine, torch.tensor(g["out"]), rtol=2e-6, atol=1e-6)
