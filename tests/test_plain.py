"""The plain implementation itself: internal consistency, and agreement with the outputs of the
reference's CPU-runnable pieces recorded in tests/golden/golden.json."""

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
