"""The step function, cache and batching logic on the CPU, with the plain PyTorch statements of
the kernels (tests/kernel_refs.py) standing in for the CUDA kernels: every way of cutting and
batching the work gives the plain implementation's logits."""

import pytest
import torch

import kernel_refs
from helpers import (make_engine, mixed_schedule, model_folder, replay_cuts, replay_mixed, replay_whole,
                     tokens_for)
from plain.m3_plain import PlainM3
from tiny_configs import ALL

TOL = dict(rtol=1e-4, atol=2e-5)
PAGE = {"A": 4, "B": 8, "C": 4, "D": 4}


@pytest.fixture
def cpu_ops(monkeypatch):
    kernel_refs.install(monkeypatch)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_cuts_and_batches_agree_with_the_plain_model(name, cpu_ops, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainM3(folder)
    V = plain.cfg.vocab
    eng = make_engine(folder, "float32", "cpu", PAGE[name], pages=40)
    toks = tokens_for(V, 70, 11)
    ref = plain.logits(toks)
    torch.testing.assert_close(replay_whole(eng, "w", toks), ref, **TOL)
    torch.testing.assert_close(replay_cuts(eng, "d", toks, [38]), ref, **TOL)  # last 32 one by one
    torch.testing.assert_close(replay_cuts(eng, "c", toks, [7, 2, 13, 2, 5, 3, 2, 11, 2]), ref, **TOL)
    eng.cache.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_mixed_steps_with_few_pages(name, cpu_ops, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainM3(folder)
    V = plain.cfg.vocab
    lengths = {"r0": 45, "r1": 60, "r2": 38, "r3": 52, "r4": 41, "r5": 47}
    seqs = {r: tokens_for(V, n, i) for i, (r, n) in enumerate(lengths.items())}
    P = PAGE[name]
    pages = 4 * (-(-64 // P))  # room for four live requests of up to 64 tokens
    eng = make_engine(folder, "float32", "cpu", P, pages=pages)
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=3))
    for r, toks in seqs.items():
        torch.testing.assert_close(got[r], plain.logits(toks), **TOL)
    pool = eng.cache.paged[0].pool
    assert pool.handed_out > pool.num_pages, "the trace was meant to use pages again"
    assert pool.free_count == pool.num_pages
