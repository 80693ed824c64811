"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16: each request
alone and whole; most of it in one step and the last 32 tokens one by one; portions of changing
size down to two tokens; up to four live requests mixed, with so few pages that they are used
again; long decoding; the first tokens of a sequence; generation through the entry point."""

from __future__ import annotations

import pytest
import torch

from freetoken_b200 import LLM, SamplingParams
from freetoken_b200.engine.engine import StepEntry
from freetoken_b200.sampling import uniform_for
from helpers import (BF16_TOL, F32_TOL, assert_bf16_close, clear_tokens, make_engine, mixed_schedule, model_folder,
                     replay_cuts, replay_mixed, replay_whole, tokens_for)
from plain.m3_plain import PlainM3, sample_reference
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
PAGE = {"A": 4, "B": 8, "C": 16, "D": 4, "E": 16}
CONFIGS = ["A", "B", "C", "D"]
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def world(tmp_path_factory):
    """Model folders, plain models and engines, made once per module."""
    root = tmp_path_factory.mktemp("models")
    cache = {}

    def get(name, dtype=None, pages=48, **kw):
        if ("plain", name) not in cache:
            folder = model_folder(root, name, ALL[name])
            cache[("plain", name)] = (folder, PlainM3(folder))
        folder, plain = cache[("plain", name)]
        if dtype is None:
            return folder, plain, None
        key = (name, dtype, pages, tuple(sorted(kw.items())))
        if key not in cache:
            cache[key] = make_engine(folder, dtype, "cuda:0", PAGE[name], pages, **kw)
        return folder, plain, cache[key]

    return get


SPARSE = {"D"}  # configurations with block-sparse layers: bfloat16 is compared on a clear prefix


def check(got, ref, dtype, margins, what, name=""):
    if dtype == "float32":
        torch.testing.assert_close(got, ref[: got.shape[0]], **F32_TOL, msg=lambda m: f"{what}: {m}")
    else:
        assert_bf16_close(got, ref, margins, what, prefix_only=name in SPARSE, name=name)


def sequence(plain, name, n, seed):
    return clear_tokens(plain, n, seed, 30) if name in SPARSE else tokens_for(plain.cfg.vocab, n, seed)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_whole_decode_and_portions(name, dtype, world):
    _, plain, eng = world(name, dtype)
    toks = sequence(plain, name, 90, 21)
    ref, margins = plain.logits(toks), plain.router_margins(toks)
    check(replay_whole(eng, "whole", toks), ref, dtype, margins, "whole", name)
    check(replay_cuts(eng, "tail", toks, [58]), ref, dtype, margins, "last 32 one by one", name)
    check(replay_cuts(eng, "cuts", toks, [7, 2, 13, 2, 5, 3, 2, 17, 2, 9, 2, 2, 11]), ref, dtype, margins,
          "portions of changing size", name)
    eng.cache.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_mixed_requests_reuse_pages(name, dtype, world):
    P = PAGE[name]
    _, plain, eng = world(name, dtype, pages=4 * (-(-64 // P)))
    lengths = {"r0": 45, "r1": 64, "r2": 38, "r3": 52, "r4": 41, "r5": 63, "r6": 34}
    seqs = {r: sequence(plain, name, n, 100 + 40 * i) for i, (r, n) in enumerate(lengths.items())}
    pool = eng.cache.paged[0].pool
    before = pool.handed_out
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=5))
    for r, toks in seqs.items():
        check(got[r], plain.logits(toks), dtype, plain.router_margins(toks), f"mixed {r}", name)
    assert pool.handed_out - before > pool.num_pages, "pages were meant to be used again"
    assert pool.free_count == pool.num_pages


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(dtype, world):
    _, plain, eng = world("A", dtype, pages=80)
    toks = tokens_for(plain.cfg.vocab, 300, 33)
    ref, margins = plain.logits(toks), plain.router_margins(toks)
    check(replay_cuts(eng, "long", toks, [3]), ref, dtype, margins, "297 tokens decoded one by one")
    assert eng.graphs, "decode steps were meant to run from CUDA graphs"
    for n in (1, 2, 3):
        check(replay_whole(eng, f"first{n}", toks[:n]), ref, dtype, margins, f"first {n} tokens")
    check(replay_cuts(eng, "ones", toks[:5], [1, 1, 1, 1, 1]), ref, dtype, margins, "from the first token on")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_steps_on_the_tensor_core_attention(dtype, world):
    """Heads of 128 and pages of 16: steps of 128 tokens and more run the tcgen05 attention kernel in
    bfloat16 (the other kernels otherwise).  Whole prompts, a prompt in two long portions, and long
    portions beside decoded tokens of other requests, all against the plain model."""
    _, plain, eng = world("E", dtype, pages=64, max_step=320)
    V = plain.cfg.vocab
    toks = tokens_for(V, 300, 77)
    ref, margins = plain.logits(toks), plain.router_margins(toks)
    check(replay_whole(eng, "w", toks), ref, dtype, margins, "300 tokens whole")
    check(replay_cuts(eng, "c", toks, [170, 129]), ref, dtype, margins, "two long portions and one token")
    seqs = {"a": tokens_for(V, 200, 78), "b": tokens_for(V, 150, 79), "c": tokens_for(V, 40, 80)}
    sched = [{"c": 30}, {"a": 190, "c": 1}, {"b": 140, "c": 1, "a": 1}] + [{"a": 1, "b": 1, "c": 1}] * 10
    got = replay_mixed(eng, seqs, sched)
    for r, t in seqs.items():
        check(got[r], plain.logits(t), dtype, plain.router_margins(t), f"mixed with long portions {r}")
    if dtype == "bfloat16":
        from freetoken_b200.kernels import ops

        assert ops.attention_tc_fits(128, 16, 3) and ops.read_status() == 0


def test_long_steps_on_the_attention_kernel_with_two_query_tiles(world, monkeypatch):
    """The same long steps on the tcgen05 kernel that gives a CTA two query tiles (the engine sends steps
    of a thousand tokens and more there; here every long step): whole, in portions, beside decoded tokens."""
    import freetoken_b200.parts.attention as attention

    monkeypatch.setattr(attention, "TC_PAIR_MIN_TOKENS", 128)
    _, plain, eng = world("E", "bfloat16", pages=64, max_step=320)
    V = plain.cfg.vocab
    toks = tokens_for(V, 300, 77)
    ref, margins = plain.logits(toks), plain.router_margins(toks)
    check(replay_whole(eng, "w", toks), ref, "bfloat16", margins, "300 tokens whole")
    check(replay_cuts(eng, "c", toks, [170, 129]), ref, "bfloat16", margins, "two long portions and one token")
    seqs = {"a": tokens_for(V, 200, 78), "b": tokens_for(V, 150, 79), "c": tokens_for(V, 40, 80)}
    sched = [{"c": 30}, {"a": 190, "c": 1}, {"b": 140, "c": 1, "a": 1}] + [{"a": 1, "b": 1, "c": 1}] * 10
    got = replay_mixed(eng, seqs, sched)
    for r, t in seqs.items():
        check(got[r], plain.logits(t), "bfloat16", plain.router_margins(t), f"mixed with long portions {r}")
    from freetoken_b200.kernels import ops

    assert ops.read_status() == 0
    assert attention.attention_tile_rows(torch.bfloat16, False, 3, 300, 128, 16) == 256


def test_decode_over_a_long_context_on_the_tensor_core_attention(world, monkeypatch):
    """Decode steps run the 16-row mma.sync kernel below a length of the longest request and the tcgen05
    kernel in its form for few rows above it (the threshold is 0 by default: always the tcgen05 kernel where it fits; it is
    raised here so that a short test crosses it): tokens decoded one by one before and after the
    switch, from CUDA graphs, against the plain model."""
    from freetoken_b200.parts import attention

    monkeypatch.setattr(attention, "TC_MIN_DECODE_SPAN", 256)
    _, plain, eng = world("E", "bfloat16", pages=64, max_step=320)
    toks = tokens_for(plain.cfg.vocab, 290, 91)
    ref, margins = plain.logits(toks), plain.router_margins(toks)
    check(replay_cuts(eng, "long-decode", toks, [100]), ref, "bfloat16", margins, "190 tokens decoded past the switch")
    import ast

    forms = {tuple(ast.literal_eval(plan)[i] for i in (2, 6)) for key in eng.graphs for plan in key[2]}
    assert {False, True} <= {f[1] for f in forms}, "the two kernels were meant to get their own graphs"


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_of_decodes_matches_each_alone(dtype, world):
    """Four requests decode together (one graph replay per step); each must see only its own cache."""
    _, plain, eng = world("B", dtype, pages=60)
    V = plain.cfg.vocab
    seqs = {f"d{i}": tokens_for(V, 40 + 3 * i, 200 + i) for i in range(4)}
    sched = [{r: 9 + 2 * i for i, r in enumerate(seqs)}] + [{r: 1 for r in seqs}] * 45
    got = replay_mixed(eng, seqs, sched)
    for r, toks in seqs.items():
        check(got[r], plain.logits(toks), dtype, plain.router_margins(toks), f"batched decode {r}")


def test_graphs_and_eager_steps_agree(world):
    folder, plain, eng = world("A", "float32")
    eager = make_engine(folder, "float32", "cuda:0", PAGE["A"], 48, cuda_graph=False)
    toks = tokens_for(plain.cfg.vocab, 40, 9)
    a = replay_cuts(eng, "g", toks, [8])
    b = replay_cuts(eager, "g", toks, [8])
    assert eng.graphs and not eager.graphs
    torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-6)


def test_step_refuses_bad_input_and_leaks_nothing(world):
    from freetoken_b200.errors import CacheError, SchedulerError

    _, plain, eng = world("A", "float32", pages=6)
    with pytest.raises(SchedulerError, match="token id"):
        eng.step([StepEntry("x", [1, 256], [0])])
    with pytest.raises(SchedulerError, match="wanted place"):
        eng.step([StepEntry("x", [1, 2], [2])])
    eng.step([StepEntry("x", list(range(20)), [])])
    with pytest.raises(CacheError, match="out of pages"):
        eng.step([StepEntry("y", list(range(8)), [])])
    eng.cache.check()
    assert eng.length("x") == 20
    out = eng.step([StepEntry("x", [5], [0])])  # the engine still works after the refusal
    assert out.logits.shape == (1, 256)
    eng.close("x")
    assert not eng.is_open("y")  # the refused step undid the open it had done
    assert eng.cache.free_request_slots() == eng.config.max_running_req
    assert eng.cache.paged[0].pool.free_count == 6


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, world):
    folder, plain, _ = world("A")
    V = plain.cfg.vocab
    prompts = [tokens_for(V, n, 300 + n) for n in (5, 9, 17)]
    llm = LLM(folder, dtype=dtype, page_size=4, num_page_override=40, max_step_tokens=16,
              max_extend_tokens=16)
    outs = llm.generate(prompts, SamplingParams(max_tokens=8))
    for p, o in zip(prompts, outs):
        assert o["finish_reason"] == "length" and len(o["token_ids"]) == 8
        toks = list(p)
        for got in o["token_ids"]:
            logits = plain.logits(toks)[-1]
            top2 = torch.topk(logits, 2).values
            if dtype == "float32" or top2[0] - top2[1] > 0.05:
                assert got == int(torch.argmax(logits))
            toks.append(got)  # follow the engine's own choice where the plain model has a near-tie


def test_temperature_generation_is_seeded(world):
    folder, plain, _ = world("B")
    V = plain.cfg.vocab
    prompts = [tokens_for(V, n, 400 + n) for n in (3, 11, 23, 40)]
    llm = LLM(folder, dtype="float32", page_size=8, num_page_override=40, max_step_tokens=7,
              max_extend_tokens=7, seed=11)
    sp = SamplingParams(temperature=0.8, max_tokens=12)
    a = llm.generate(prompts, sp)
    b = llm.generate(prompts[::-1], sp)[::-1]  # other batch composition and order of arrival
    for i, (x, y) in enumerate(zip(a, b)):
        assert len(x["token_ids"]) == 12
    # request ids differ between the two calls (they follow the order of arrival), so compare
    # with the plain sampler instead: same seed, same request id, same step -> same draw
    toks = list(prompts[2])
    for step, got in enumerate(a[2]["token_ids"]):
        want = sample_reference(plain.logits(toks)[-1], 0.8, -1, 1.0, uniform_for(11, 2, step))
        assert got == want
        toks.append(got)
    again = llm.generate(prompts, sp)
    assert [x["token_ids"] for x in again] == [x["token_ids"] for x in a]


def test_kernels_ran_and_the_library_is_loaded(world):
    from freetoken_b200.kernels import library, ops

    _, plain, eng = world("A", "bfloat16")
    before = ops.launch_count()
    eng.step([StepEntry("k", [1, 2, 3], [2])])
    eng.close("k")
    assert ops.launch_count() - before > 12
    path = library.library_path()
    assert path and path.endswith(".so")
    with open("/proc/self/maps") as f:
        assert any(path in line for line in f)


@pytest.mark.parametrize("unit,code", [(0, 103), (1, 7)])
def test_a_given_up_wait_reaches_the_caller_as_an_error(unit, code, world):
    """The tensor-core kernels bound every wait and leave a code in a status word when one runs out.
    Here the word is written from the host (no wait is made to run out): the engine's check raises
    ``KernelError`` naming the code, the word is cleared by the read, and the engine goes on working."""
    from freetoken_b200.errors import KernelError
    from freetoken_b200.kernels import ops

    _, plain, eng = world("A", "bfloat16")
    eng.check_kernels()  # clean to begin with
    ops.debug_set_status(unit, code)
    with pytest.raises(KernelError, match=f"status {code}"):
        eng.check_kernels()
    eng.check_kernels()  # reading cleared it
    assert ops.read_status() == 0
    # the first step of a fresh engine looks at the word as well
    fresh = make_engine(world("A")[0], "bfloat16", "cuda:0", 4, 16)
    ops.debug_set_status(unit, code)
    with pytest.raises(KernelError, match="gave up waiting"):
        fresh.step([StepEntry("s", [1, 2, 3], [2])])
    out = fresh.step([StepEntry("s", [4], [0])])
    assert torch.isfinite(out.logits).all()
    fresh.close("s")
    with pytest.raises(KernelError, match="unit must be"):
        ops.debug_set_status(5, 1)
