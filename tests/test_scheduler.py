"""The scheduler's decisions, on the CPU (kernels replaced by their plain statements): admission,
portions under the token budget, mixed steps, finishing and freeing, what happens when the
cache is too small."""

import pytest
import torch

import kernel_refs
from freetoken_b200.engine.scheduler import Scheduler
from freetoken_b200.sampling import Sampler, SamplingParams, uniform_for
from helpers import make_engine, model_folder, tokens_for
from plain.m3_plain import PlainM3, sample_reference
from tiny_configs import TINY_A, TINY_B


@pytest.fixture
def setup(monkeypatch, tmp_path_factory):
    kernel_refs.install(monkeypatch)

    def make(raw=TINY_A, name="A", pages=40, page=4, max_step=16, reqs=4, eos=()):
        folder = model_folder(tmp_path_factory.getbasetemp(), name, raw)
        eng = make_engine(folder, "float32", "cpu", page, pages, max_step=max_step, reqs=reqs)
        sampler = Sampler(eng.device, eng.spec.vocab_size, reqs)
        return Scheduler(eng, sampler, eos), PlainM3(folder)

    return make


def test_portions_respect_the_budget_and_mix_with_decodes(setup):
    sched, plain = setup(max_step=16)
    V = plain.cfg.vocab
    prompts = {0: tokens_for(V, 5, 0), 1: tokens_for(V, 30, 1), 2: tokens_for(V, 9, 2)}
    for rid, p in prompts.items():
        sched.add_request(p, SamplingParams(max_tokens=6), rid=rid)
    reports = []
    while not sched.idle:
        reports.append(sched.step())
        sched.engine.cache.check()
    assert reports[0].entries == [(0, 5), (1, 11)]  # FIFO, cut by the budget of 16
    assert reports[0].sampled[0][0] == 0 and len(reports[0].sampled) == 1  # a portion is not sampled
    assert reports[1].entries == [(0, 1), (1, 15)]  # the decode goes first, the prompt takes the rest
    assert reports[2].entries[:2] == [(0, 1), (1, 4)] and reports[2].entries[2][0] == 2
    assert all(sum(n for _, n in r.entries) <= 16 for r in reports)
    for rid, p in prompts.items():
        assert sched.done[rid].output == plain.greedy(p, 6)
        assert sched.done[rid].finish_reason == "length"
    assert all(g.pool.free_count == g.pool.num_pages for g in sched.engine.cache.paged)
    assert sched.reserved == [0]


def test_admission_waits_for_pages_and_request_slots(setup):
    sched, plain = setup(pages=12, page=4, reqs=2)  # 48 tokens of cache
    V = plain.cfg.vocab
    a = sched.add_request(tokens_for(V, 10, 0), SamplingParams(max_tokens=10))  # 5 pages
    b = sched.add_request(tokens_for(V, 17, 1), SamplingParams(max_tokens=8))   # 7 pages
    c = sched.add_request(tokens_for(V, 3, 2), SamplingParams(max_tokens=2))    # 2 pages, waits for a slot
    r = sched.step()
    assert r.admitted == [a, b] and len(sched.waiting) == 1
    big = sched.add_request(tokens_for(V, 20, 3), SamplingParams(max_tokens=20))  # 10 pages
    order = []
    while not sched.idle:
        rep = sched.step()
        order += rep.admitted
        sched.engine.cache.check()
        assert all(x <= p for x, p in zip(sched.reserved, sched.pool_pages))
    assert order == [c, big]  # first in, first out; big had to wait for pages
    assert all(sched.done[x].finish_reason == "length" for x in (a, b, c, big))


def test_requests_that_cannot_fit_get_an_error_not_a_hang(setup):
    sched, plain = setup(pages=6, page=4)  # 24 tokens
    V = plain.cfg.vocab
    too_big = sched.add_request(tokens_for(V, 20, 0), SamplingParams(max_tokens=30))
    empty = sched.add_request([], SamplingParams())
    bad = sched.add_request([1, 99999], SamplingParams())
    assert sched.done[empty].finish_reason == "error" and "empty" in sched.done[empty].error
    assert sched.done[bad].finish_reason == "error" and "token id" in sched.done[bad].error
    long = sched.add_request(tokens_for(V, 24, 1), SamplingParams(max_tokens=4))
    assert sched.done[long].finish_reason == "error" and "longest sequence" in sched.done[long].error
    # max_tokens is clamped to what the longest sequence leaves
    ok = sched.add_request(tokens_for(V, 20, 2), SamplingParams(max_tokens=30))
    sched.run()
    assert sched.done[ok].finish_reason == "length" and len(sched.done[ok].output) == 4
    assert sched.done[too_big].finish_reason == "length" and len(sched.done[too_big].output) == 4


def test_eos_finishes_and_abort_frees(setup):
    sched, plain = setup()
    V = plain.cfg.vocab
    p = tokens_for(V, 7, 5)
    greedy = plain.greedy(p, 5)
    sched.eos = {greedy[2]}
    a = sched.add_request(p, SamplingParams(max_tokens=5))
    b = sched.add_request(p, SamplingParams(max_tokens=5, ignore_eos=True))
    c = sched.add_request(tokens_for(V, 9, 6), SamplingParams(max_tokens=50))
    for _ in range(3):
        sched.step()
    assert sched.abort(c) and sched.done[c].finish_reason == "abort"
    sched.run()
    first = greedy.index(greedy[2])
    assert sched.done[a].output == greedy[:first + 1] and sched.done[a].finish_reason == "stop"
    assert sched.done[b].output == greedy and sched.done[b].finish_reason == "length"
    sched.engine.cache.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in sched.engine.cache.paged)


def test_overlapped_steps_give_the_same_tokens_as_plain_steps(setup):
    """Launching step N+1 before step N's tokens are read changes nothing but the timing: the
    same outputs, an EOS seen one step late with the token past it dropped, every page back."""
    outs = {}
    for overlap in (False, True):
        sched, plain = setup(pages=14, page=4, reqs=3, max_step=9)
        V = plain.cfg.vocab
        prompts = [tokens_for(V, n, 50 + n) for n in (6, 13, 4, 10, 3)]
        greedy = plain.greedy(prompts[0], 9)
        sched.eos = {greedy[3]}
        for i, p in enumerate(prompts):
            sched.add_request(p, SamplingParams(max_tokens=9 if i != 2 else 1, temperature=0.0 if i % 2 == 0 else 0.7,
                                                seed=3), rid=i)
        fed = {i: 0 for i in range(5)}
        while not sched.idle:
            rep = sched.step_overlapped() if overlap else sched.step()
            for rid, n in rep.entries:
                fed[rid] += n
            sched.engine.cache.check()
            assert all(x <= p for x, p in zip(sched.reserved, sched.pool_pages))
        assert sched.drain() is None or overlap
        outs[overlap] = {i: (sched.done[i].output, sched.done[i].finish_reason) for i in range(5)}
        first = greedy.index(greedy[3])
        assert outs[overlap][0] == (greedy[:first + 1], "stop")
        assert len(outs[overlap][2][0]) == 1
        assert all(g.pool.free_count == g.pool.num_pages for g in sched.engine.cache.paged)
        assert sched.reserved == [0]
        if not overlap:  # a plain step never feeds a token past the end
            assert fed[0] == len(prompts[0]) + first
    assert outs[True] == outs[False]


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(setup):
    sched, plain = setup(raw=TINY_B, name="B", page=8, pages=30, max_step=7)
    V = plain.cfg.vocab
    prompts = [tokens_for(V, n, n) for n in (3, 11, 23, 40)]
    sp = SamplingParams(temperature=0.8, max_tokens=12, seed=7)
    for i, p in enumerate(prompts):
        sched.add_request(p, sp, rid=i)
    sched.run()
    together = {i: sched.done[i].output for i in range(4)}
    for i, p in enumerate(prompts):  # alone, one at a time: same tokens
        sched.add_request(p, sp, rid=i)
        sched.run()
        assert sched.done[i].output == together[i]
    # and they are what the plain sampler draws from the plain model's logits
    toks = list(prompts[1])
    for step, got in enumerate(together[1]):
        want = sample_reference(plain.logits(toks)[-1], 0.8, -1, 1.0, uniform_for(7, 1, step))
        assert got == want
        toks.append(got)
    other = SamplingParams(temperature=0.8, max_tokens=12, seed=8)
    sched.add_request(prompts[3], other, rid=3)
    sched.run()
    assert sched.done[3].output != together[3]


def test_sampling_params_follow_the_reference():
    assert SamplingParams().is_greedy and SamplingParams(temperature=1.0, top_k=1).is_greedy
    assert not SamplingParams(temperature=0.0, top_p=0.9).is_greedy
    assert not SamplingParams(temperature=0.5).is_greedy
    assert SamplingParams().max_tokens == 1024 and SamplingParams().top_k == -1
    assert 0.0 <= uniform_for(1, "a", 3) < 1.0 and uniform_for(1, "a", 3) == uniform_for(1, "a", 3)
    assert uniform_for(1, "a", 3) != uniform_for(1, "a", 4)


def test_windowed_groups_are_reserved_at_their_peak(setup, tmp_path_factory):
    """A mixer with a window keeps few pages between steps but needs those of a whole portion while
    a step runs: admission reserves that peak, so admitted requests never meet "out of pages", with
    portions longer than a token and a pool that holds barely more than one request."""
    import dataclasses

    from freetoken_b200.config.engine_config import EngineConfig
    from freetoken_b200.config.spec import PartSpec
    from freetoken_b200.engine.engine import Engine

    sched0, plain = setup()
    base = sched0.engine
    folder = base.config.model_path
    layers = tuple(dataclasses.replace(ls, mixer=PartSpec(ls.mixer.kind, dict(ls.mixer.params, window=8)))
                   for ls in base.spec.layers)
    spec = dataclasses.replace(base.spec, layers=layers)

    def run(pages, max_step, prompts):
        cfg = EngineConfig(model_path=folder, dtype="float32", device="cpu", page_size=4, num_page_override=pages,
                           max_step_tokens=max_step, max_extend_tokens=max_step, max_running_req=3, check_cache=True)
        eng = Engine(cfg, spec=spec)
        s = Scheduler(eng, Sampler(eng.device, eng.spec.vocab_size, 3))
        ids = [s.add_request(p, SamplingParams(max_tokens=12)) for p in prompts]
        live = 0
        while not s.idle:
            s.step()
            live = max(live, len(s.running))
            eng.cache.check()
            assert all(x <= p for x, p in zip(s.reserved, s.pool_pages))
        assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)
        return [s.done[i] for i in ids], live, s

    V = plain.cfg.vocab
    prompts = [tokens_for(V, n, 70 + n) for n in (100, 61, 33)]
    roomy, live_roomy, _ = run(pages=200, max_step=8, prompts=prompts)
    tight, live_tight, s = run(pages=6, max_step=8, prompts=prompts)  # ceil((7 + 8) / 4) + 1 = 5 pages a request
    assert [r.finish_reason for r in tight] == ["length"] * 3
    assert [r.output for r in tight] == [r.output for r in roomy]  # same tokens, only later
    assert live_roomy == 3 and live_tight == 1
    assert s.engine.cache.pages_to_admit(112, 8) == [5]
    # a step size whose peak the pool cannot hold is answered with an error, not admitted to fail later
    refused, _, _ = run(pages=6, max_step=64, prompts=prompts[:1])
    assert refused[0].finish_reason == "error" and "pages" in refused[0].error


def test_status_lines_in_the_references_words(setup):
    """A line per step that reads prompt tokens, and one every ``decode_log_interval`` decode steps."""
    from freetoken_b200.engine.status import StatusLine

    sched, plain = setup(max_step=16)
    lines, t = [], [0.0]

    def clock():
        t[0] += 0.5
        return t[0]

    sched.status = StatusLine(decode_log_interval=3, log=lines.append, clock=clock)
    V = plain.cfg.vocab
    for n in (5, 30):
        sched.add_request(tokens_for(V, n, n), SamplingParams(max_tokens=7))
    sched.run(overlap=False)
    prefill = [l for l in lines if l.startswith("Prefill batch")]
    decode = [l for l in lines if l.startswith("Decode batch")]
    assert len(prefill) == 3 and "#new-token: 16" in prefill[0] and "#new-seq: 2" in prefill[0]  # 5 + 11, then 15, then 4
    assert "#queue-req: 0" in prefill[0] and "input throughput (token/s):" in prefill[0]
    assert len(decode) >= 2 and "gen throughput (token/s):" in decode[0] and "#running-req:" in decode[0]
    assert "token usage: 0." in decode[0]
