"""Helpers shared by the tests: model folders in temp dirs, engines, traces of steps."""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from freetoken_b200.config.engine_config import EngineConfig
from freetoken_b200.engine.engine import Engine, StepEntry
from freetoken_b200.weights.random_init import write_model_folder
from plain.m3_plain import PlainM3

_FOLDERS: Dict[Tuple[str, int], str] = {}

# PlainM3.router_margins reports a token's smallest gap in a discrete choice (expert, key block), or 0
# when bfloat16 rounding moves the scores by a sizeable part of that gap.  At such a token a bfloat16
# run may legitimately choose otherwise, which changes its logits by more than rounding; bfloat16
# comparisons check those tokens only loosely and require them to be a minority.
NEAR_TIE = 0.0
# bfloat16 logits against the 32-bit plain model.  Measured on the tiny configurations (whole prompts and
# portions, six sequences each, positions clear of near-ties): the engine's largest error is 0.0049 (A),
# 0.0046 (B), 0.0030 (D), 0.0045 (E), which is also what the plain model's own bfloat16 emulation makes
# (0.0049 / 0.0044 / 0.0031 / 0.0052), on logits that spread by 0.16 to 0.21; C, whose experts' output is
# doubled (routed_scaling_factor 2) and joined by a shared expert, reaches 0.0126.  The bound is about twice
# that: it is far below the reference's own bound for its bfloat16 kernels (3e-2 max-abs,
# tests/kernels/test_minimax_m3_sparse.py:275-276), so that a fault the size of the noise shows.
BF16_TOL = dict(rtol=2e-2, atol=8e-3)
BF16_NOISE = {"C": 2.0}  # configurations whose bfloat16 noise is a multiple of the others'
F32_TOL = dict(rtol=1e-4, atol=2e-5)


def bf16_tol(name: str = "") -> dict:
    f = BF16_NOISE.get(name, 1.0)
    return dict(rtol=BF16_TOL["rtol"], atol=BF16_TOL["atol"] * f)


def assert_bf16_close(got: torch.Tensor, ref: torch.Tensor, margins: torch.Tensor, what: str = "",
                      prefix_only: bool = False, name: str = "") -> None:
    """``got`` (bfloat16 engine) against ``ref`` (32-bit plain) at every position whose router
    gaps are clear of bfloat16 noise; the others are checked loosely.  ``prefix_only`` (models
    with block-sparse layers, where a flip spreads to later tokens) compares strictly only the
    positions before the first near-tie."""
    sure = margins[: got.shape[0]] > NEAR_TIE
    if prefix_only:
        first = int((~sure).float().argmax()) if (~sure).any() else sure.numel()
        sure = torch.arange(sure.numel()) < first
        assert first >= min(24, sure.numel()), f"{what}: the first near-tie comes at {first}, too early to compare"
    else:
        assert sure.float().mean() > 0.5, f"{what}: too many near-ties for a meaningful comparison"
    torch.testing.assert_close(got[sure], ref[: got.shape[0]][sure], **bf16_tol(name), msg=lambda m: f"{what}: {m}")
    assert torch.isfinite(got).all()
    assert (got - ref[: got.shape[0]]).abs().max() < 0.5, what


def model_folder(tmp_root, name: str, raw: dict, seed: int = 1) -> str:
    key = (name, seed)
    if key not in _FOLDERS or not os.path.isdir(_FOLDERS[key]):
        d = os.path.join(str(tmp_root), f"model_{name}_{seed}")
        write_model_folder(raw, d, seed=seed)
        _FOLDERS[key] = d
    return _FOLDERS[key]


def make_engine(folder: str, dtype: str, device: str, page_size: int, pages: int, max_step: int = 256,
                reqs: int = 4, **kw) -> Engine:
    return Engine(EngineConfig(model_path=folder, dtype=dtype, device=device, page_size=page_size,
                               num_page_override=pages, max_step_tokens=max_step, max_extend_tokens=max_step,
                               max_running_req=reqs, check_cache=True, **kw))


def tokens_for(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def clear_tokens(plain, n: int, seed: int, min_prefix: int, tries: int = 300) -> List[int]:
    """A random sequence whose first router / block-choice near-tie (by the plain model) comes no
    earlier than ``min_prefix``: seeds ``seed, seed + 1, ...`` are tried in order."""
    for s in range(seed, seed + tries):
        toks = tokens_for(plain.cfg.vocab, n, s)
        unsure = plain.router_margins(toks) <= NEAR_TIE
        first = int(unsure.float().argmax()) if unsure.any() else n
        if first >= min(min_prefix, n):
            return toks
    raise AssertionError(f"no sequence with a clear prefix of {min_prefix} among {tries} seeds")


def replay_whole(engine: Engine, rid, toks: Sequence[int]) -> torch.Tensor:
    out = engine.step([StepEntry(rid, list(toks), list(range(len(toks))))])
    engine.close(rid)
    return out.logits.float().cpu().clone()


def replay_cuts(engine: Engine, rid, toks: Sequence[int], cuts: Sequence[int]) -> torch.Tensor:
    """Feed ``toks`` in portions of the given sizes (the rest one by one); logits at every place."""
    got, i = [], 0
    cuts = list(cuts)
    while i < len(toks):
        c = min(cuts.pop(0) if cuts else 1, len(toks) - i)
        out = engine.step([StepEntry(rid, list(toks[i:i + c]), list(range(c)))])
        got.append(out.logits.float().cpu().clone())
        i += c
    engine.close(rid)
    return torch.cat(got)


def replay_mixed(engine: Engine, seqs: Dict[str, Sequence[int]], schedule: Sequence[Dict[str, int]],
                 max_live: int = 4) -> Dict[str, torch.Tensor]:
    """``schedule``: per step, request -> number of its next tokens.  A request ends (and gives
    its pages back) right after the step that fed its last token.  Returns logits at every place."""
    fed = {r: 0 for r in seqs}
    got: Dict[str, List[torch.Tensor]] = {r: [] for r in seqs}
    for stepdef in schedule:
        entries, order = [], []
        for r, n in stepdef.items():
            n = min(n, len(seqs[r]) - fed[r])
            if n <= 0:
                continue
            entries.append(StepEntry(r, list(seqs[r][fed[r]:fed[r] + n]), list(range(n))))
            order.append((r, n))
        if not entries:
            continue
        out = engine.step(entries)
        logits = out.logits.float().cpu()
        i = 0
        for r, n in order:
            got[r].append(logits[i:i + n].clone())
            i += n
            fed[r] += n
            if fed[r] == len(seqs[r]):
                engine.close(r)
    assert all(fed[r] == len(seqs[r]) for r in seqs), "the schedule did not feed every token"
    return {r: torch.cat(v) for r, v in got.items()}


def mixed_schedule(lengths: Dict[str, int], seed: int, max_live: int = 4, budget: int = 40) -> List[Dict[str, int]]:
    """A schedule with up to ``max_live`` live requests: new ones start while others decode one
    token at a time; portion sizes change from step to step, down to two tokens."""
    import random

    rng = random.Random(seed)
    waiting = list(lengths)
    live: Dict[str, int] = {}
    left = dict(lengths)
    phase: Dict[str, str] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and rng.random() < 0.7:
            r = waiting.pop(0)
            live[r] = 0
            phase[r] = "prompt"
        step: Dict[str, int] = {}
        room = budget
        for r in list(live):
            if rng.random() < 0.15 and len(live) > 1:
                continue  # a request may sit a step out
            if phase[r] == "decode":
                n = 1
            else:
                n = rng.choice([2, 2, 3, 5, 7, 11, 13])
            n = min(n, left[r], room)
            if n <= 0:
                continue
            step[r] = n
            room -= n
            left[r] -= n
            if phase[r] == "prompt" and left[r] <= 32:
                phase[r] = "decode"
            if left[r] == 0:
                del live[r]
        if step:
            steps.append(step)
    return steps
