"""The scheduler: admits requests, cuts prompts into portions, decodes, finishes and frees.

Every step carries one token for each request that is decoding plus, under the step's token
budget, the next portions of the prompts being read, so prompt work and decoding share steps.
The reference never mixes the two (prefill first, python/freetoken/scheduler/scheduler.py:828-833)
but the rest follows it: first-in first-out admission that stops at the first request that does
not fit (python/freetoken/scheduler/prefill.py:244-290), a request is admitted only when a
request slot is free and the pages for its prompt *and* its whole output are free beside what
the running requests still may take (prefill.py:51-67, python/freetoken/scheduler/decode.py:27-30),
``max_tokens`` is clamped to what the longest sequence leaves, and a prompt that is too long is
answered with an error instead of waiting forever (scheduler.py:489-519).  A portion of a prompt
is never sampled (prefill.py:28-37).  A request finishes by length or by an EOS token id
(scheduler.py:334-353) and its pages and state slot return to the free lists at once.

What happens when pages run out: they cannot, for admitted requests, because admission reserves
the pages of the whole request (prompt + max_tokens) in every cache group.  A request that could
not fit even in an empty cache is finished at once with ``finish_reason="error"``.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..errors import SchedulerError
from ..sampling.params import SamplingParams
from .engine import StepEntry


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    max_tokens: int  # clamped
    fed: int = 0  # prompt tokens already given to the engine
    output: List[int] = field(default_factory=list)
    last_token: Optional[int] = None  # sampled, not yet fed
    finished: bool = False
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    reserved: List[int] = field(default_factory=list)  # pages reserved per cache group

    @property
    def decoding(self) -> bool:
        return self.fed == len(self.prompt)


@dataclass
class StepReport:
    """What one scheduler step did (for tests, logs and the benchmark)."""

    entries: List[Tuple[Hashable, int]]  # (request, tokens fed) in step order
    sampled: List[Tuple[Hashable, int]]  # (request, new token)
    finished: List[Hashable]
    admitted: List[Hashable]


class Scheduler:
    def __init__(self, engine, sampler, eos_token_ids: Sequence[int] = ()):
        self.engine = engine
        self.sampler = sampler
        self.eos = set(int(e) for e in eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.done: Dict[Hashable, Request] = {}
        self._next_id = 0
        cache = engine.cache
        self.pool_pages = [g.pool.num_pages for g in cache.paged]
        self.reserved = [0] * len(cache.paged)
        self.max_running = engine.config.max_running_req
        self.max_step_tokens = engine.max_step_tokens
        self.max_extend = engine.config.max_extend_tokens
        self.max_seq_len = engine.max_seq_len

    # ------------------------------------------------------------------ intake
    def add_request(self, prompt: Sequence[int], params: SamplingParams, rid: Optional[Hashable] = None) -> Hashable:
        if rid is None:
            rid = self._next_id
            self._next_id += 1
        prompt = [int(t) for t in prompt]
        req = Request(rid=rid, prompt=prompt, params=params, max_tokens=params.max_tokens)
        vocab = self.engine.spec.vocab_size
        if not prompt:
            return self._reject(req, "empty prompt")
        if min(prompt) < 0 or max(prompt) >= vocab:
            return self._reject(req, f"token id outside [0, {vocab})")
        if len(prompt) >= self.max_seq_len:
            return self._reject(req, f"prompt of {len(prompt)} tokens does not fit the longest "
                                     f"sequence of {self.max_seq_len}")
        req.max_tokens = min(params.max_tokens, self.max_seq_len - len(prompt))
        need = self.engine.cache.pages_to_admit(len(prompt) + req.max_tokens)
        if any(n > p for n, p in zip(need, self.pool_pages)):
            return self._reject(req, f"needs {need} pages, the cache has {self.pool_pages}")
        req.reserved = need
        self.waiting.append(req)
        return rid

    def _reject(self, req: Request, why: str) -> Hashable:
        req.finished, req.finish_reason, req.error = True, "error", why
        self.done[req.rid] = req
        return req.rid

    # ------------------------------------------------------------------ decisions
    def _admit(self) -> List[Hashable]:
        admitted = []
        while self.waiting and len(self.running) < self.max_running:
            req = self.waiting[0]
            if any(r + n > p for r, n, p in zip(self.reserved, req.reserved, self.pool_pages)):
                break  # the first request that does not fit stops the pass
            self.waiting.popleft()
            for i, n in enumerate(req.reserved):
                self.reserved[i] += n
            self.engine.open(req.rid)
            self.running.append(req)
            admitted.append(req.rid)
        return admitted

    def plan_step(self) -> List[Tuple[Request, List[int], List[int]]]:
        """(request, tokens, wanted places) for the next step: decodes first, then prompt portions."""
        plan = []
        budget = self.max_step_tokens
        for req in self.running:
            if req.decoding and budget > 0:
                plan.append((req, [req.last_token], [0]))
                budget -= 1
        for req in self.running:
            if not req.decoding and budget > 0:
                n = min(budget, self.max_extend, len(req.prompt) - req.fed)
                last = req.fed + n == len(req.prompt)
                plan.append((req, req.prompt[req.fed:req.fed + n], [n - 1] if last else []))
                budget -= n
        return plan

    # ------------------------------------------------------------------ one step
    def step(self) -> StepReport:
        admitted = self._admit()
        plan = self.plan_step()
        if not plan:
            if self.waiting and not self.running:
                raise SchedulerError("a waiting request cannot be admitted into an empty engine")
            return StepReport([], [], [], admitted)
        out = self.engine.step([StepEntry(r.rid, toks, want) for r, toks, want in plan])
        by_rid = {r.rid: r for r, _, _ in plan}
        for req, toks, _ in plan:
            if not req.decoding:
                req.fed += len(toks)
        rows = [by_rid[rid] for rid, _ in out.rows]
        tokens = self.sampler.sample(out.logits, [r.params for r in rows], [r.rid for r in rows],
                                     [len(r.output) for r in rows])
        sampled, finished = [], []
        for req, tok in zip(rows, tokens):
            req.output.append(tok)
            req.last_token = tok
            sampled.append((req.rid, tok))
            if tok in self.eos and not req.params.ignore_eos:
                req.finished, req.finish_reason = True, "stop"
            elif len(req.output) >= req.max_tokens:
                req.finished, req.finish_reason = True, "length"
            if req.finished:
                finished.append(req.rid)
        for rid in finished:
            req = by_rid[rid]
            self.running.remove(req)
            self.engine.close(rid)
            for i, n in enumerate(req.reserved):
                self.reserved[i] -= n
            self.done[rid] = req
        return StepReport([(r.rid, len(t)) for r, t, _ in plan], sampled, finished, admitted)

    def abort(self, rid: Hashable) -> bool:
        """Drop a request between steps; its pages and slot are given back."""
        for req in list(self.waiting):
            if req.rid == rid:
                self.waiting.remove(req)
                req.finished, req.finish_reason = True, "abort"
                self.done[rid] = req
                return True
        for req in self.running:
            if req.rid == rid:
                self.running.remove(req)
                self.engine.close(rid)
                for i, n in enumerate(req.reserved):
                    self.reserved[i] -= n
                req.finished, req.finish_reason = True, "abort"
                self.done[rid] = req
                return True
        return False

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    def run(self) -> None:
        while not self.idle:
            self.step()
