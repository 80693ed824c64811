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

Steps can be overlapped (``step_overlapped``, the default of ``run``): the next step is planned and
launched while the device still computes the one before, whose sampled tokens stay on the device and
are copied into the next step's token ids there; the host reads them one step late
(scheduler.py:194-256 in the reference).  ``step`` launches and reads in one go.

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
    in_flight: int = 0  # tokens sampled on the device and not yet read by the host
    source: Optional[Tuple[Any, int]] = None  # (device tensor, index) of the newest such token

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


@dataclass
class Flight:
    """A step that runs on the device: what it fed, whom it samples for, and the sampler's ticket."""

    entries: List[Tuple[Hashable, int]]
    rows: List[Request]
    ticket: Any
    admitted: List[Hashable]


class Scheduler:
    def __init__(self, engine, sampler, eos_token_ids: Sequence[int] = (), status=None):
        """``status``: a :class:`freetoken_b200.engine.status.StatusLine` that is told of every resolved step."""
        self.engine = engine
        self.sampler = sampler
        self.status = status
        self.eos = set(int(e) for e in eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.done: Dict[Hashable, Request] = {}
        self._next_id = 0
        self._flight: Optional[Flight] = None
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
        need = self.engine.cache.pages_to_admit(len(prompt) + req.max_tokens,
                                                  min(self.max_step_tokens, self.max_extend))
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
        """(request, tokens, wanted places) for the next step: decodes first, then prompt portions.

        A request whose newest token is still on the device (``in_flight``) is planned with a
        placeholder token; a request whose launched tokens already reach ``max_tokens`` is left
        out (it finishes by length when its last launch is resolved)."""
        plan = []
        budget = self.max_step_tokens
        for req in self.running:
            if req.decoding and budget > 0 and len(req.output) + req.in_flight < req.max_tokens:
                plan.append((req, [0 if req.in_flight else req.last_token], [0]))
                budget -= 1
        for req in self.running:
            if not req.decoding and budget > 0:
                n = min(budget, self.max_extend, len(req.prompt) - req.fed)
                last = req.fed + n == len(req.prompt)
                plan.append((req, req.prompt[req.fed:req.fed + n], [n - 1] if last else []))
                budget -= n
        return plan

    # ------------------------------------------------------------------ one step
    def _launch(self) -> Optional[Flight]:
        """Admit, plan and start one step on the device; nothing waits for it."""
        admitted = self._admit()
        plan = self.plan_step()
        if not plan:
            return Flight([], [], None, admitted) if admitted else None
        entries = [StepEntry(r.rid, toks, want, device_token=r.source if (r.decoding and r.in_flight) else None)
                   for r, toks, want in plan]
        out = self.engine.step(entries)
        by_rid = {r.rid: r for r, _, _ in plan}
        for req, toks, _ in plan:
            if not req.decoding:
                req.fed += len(toks)
        rows = [by_rid[rid] for rid, _ in out.rows]
        ticket = self.sampler.launch(out.logits, [r.params for r in rows], [r.rid for r in rows],
                                     [len(r.output) + r.in_flight for r in rows])
        for i, req in enumerate(rows):
            req.in_flight += 1
            req.source = (ticket.device_tokens, i)
        return Flight([(r.rid, len(t)) for r, t, _ in plan], rows, ticket, admitted)

    def _resolve(self, flight: Flight) -> StepReport:
        """Take a launched step's tokens to the host; finish and free what ended."""
        tokens = self.sampler.result(flight.ticket) if flight.ticket is not None else []
        sampled, finished = [], []
        for req, tok in zip(flight.rows, tokens):
            req.in_flight -= 1
            if req.finished:
                continue  # ended by an earlier token; this one was computed ahead and is dropped
            req.output.append(tok)
            req.last_token = tok
            sampled.append((req.rid, tok))
            if tok in self.eos and not req.params.ignore_eos:
                req.finished, req.finish_reason = True, "stop"
            elif len(req.output) >= req.max_tokens:
                req.finished, req.finish_reason = True, "length"
            if req.finished:
                finished.append(req.rid)
                # a step that already runs with this request is ordered before any later step
                # on the stream, so its pages can go back now
                self.running.remove(req)
                self.engine.close(req.rid)
                for i, n in enumerate(req.reserved):
                    self.reserved[i] -= n
                self.done[req.rid] = req
        report = StepReport(flight.entries, sampled, finished, flight.admitted)
        if self.status is not None:
            self.status.step(report, self)
        return report

    def step(self) -> StepReport:
        """One step, launched and resolved (nothing stays in flight)."""
        if self._flight is not None:
            return self._resolve(self._take())
        flight = self._launch()
        if flight is None:
            if self.waiting and not self.running:
                raise SchedulerError("a waiting request cannot be admitted into an empty engine")
            return StepReport([], [], [], [])
        return self._resolve(flight)

    def _take(self) -> Flight:
        flight, self._flight = self._flight, None
        return flight

    def step_overlapped(self) -> StepReport:
        """Launch the next step, then resolve the one before it: the host's work for step N+1
        (planning, metadata, launches) runs while the device computes step N.  The newest token
        of every decoding request stays on the device and is copied into the next step's
        token ids there; an EOS is seen one step late and the token computed past it is dropped.
        The reference overlaps the same way (python/freetoken/scheduler/scheduler.py:194-256)."""
        before = self._flight
        self._flight = self._launch()
        if before is not None:
            return self._resolve(before)
        if self._flight is None:
            if self.waiting and not self.running:
                raise SchedulerError("a waiting request cannot be admitted into an empty engine")
            return StepReport([], [], [], [])
        if self._flight.ticket is None or not self._flight.rows:
            return self._resolve(self._take())  # nothing to wait for: no token was sampled
        return StepReport([], [], [], [])

    def drain(self) -> Optional[StepReport]:
        """Resolve what is in flight."""
        return self._resolve(self._take()) if self._flight is not None else None

    def abort(self, rid: Hashable) -> bool:
        """Drop a request between steps; its pages and slot are given back.  A token computed
        ahead for it (overlapped scheduling) is dropped when its step is resolved."""
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

    def run(self, overlap: bool = True) -> None:
        while not self.idle:
            if overlap:
                self.step_overlapped()
            else:
                self.step()
        self.drain()
