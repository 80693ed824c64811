"""Turns logits into tokens.

Greedy requests take the argmax; the others ``softmax(logits / max(T, 1e-6))``, top-k, then
top-p, then an inverse-CDF draw (python/freetoken/engine/sample.py:54-80).  One kernel
handles a whole batch, greedy and sampled rows together.  The uniform number of each draw is
made on the host from (seed, request, step) with a counter-based hash, so the same request
gives the same tokens whatever else shares its steps; the reference draws from the device's
global generator (python/freetoken/kernel/triton/sampling.py:398-409).
"""

from __future__ import annotations

import hashlib
from typing import Hashable, List, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams

MIN_T = 1e-6
MIN_P = 1e-6


def uniform_for(seed: int, request: Hashable, step: int) -> float:
    """A number in [0, 1) that depends only on its three arguments."""
    h = hashlib.blake2b(f"{seed}|{request!r}|{step}".encode(), digest_size=8).digest()
    return (int.from_bytes(h, "little") >> 40) / float(1 << 24)


class SampleTicket:
    """A launched sampling call: the tokens are on the device (``device_tokens``) and on their way to
    the host; :meth:`Sampler.result` waits for them."""

    def __init__(self, n: int, device_tokens: torch.Tensor, host_tokens: torch.Tensor, event):
        self.n = n
        self.device_tokens = device_tokens
        self.host_tokens = host_tokens
        self.event = event


class Sampler:
    BUFFERS = 3  # launches that may be in flight before a buffer is used again

    def __init__(self, device: torch.device, vocab_size: int, max_rows: int, default_seed: int = 0):
        self.device = device
        self.vocab_size = vocab_size
        self.default_seed = default_seed
        self.max_rows = max_rows
        pin = device.type == "cuda"
        # per buffer, one packed staging area: temperature, top_p, u (float32 as raw bits) and top_k
        self._host = [torch.empty(4 * max_rows, dtype=torch.int32, pin_memory=pin) for _ in range(self.BUFFERS)]
        self._host_np = [h.numpy() for h in self._host]
        self._dev = [torch.empty(4 * max_rows, dtype=torch.int32, device=device) for _ in range(self.BUFFERS)]
        self._out = [torch.zeros(max_rows, dtype=torch.int32, device=device) for _ in range(self.BUFFERS)]
        self._out_host = [torch.empty(max_rows, dtype=torch.int32, pin_memory=pin) for _ in range(self.BUFFERS)]
        self._turn = 0

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               requests: Sequence[Hashable], steps: Sequence[int]) -> SampleTicket:
        """Start sampling one token per row of ``logits``; nothing waits for the device."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows to sample, the sampler was built for {self.max_rows}")
        b = self._turn
        self._turn = (self._turn + 1) % self.BUFFERS
        if R == 0:
            return SampleTicket(0, self._out[b], self._out_host[b], None)
        m = self.max_rows
        ints = self._host_np[b]
        f = ints.view(np.float32)
        for i, (p, rid, st) in enumerate(zip(params, requests, steps)):
            greedy = p.is_greedy
            f[i] = 0.0 if greedy else max(p.temperature, MIN_T)
            f[m + i] = 1.0 if greedy else min(max(p.top_p, MIN_P), 1.0)
            seed = p.seed if p.seed is not None else self.default_seed
            f[2 * m + i] = 0.0 if greedy else uniform_for(seed, rid, st)
            ints[3 * m + i] = 0 if (greedy or p.top_k < 1) else min(p.top_k, self.vocab_size)
        dev = self._dev[b]
        dev.copy_(self._host[b], non_blocking=True)
        fd = dev.view(torch.float32)
        ops.sample(logits, fd[0:m], dev[3 * m:4 * m], fd[m:2 * m], fd[2 * m:3 * m], self._out[b])
        self._out_host[b][:R].copy_(self._out[b][:R], non_blocking=True)
        event = None
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
        return SampleTicket(R, self._out[b], self._out_host[b], event)

    def result(self, ticket: SampleTicket) -> List[int]:
        """The tokens of a launched call (waits for the device)."""
        if ticket.event is not None:
            ticket.event.synchronize()
        return ticket.host_tokens[: ticket.n].tolist()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               requests: Sequence[Hashable], steps: Sequence[int]) -> List[int]:
        """One token per row of ``logits`` (host list; the call waits for the device)."""
        return self.result(self.launch(logits, params, requests, steps))
