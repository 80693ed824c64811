"""A status line now and then while requests are served, in the words of the reference's
(python/freetoken/scheduler/status.py:60-130): for steps that read prompts, how many new tokens went in
and how fast; every ``decode_log_interval`` decode steps (``--decode-log-interval``, 40 in the reference's
server, python/freetoken/server/args.py), the running and waiting requests, the share of the cache in
use and the tokens generated per second.  Lines go to the ``freetoken_b200`` logger at INFO level."""

from __future__ import annotations

import logging
import time
from typing import Callable, Optional

logger = logging.getLogger("freetoken_b200")


class StatusLine:
    def __init__(self, decode_log_interval: int = 40, log: Optional[Callable[[str], None]] = None,
                 clock: Callable[[], float] = time.perf_counter):
        self.interval = max(1, int(decode_log_interval))
        self.log = log or logger.info
        self.clock = clock
        self._last_prefill = self._last_decode = clock()
        self._decode_steps = 0
        self._decoded = 0

    def step(self, report, scheduler) -> None:
        """``report``: the :class:`StepReport` of a resolved step; ``scheduler``: where it came from."""
        cache = scheduler.engine.cache
        used = sum(g.pool.num_pages - g.pool.free_count for g in cache.paged)
        total = sum(g.pool.num_pages for g in cache.paged)
        usage = used / total if total else 0.0
        prompt_tokens = sum(n for _, n in report.entries if n > 1)
        now = self.clock()
        if prompt_tokens:
            gap = now - self._last_prefill
            self._last_prefill = now
            self.log(f"Prefill batch, #new-seq: {len(report.admitted)}, #new-token: {prompt_tokens}, "
                     f"token usage: {usage:.2f}, #running-req: {len(scheduler.running)}, "
                     f"#queue-req: {len(scheduler.waiting)}, "
                     f"input throughput (token/s): {prompt_tokens / gap if gap > 0 else 0.0:.2f}")
        if report.sampled:
            self._decode_steps += 1
            self._decoded += len(report.sampled)
            if self._decode_steps % self.interval == 0:
                gap = now - self._last_decode
                self._last_decode = now
                rate = self._decoded / gap if gap > 0 else 0.0
                self._decoded = 0
                self.log(f"Decode batch, #running-req: {len(scheduler.running)}, #token: {used * cache.page_size}, "
                         f"token usage: {usage:.2f}, gen throughput (token/s): {rate:.2f}, "
                         f"#queue-req: {len(scheduler.waiting)}")
