"""Per-request sampling parameters, with the reference's names, defaults and greedy rule
(python/freetoken/core.py:18-31).  ``seed`` is added: draws are a function of (seed, request,
step) only, so they do not depend on what else is in the batch."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from ..errors import ConfigError


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    ignore_eos: bool = False
    max_tokens: int = 1024
    stop_strs: List[str] = field(default_factory=list)
    seed: Optional[int] = None

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ConfigError(f"max_tokens must be >= 1, got {self.max_tokens}")
        if not 0.0 < self.top_p <= 1.0:
            raise ConfigError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.stop_strs:
            raise ConfigError("stop_strs need a tokenizer, which this engine does not carry; "
                              "stop on token ids through eos_token_id instead")

    @property
    def is_greedy(self) -> bool:
        return (self.temperature <= 0.0 or self.top_k == 1) and self.top_p == 1.0
