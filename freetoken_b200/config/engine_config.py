"""Engine options.

Names and meanings follow the reference's ``EngineConfig`` / ``SchedulerConfig``
(python/freetoken/engine/config.py:17-106, python/freetoken/scheduler/config.py:14-20)
where it has them: ``max_running_req``, ``page_size``, ``memory_ratio``,
``use_dummy_weight``, ``max_seq_len_override``, ``num_page_override``,
``num_token_override``, ``max_extend_tokens``.  Added here: ``num_layers`` (layer cap;
the reference uses an environment switch, python/freetoken/models/minimax_m3/config.py:64-76),
``max_step_tokens`` (token budget of one mixed step), ``seed`` and ``cuda_graph``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..errors import ConfigError

_DTYPES = {
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
    "float": "float32",
}


def normalize_dtype(dtype) -> str:
    """Accept a name or a ``torch.dtype``; return ``"bfloat16"`` or ``"float32"``."""
    name = str(dtype).replace("torch.", "")
    if name not in _DTYPES:
        raise ConfigError(f"dtype {dtype!r} is not supported (bfloat16 or float32)")
    return _DTYPES[name]


@dataclass
class EngineConfig:
    model_path: str
    dtype: str = "auto"  # "auto" takes config.json's torch_dtype, else bfloat16
    device: str = "cuda:0"
    max_running_req: int = 4
    page_size: int = 16
    memory_ratio: float = 0.9
    use_dummy_weight: bool = False  # random weights made on the device from `seed`
    max_seq_len_override: Optional[int] = None
    num_page_override: Optional[int] = None
    num_token_override: Optional[int] = None
    max_extend_tokens: int = 8192  # most prompt tokens of one request in one step
    max_step_tokens: Optional[int] = None  # token budget of one step (default: max_extend_tokens)
    num_layers: Optional[int] = None
    seed: int = 0
    cuda_graph: bool = True  # replay decode-only steps from CUDA graphs
    cuda_graph_max_bs: Optional[int] = None
    check_cache: bool = False  # run the cache manager's conservation check after every step
    # launch step N+1 before step N's tokens are read; the reference's switch is the environment
    # variable FREETOKEN_DISABLE_OVERLAP_SCHEDULING (python/freetoken/env.py:72), honoured here too
    overlap_scheduling: bool = True
    decode_log_interval: int = 0  # a status line every so many decode steps (the reference's server: 40); 0 = none

    def __post_init__(self) -> None:
        if self.dtype != "auto":
            self.dtype = normalize_dtype(self.dtype)
        if self.page_size < 1:
            raise ConfigError(f"page_size must be >= 1, got {self.page_size}")
        if self.max_running_req < 1:
            raise ConfigError(f"max_running_req must be >= 1, got {self.max_running_req}")
        if not 0.0 < self.memory_ratio <= 1.0:
            raise ConfigError(f"memory_ratio must be in (0, 1], got {self.memory_ratio}")
        if self.num_token_override is not None:
            if self.num_page_override is not None:
                raise ConfigError("give num_token_override or num_page_override, not both")
            if self.num_token_override % self.page_size:
                raise ConfigError(
                    f"num_token_override={self.num_token_override} must be a multiple of page_size={self.page_size}"
                )
            self.num_page_override = self.num_token_override // self.page_size
        if self.max_step_tokens is None:
            self.max_step_tokens = self.max_extend_tokens
        if self.max_extend_tokens < 1 or self.max_step_tokens < 1:
            raise ConfigError("max_extend_tokens and max_step_tokens must be >= 1")
