"""Typed configuration: model descriptions (:mod:`spec`), the MiniMax-M3 reader, engine options."""

from .spec import (
    CacheNeed,
    LayerSpec,
    ModelSpec,
    PagedKVNeed,
    ParamSpec,
    PartSpec,
    ScheduleEntry,
    StateNeed,
)
from .engine_config import EngineConfig

__all__ = [
    "CacheNeed",
    "EngineConfig",
    "LayerSpec",
    "ModelSpec",
    "PagedKVNeed",
    "ParamSpec",
    "PartSpec",
    "ScheduleEntry",
    "StateNeed",
]
