"""One registry from an architecture's name (``config.json``'s ``architectures[0]``) to its model.

An :class:`Architecture` bundles what is specific to one model family: how to read its
config.json into a typed config, how to turn that into a :class:`ModelSpec`, and how its
checkpoint names map onto the model's tensors.  Entries are imported lazily, as the
reference does (python/freetoken/models/register.py:12-17,19-125,128-143).

Adding an architecture: write a module that builds an ``Architecture`` and calls
:func:`register_architecture`, and add its module path to ``_LAZY`` (or import it yourself
before building an engine).
"""

from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

from .errors import ConfigError


@dataclass
class Architecture:
    names: Sequence[str]
    parse_config: Callable[..., Any]  # (raw config.json dict, num_layers=None) -> typed config
    build_spec: Callable[[Any], Any]  # typed config -> ModelSpec
    fusion_rules: Callable[[Any], List[Any]] = lambda cfg: []
    name_prefixes: Tuple[str, ...] = ()  # prefixes dropped from checkpoint tensor names
    ignorable: Callable[[str], bool] = lambda name: False  # checkpoint tensors never read


_REGISTRY: Dict[str, Architecture] = {}
_LAZY: Dict[str, str] = {
    "MiniMaxM3SparseForCausalLM": "freetoken_b200.models.minimax_m3",
    "MiniMaxM3SparseForConditionalGeneration": "freetoken_b200.models.minimax_m3",
}


def register_architecture(arch: Architecture) -> None:
    for n in arch.names:
        _REGISTRY[n] = arch


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def get_architecture(name: str) -> Architecture:
    if name not in _REGISTRY and name in _LAZY:
        importlib.import_module(_LAZY[name])
    if name not in _REGISTRY:
        known = sorted(set(_REGISTRY) | set(_LAZY))
        raise ConfigError(f"Model architecture '{name}' not supported (known: {known})")
    return _REGISTRY[name]


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    archs = raw.get("architectures")
    if not archs:
        raise ConfigError("config.json: 'architectures' is missing or empty")
    return get_architecture(str(archs[0]))


def known_architectures() -> List[str]:
    return sorted(set(_REGISTRY) | set(_LAZY))
