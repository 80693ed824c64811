"""Architecture-neutral description of a decoder model as data.

A model is a list of layers; a layer names an arrangement (block), a mixer, a
feed-forward and its norms, each as a :class:`PartSpec` = (kind, parameters).
The kind selects a class from a part registry (:mod:`freetoken_b200.parts`), the
parameters carry every size and constant, so no part needs to know which model
it belongs to.  The order in which layers run is data too (:class:`ScheduleEntry`):
a schedule may run a layer twice, and an entry may read the cache that an
earlier entry wrote instead of owning one.

The reference keeps the same information in ``ModelConfig`` plus per-group specs
(python/freetoken/models/config.py:87-111,199-293); here it is flattened into
per-layer specs so that mixed stacks need no special cases.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` picks the class, ``params`` are its constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def key(self) -> Tuple:
        """Hashable identity (used to share e.g. one rope table between layers)."""

        def freeze(v):
            if isinstance(v, PartSpec):
                return v.key()
            if isinstance(v, Mapping):
                return tuple(sorted((k, freeze(x)) for k, x in v.items()))
            if isinstance(v, (list, tuple)):
                return tuple(freeze(x) for x in v)
            return v

        return (self.kind, freeze(self.params))


@dataclass(frozen=True)
class ParamSpec:
    """A tensor a part owns.

    ``dtype`` is ``"compute"`` (bfloat16 in the serving path, float32 in the
    32-bit path), ``"float32"`` (kept in 32-bit in both paths: norm scales, router
    matrices and biases) or ``"int32"`` (integer tables).
    ``init`` describes the random-weights distribution: ``("normal", mean, std)``,
    ``("zeros",)`` or ``("ones",)``.  ``store`` is the dtype the random-weights writer
    uses in the file (``None``: bfloat16 for ``"compute"``, else ``dtype``).
    """

    shape: Tuple[int, ...]
    dtype: str = "compute"
    init: Tuple = ("normal", 0.0, 0.02)
    store: Optional[str] = None

    def storage_dtype(self) -> str:
        if self.store is not None:
            return self.store
        return "bfloat16" if self.dtype == "compute" else self.dtype


@dataclass(frozen=True)
class PagedKVNeed:
    """A mixer that keeps per-token rows in pages.

    ``slabs`` lists what one token stores: ``(name, heads, dim)`` per slab
    (``("k", Hkv, D), ("v", Hkv, D)`` for attention; an indexer adds ``("index_k", 1, Di)``).
    A slab is laid out ``[pages, heads, page_size, dim]`` per owning schedule entry.
    ``window`` is ``None`` when every earlier token stays readable, else the number
    of most recent tokens that do; pages wholly older than that are given back.
    Mixers with equal needs share a group (one page pool, one block table).
    """

    slabs: Tuple[Tuple[str, int, int], ...]
    window: Optional[int] = None

    def group_key(self) -> Tuple:
        return ("paged", self.slabs, self.window)


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a fixed-size state per request (one slot per request).

    ``tensors`` maps a name to (shape of one request's state, dtype name).
    """

    tensors: Tuple[Tuple[str, Tuple[int, ...], str], ...]

    def group_key(self) -> Tuple:
        return ("state", self.tensors)


CacheNeed = Any  # PagedKVNeed | StateNeed | None


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer.  ``name`` is the weight-name prefix (``model.layers.3``)."""

    name: str
    block: PartSpec
    mixer: PartSpec
    ffn: PartSpec
    mixer_name: str = "self_attn"
    ffn_name: str = "mlp"


@dataclass(frozen=True)
class ScheduleEntry:
    """One step of the forward pass: run ``layer``.

    ``cache_from`` is ``None`` when the entry owns a cache of its own, else the index
    of an earlier schedule entry whose cache this entry's mixer reads (it then
    writes nothing).
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    max_position: int
    eos_token_ids: Tuple[int, ...] = ()
    embedding_name: str = "model.embed_tokens"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head"
    source: Any = None  # the architecture's own typed config, kept for reporting

    def validate(self) -> None:
        from ..errors import ConfigError

        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ConfigError(f"schedule[{i}] names layer {e.layer}, model has {n} layers")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ConfigError(
                        f"schedule[{i}].cache_from={e.cache_from} must name an earlier entry"
                    )
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ConfigError(
                        f"schedule[{i}].cache_from={e.cache_from} names an entry that owns no cache"
                    )
