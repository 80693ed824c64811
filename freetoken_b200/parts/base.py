"""Interfaces of the parts a layer is put together from, and their registries.

Seven kinds of part exist: mixer (attention, or anything else that mixes tokens),
feed-forward, norm, position encoding, block (the arrangement of those four in a layer),
and the model's two ends, embedding and head.  A part is built from a :class:`PartSpec` (its sizes and constants) and a
:class:`BuildEnv`; it declares the tensors it owns (:meth:`Part.param_specs`), gets
them bound by name (:meth:`Part.bind`), and runs on the tokens of one step.  No part
looks at the model it is in.

Adding a part: subclass the interface, decorate with the registry, e.g.
``@MIXERS.register("my_mixer")``, and name ``"my_mixer"`` as the ``kind`` of a
``PartSpec`` in a model description.  Nothing else in the framework changes.

The reference expresses the same roles as ``BaseOP`` trees whose attribute names are
the state-dict keys (python/freetoken/layers/base.py:15-53) and an attention-backend
interface reached through a process-global context (python/freetoken/attention/base.py:48-82,
python/freetoken/core.py:167-205); here the step's state is passed explicitly.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Generic, List, Mapping, Optional, Tuple, TypeVar

import torch

from ..config.spec import CacheNeed, ParamSpec, PartSpec
from ..errors import ConfigError

T = TypeVar("T")


class PartRegistry(Generic[T]):
    """Name -> class for one kind of part."""

    def __init__(self, what: str):
        self.what = what
        self._classes: Dict[str, Callable[..., T]] = {}

    def register(self, kind: str):
        def deco(cls):
            if kind in self._classes and self._classes[kind] is not cls:
                raise ConfigError(f"{self.what} kind '{kind}' is registered twice")
            self._classes[kind] = cls
            cls.kind = kind
            return cls

        return deco

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def build(self, spec: PartSpec, env: "BuildEnv", **kw) -> T:
        if spec.kind not in self._classes:
            raise ConfigError(
                f"unknown {self.what} kind '{spec.kind}' (registered: {sorted(self._classes)})"
            )
        return self._classes[spec.kind](spec, env, **kw)

    def kinds(self) -> List[str]:
        return sorted(self._classes)


_NVTX: Optional[bool] = None


class nvtx_range:
    """``with nvtx_range("layer 3"):`` marks a stretch of host work (and the launches it makes) for a
    profiler's timeline when ``FREETOKEN_NVTX=1`` is set, and does nothing otherwise.  The reference marks
    its layers the same way (python/freetoken/utils/torch_utils.py:23-37)."""

    def __init__(self, name: str):
        global _NVTX
        if _NVTX is None:
            import os

            _NVTX = os.environ.get("FREETOKEN_NVTX", "").lower() in ("1", "true", "yes", "on") and torch.cuda.is_available()
        self.name = name if _NVTX else None

    def __enter__(self):
        if self.name is not None:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.name is not None:
            torch.cuda.nvtx.range_pop()
        return False


MIXERS: PartRegistry = PartRegistry("mixer")
FEED_FORWARDS: PartRegistry = PartRegistry("feed-forward")
NORMS: PartRegistry = PartRegistry("norm")
POSITIONS: PartRegistry = PartRegistry("position encoding")
BLOCKS: PartRegistry = PartRegistry("block")
EMBEDDINGS: PartRegistry = PartRegistry("embedding")
HEADS: PartRegistry = PartRegistry("head")


@dataclass
class BuildEnv:
    """What a part needs to know about the engine it is built for."""

    dtype: torch.dtype  # compute dtype: torch.bfloat16 or torch.float32
    device: torch.device
    max_seq_len: int  # longest sequence a request may reach (sizes position tables); an upper bound while
    # parts are built, final (it may have shrunk to what the cache holds) before the first step
    max_step_tokens: int  # most tokens one step carries (sizes work buffers)
    workspace: "Workspace"
    max_decode_rows: int = 64  # most rows of logits a decode-only step asks for
    shared: Dict[Any, Any] = field(default_factory=dict)  # parts shared by spec (rope tables)


class Workspace:
    """Named device buffers that live as long as the engine.

    A buffer is allocated at its first request with the largest size any step can ask
    for and handed out as a view afterwards, so steps allocate nothing and CUDA graphs
    see fixed addresses."""

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[str, torch.Tensor] = {}

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype,
            max_shape: Optional[Tuple[int, ...]] = None) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            cap = n
            if max_shape is not None:
                cap = 1
                for s in max_shape:
                    cap *= s
                cap = max(cap, n)
            buf = torch.empty(max(cap, 1), dtype=dtype, device=self.device)
            self._buffers[name] = buf
        return buf[:n].view(shape)

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class Part:
    """Common base: parameters by local name."""

    kind: str = ""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env
        self.params: Dict[str, torch.Tensor] = {}

    def param_specs(self) -> Dict[str, ParamSpec]:
        """Local tensor name -> shape, dtype policy and random-init distribution."""
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the tensors of :meth:`param_specs` (already on the device, in their dtype)."""
        self.params = dict(tensors)

    def children(self) -> Dict[str, "Part"]:
        """Sub-parts by local name (their parameters are prefixed with ``name.``)."""
        return {}

    def workspace_bytes(self, n_tokens: int) -> int:
        """Bytes of work buffers this part (without its children) asks the :class:`Workspace` for
        in a step of ``n_tokens`` tokens.  The engine sets that much memory aside before it sizes
        the cache, because the buffers are only allocated at the first steps."""
        return 0


class RouteSum:
    """A feed-forward output that is still a sum to be taken: row ``t`` is
    ``sum_j y[pos[t * top_k + j]] (+ shared[t])``.  A norm with ``takes_route_sum`` adds it to the
    residual without the sum's trip through memory; for any other consumer :func:`as_rows` takes it."""

    def __init__(self, y: torch.Tensor, pos: torch.Tensor, top_k: int, shared: Optional[torch.Tensor],
                 n_tokens: int, out: torch.Tensor):
        self.y, self.pos, self.top_k, self.shared, self.n_tokens, self.out = y, pos, top_k, shared, n_tokens, out

    def rows(self) -> torch.Tensor:
        from ..kernels import ops

        ops.moe_combine(self.y, self.pos, self.n_tokens, self.top_k, self.shared, self.out)
        return self.out


def as_rows(x: Any, consumer: Any = None) -> Any:
    """``x`` as the consumer can take it: a :class:`RouteSum` stays one only for a norm that says it
    takes one."""
    if isinstance(x, RouteSum) and not getattr(consumer, "takes_route_sum", False):
        return x.rows()
    return x


class Norm(Part):
    takes_route_sum: bool = False  # add_forward accepts a RouteSum as x

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``out = norm(x)`` row by row."""
        raise NotImplementedError

    def add_forward(self, x: Optional[torch.Tensor], residual: torch.Tensor, out: torch.Tensor,
                    out_f32: Optional[torch.Tensor] = None,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += x`` (32-bit sum; skipped when ``x`` is None), ``out = norm(residual)``.

        With ``rows`` the sum and norm are taken only at those rows and the residual is left
        unchanged (used for the rows whose logits are wanted)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Owns whatever tables the encoding needs; mixers apply it inside their kernels."""

    def table(self) -> Optional[torch.Tensor]:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        """What the mixer keeps between steps: ``PagedKVNeed``, ``StateNeed`` or ``None``."""
        return None

    def forward(self, h: torch.Tensor, step: "StepState", cache: Any, writes_cache: bool) -> torch.Tensor:
        """``h [T, hidden]`` (normed input) -> ``[T, hidden]``.

        ``cache`` is the view of this schedule entry's cache for this step
        (``PagedCacheView``, ``StateCacheView`` or ``None``); ``writes_cache`` is false when
        the entry reads the cache another entry wrote."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, step: "StepState", h_f32: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    # Optional: ``forward_lazy(h, step, h_f32)`` may return a :class:`RouteSum` instead of rows; blocks
    # call it when it exists and hand the result to :func:`as_rows` before any consumer but a norm.

    wants_f32_input: bool = False  # ask the preceding norm for a 32-bit copy of its output

    def f32_input_needed(self, n_tokens: int) -> bool:
        """Whether a step of ``n_tokens`` tokens will read that copy (``h_f32`` may be None otherwise)."""
        return self.wants_f32_input


class Embedding(Part):
    """Token ids to rows of the 32-bit residual stream."""

    def forward(self, token_ids: torch.Tensor, residual: torch.Tensor) -> None:
        """``residual[t] = float32(row of token_ids[t])`` for the step's tokens (``residual [T, hidden]``)."""
        raise NotImplementedError

    def table(self) -> torch.Tensor:
        """The ``[vocab, hidden]`` table, for a head that is tied to it."""
        raise NotImplementedError


class Head(Part):
    """Normed rows to float32 logits."""

    tied: bool = False  # the head owns no matrix and is given the embedding by :meth:`tie`

    def tie(self, embedding: Embedding) -> None:
        raise NotImplementedError

    def forward(self, y: torch.Tensor, logits: torch.Tensor) -> None:
        """``logits [R, vocab]`` (float32, preallocated) from ``y [R, hidden]``."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of norm, mixer and feed-forward in one layer."""

    def __init__(self, spec: PartSpec, env: BuildEnv, mixer: Mixer, ffn: FeedForward,
                 mixer_name: str, ffn_name: str):
        super().__init__(spec, env)
        self.mixer = mixer
        self.ffn = ffn
        self.mixer_name = mixer_name
        self.ffn_name = ffn_name

    def forward(self, x: Optional[torch.Tensor], residual: torch.Tensor, step: "StepState",
                cache: Any, writes_cache: bool) -> torch.Tensor:
        """Consume the previous layer's output ``x`` (None for the first layer) and the
        running 32-bit ``residual`` (updated in place); return this layer's output, which the
        next layer (or the final norm) adds to the residual."""
        raise NotImplementedError


@dataclass
class Segment:
    """One request's share of a step (host side)."""

    request_id: Any
    q_start: int  # index of its first token among the step's tokens
    q_len: int
    kv_len: int  # tokens the request holds after this step
    state_slot: int = 0
    is_fresh: bool = False  # the request's first tokens ever (state must start from zero)

    @property
    def pos_start(self) -> int:
        return self.kv_len - self.q_len


@dataclass
class StepState:
    """Everything a part may read about the current step.  Device tensors are int32."""

    n_tokens: int
    segments: List[Segment]
    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T]
    seg_info: torch.Tensor  # [S, 4]: q_start, q_len, kv_len, block-table row
    state_slots: torch.Tensor  # [S]
    logit_rows: torch.Tensor  # [R] token indices whose logits are wanted
    n_logit_rows: int
    attention_plans: Dict[Any, Any] = field(default_factory=dict)  # per (group sizes, window)
    extras: Dict[str, Any] = field(default_factory=dict)
    decode_only: bool = False  # every segment brings exactly one token
    capturing: bool = False  # the step is being recorded into a CUDA graph
