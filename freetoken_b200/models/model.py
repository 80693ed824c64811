"""A decoder model built from a :class:`ModelSpec`: embedding, scheduled layers, final norm, head.

The class knows no architecture: layers come from the part registries, their order from
``spec.schedule``.  Parameter names are the dotted paths of the part tree
(``model.layers.3.self_attn.qkv_proj.weight``), which is how the reference names its state
dict (python/freetoken/layers/base.py:15-53).

Forward (the order every model class of the reference follows, e.g. its M3 ``model.py:75-80,96-97``;
python/freetoken/layers/embedding.py:40-57,103-113): the
embedding part fills the 32-bit residual stream, the schedule runs, the last layer's output is
added and the final norm applied at the rows whose logits are wanted only, and the head part
turns those rows into float32 logits.  Embedding and head come from registries like every other
part (``spec.embedding.kind``, ``spec.head.kind``); the model hands them its vocabulary and width
as default parameters.
"""

from __future__ import annotations

from typing import Any, Dict, List, Tuple

import torch

from ..config.spec import ModelSpec, ParamSpec, PartSpec
from ..errors import ConfigError
from ..parts import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, BuildEnv, Part, StepState
from ..parts.base import as_rows, nvtx_range


def _walk(prefix: str, part: Part, out: Dict[str, Tuple[Part, str, ParamSpec]]) -> None:
    for local, ps in part.param_specs().items():
        out[f"{prefix}.{local}"] = (part, local, ps)
    for name, child in part.children().items():
        _walk(f"{prefix}.{name}", child, out)


class Model:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        spec.validate()
        self.spec = spec
        self.env = env
        self.hidden = spec.hidden_size
        self.vocab = spec.vocab_size
        ends = dict(vocab=self.vocab, hidden=self.hidden)
        self.embedding = EMBEDDINGS.build(PartSpec(spec.embedding.kind, {**ends, **spec.embedding.params}), env)
        self.head = HEADS.build(PartSpec(spec.head.kind, {**ends, **spec.head.params}), env)
        self.tied = bool(self.head.tied)
        self.blocks = []
        for ls in spec.layers:
            mixer = MIXERS.build(ls.mixer, env)
            ffn = FEED_FORWARDS.build(ls.ffn, env)
            self.blocks.append(BLOCKS.build(ls.block, env, mixer=mixer, ffn=ffn,
                                            mixer_name=ls.mixer_name, ffn_name=ls.ffn_name))
        self.final_norm = NORMS.build(spec.final_norm, env)
        self._index: Dict[str, Tuple[Part, str, ParamSpec]] = {}
        _walk(spec.embedding_name, self.embedding, self._index)
        _walk(spec.head_name, self.head, self._index)
        for ls, block in zip(spec.layers, self.blocks):
            _walk(ls.name, block, self._index)
        _walk(spec.final_norm_name, self.final_norm, self._index)

    # ------------------------------------------------------------------ tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        """Every tensor the model expects, by full name."""
        return {name: ps for name, (_, _, ps) in self._index.items()}

    def param_dtype(self, ps: ParamSpec) -> torch.dtype:
        if ps.dtype == "compute":
            return self.env.dtype
        return {"float32": torch.float32, "int32": torch.int32}[ps.dtype]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors``: full name -> device tensor of the expected shape and dtype."""
        per_part: Dict[int, Tuple[Part, Dict[str, torch.Tensor]]] = {}
        for name, (part, local, ps) in self._index.items():
            t = tensors[name]
            if tuple(t.shape) != tuple(ps.shape) or t.dtype != self.param_dtype(ps):
                raise ConfigError(f"bind: tensor '{name}' is {tuple(t.shape)} {t.dtype}, "
                                  f"expected {tuple(ps.shape)} {self.param_dtype(ps)}")
            per_part.setdefault(id(part), (part, {}))[1][local] = t
        for part, ts in per_part.values():
            part.bind(ts)
        if self.tied:
            self.head.tie(self.embedding)

    def cache_needs(self) -> List[Tuple[int, Any]]:
        """(schedule entry, need) for every entry that owns a cache."""
        out = []
        for i, e in enumerate(self.spec.schedule):
            if e.cache_from is None:
                need = self.blocks[e.layer].mixer.cache_need()
                if need is not None:
                    out.append((i, need))
        return out

    def mixers(self):
        return [b.mixer for b in self.blocks]

    def parts(self) -> List[Part]:
        """Every part of the model, each once (parts shared through ``env.shared`` included)."""
        seen: Dict[int, Part] = {}

        def visit(p: Part) -> None:
            if id(p) in seen:
                return
            seen[id(p)] = p
            for c in p.children().values():
                visit(c)

        for p in (self.embedding, *self.blocks, self.final_norm, self.head):
            visit(p)
        for p in self.env.shared.values():
            if isinstance(p, Part):
                visit(p)
        return list(seen.values())

    def workspace_bytes(self, n_tokens: int) -> int:
        """Work buffers of a step of ``n_tokens`` tokens: the model's own (residual stream, final
        rows, logits for ``env.max_decode_rows`` rows) and what its parts report.  Parts of equal
        kind and parameters share their buffers (they are named by the part, not by the layer),
        so each distinct one counts once."""
        own = n_tokens * self.hidden * (4 + 4) + self.env.max_decode_rows * self.vocab * 4
        distinct: Dict[Any, int] = {}
        for p in self.parts():
            distinct[(type(p), p.spec.key())] = max(distinct.get((type(p), p.spec.key()), 0),
                                                    int(p.workspace_bytes(n_tokens)))
        return own + sum(distinct.values())

    # ------------------------------------------------------------------ forward
    def forward(self, step: StepState, cache_views: List[Any]) -> torch.Tensor:
        """Run the step's tokens; return float32 logits ``[n_logit_rows, vocab]``.

        ``cache_views[i]`` is the cache view of schedule entry ``i`` (the owner's view when the
        entry reads another entry's cache)."""
        T = step.n_tokens
        env = self.env
        ws, dt, cap = env.workspace, env.dtype, env.max_step_tokens
        residual = ws.get("model.residual", (T, self.hidden), torch.float32, (cap, self.hidden))
        self.embedding.forward(step.token_ids, residual)
        x = None
        for i, e in enumerate(self.spec.schedule):
            with nvtx_range(f"layer {e.layer}"):
                x = self.blocks[e.layer].forward(x, residual, step, cache_views[i], e.cache_from is None)
        R = step.n_logit_rows
        if R == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=env.device)
        if step.decode_only:  # fixed address: CUDA graphs of decode steps write here
            logits = ws.get("model.logits.decode", (R, self.vocab), torch.float32,
                            (env.max_decode_rows, self.vocab))
        else:  # grows with the largest request for logits seen so far
            logits = ws.get("model.logits", (R, self.vocab), torch.float32)
        y = ws.get("model.final", (R, self.hidden), dt, (cap, self.hidden))
        with nvtx_range("final norm + head"):
            self.final_norm.add_forward(as_rows(x, self.final_norm), residual, y, rows=step.logit_rows)
            self.head.forward(y, logits)
        return logits
