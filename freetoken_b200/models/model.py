"""A decoder model built from a :class:`ModelSpec`: embedding, scheduled layers, final norm, head.

The class knows no architecture: layers come from the part registries, their order from
``spec.schedule``.  Parameter names are the dotted paths of the part tree
(``model.layers.3.self_attn.qkv_proj.weight``), which is how the reference names its state
dict (python/freetoken/layers/base.py:15-53, python/freetoken/models/minimax_m3/model.py:25-97).

Forward (model.py:75-80,96-97; python/freetoken/layers/embedding.py:40-57,103-113): gather
embedding rows (no scaling) into the 32-bit residual stream, run the schedule, add the last
layer's output and apply the final norm at the rows whose logits are wanted only, multiply
by the head matrix (the embedding table when tied) into float32 logits.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from ..config.spec import ModelSpec, ParamSpec
from ..errors import ConfigError
from ..kernels import ops
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, BuildEnv, Part, StepState
from ..parts.base import as_rows


def _walk(prefix: str, part: Part, out: Dict[str, Tuple[Part, str, ParamSpec]]) -> None:
    for local, ps in part.param_specs().items():
        out[f"{prefix}.{local}"] = (part, local, ps)
    for name, child in part.children().items():
        _walk(f"{prefix}.{name}", child, out)


def head_matmul(y: torch.Tensor, w: torch.Tensor, logits: torch.Tensor) -> None:
    """``logits = y @ w^T`` as float32.  bfloat16 operands keep their 32-bit accumulator
    (the reference rounds the logits to bfloat16 and widens them again for sampling,
    python/freetoken/layers/embedding.py:113, python/freetoken/engine/sample.py:80)."""
    if y.dtype == torch.float32:
        torch.matmul(y, w.t(), out=logits)
    else:
        torch.mm(y, w.t(), out=logits, out_dtype=torch.float32)


class Model:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        spec.validate()
        self.spec = spec
        self.env = env
        self.hidden = spec.hidden_size
        self.vocab = spec.vocab_size
        self.tied = bool(spec.head.get("tied", False))
        self.blocks = []
        for ls in spec.layers:
            mixer = MIXERS.build(ls.mixer, env)
            ffn = FEED_FORWARDS.build(ls.ffn, env)
            self.blocks.append(BLOCKS.build(ls.block, env, mixer=mixer, ffn=ffn,
                                            mixer_name=ls.mixer_name, ffn_name=ls.ffn_name))
        self.final_norm = NORMS.build(spec.final_norm, env)
        self.embed_weight: Optional[torch.Tensor] = None
        self.head_weight: Optional[torch.Tensor] = None
        self._index: Dict[str, Tuple[Optional[Part], str, ParamSpec]] = {}
        self._index[f"{spec.embedding_name}.weight"] = (None, "embed", ParamSpec((self.vocab, self.hidden)))
        if not self.tied:
            self._index[f"{spec.head_name}.weight"] = (None, "head", ParamSpec((self.vocab, self.hidden)))
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
            if part is None:
                if local == "embed":
                    self.embed_weight = t
                else:
                    self.head_weight = t
            else:
                per_part.setdefault(id(part), (part, {}))[1][local] = t
        for part, ts in per_part.values():
            part.bind(ts)
        if self.tied:
            self.head_weight = self.embed_weight

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

    # ------------------------------------------------------------------ forward
    def forward(self, step: StepState, cache_views: List[Any]) -> torch.Tensor:
        """Run the step's tokens; return float32 logits ``[n_logit_rows, vocab]``.

        ``cache_views[i]`` is the cache view of schedule entry ``i`` (the owner's view when the
        entry reads another entry's cache)."""
        T = step.n_tokens
        env = self.env
        ws, dt, cap = env.workspace, env.dtype, env.max_step_tokens
        residual = ws.get("model.residual", (T, self.hidden), torch.float32, (cap, self.hidden))
        ops.embedding_gather(self.embed_weight, step.token_ids, residual)
        x = None
        for i, e in enumerate(self.spec.schedule):
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
        self.final_norm.add_forward(as_rows(x, self.final_norm), residual, y, rows=step.logit_rows)
        head_matmul(y, self.head_weight, logits)
        return logits
