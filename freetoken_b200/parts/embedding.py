"""The two ends of a model: token embedding and output head.

``token_embedding`` (python/freetoken/layers/embedding.py:40-57, ``embed_scale=None`` in
python/freetoken/models/minimax_m3/model.py:67-70,76): a pure row gather of ``[vocab, hidden]``
into the 32-bit residual stream, without scaling.

``linear_head`` (python/freetoken/layers/embedding.py:103-113): ``logits = y W^T`` without a bias,
kept as the float32 accumulator of the library product (the reference rounds the logits to
bfloat16 and widens them again for sampling, python/freetoken/engine/sample.py:80).  A tied head
multiplies by the embedding table and owns no tensor; a stray ``lm_head.weight`` in the file is
then ignored (embedding.py:81-90).

Other embeddings (scaled, with added position rows) and heads (bias, soft-cap, several outputs)
are other kinds in the same registries; the model asks for them by ``spec.embedding.kind`` and
``spec.head.kind``.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import ParamSpec, PartSpec
from ..errors import ConfigError
from ..kernels import ops
from .base import EMBEDDINGS, HEADS, BuildEnv, Embedding, Head


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab``, ``hidden``."""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab"])
        self.hidden = int(spec["hidden"])

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def forward(self, token_ids: torch.Tensor, residual: torch.Tensor) -> None:
        ops.embedding_gather(self.params["weight"], token_ids, residual)

    def table(self) -> torch.Tensor:
        return self.params["weight"]


@HEADS.register("linear_head")
class LinearHead(Head):
    """params: ``vocab``, ``hidden``, ``tied`` (bool: multiply by the embedding's table)."""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab"])
        self.hidden = int(spec["hidden"])
        self.tied = bool(spec.get("tied", False))
        self._tied_weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {} if self.tied else {"weight": ParamSpec((self.vocab, self.hidden))}

    def tie(self, embedding: Embedding) -> None:
        w = embedding.table()
        if tuple(w.shape) != (self.vocab, self.hidden):
            raise ConfigError(f"linear_head: cannot tie to an embedding table of shape {tuple(w.shape)}")
        self._tied_weight = w

    def weight(self) -> torch.Tensor:
        return self._tied_weight if self.tied else self.params["weight"]

    def forward(self, y: torch.Tensor, logits: torch.Tensor) -> None:
        w = self.weight()
        if y.dtype == torch.float32:
            torch.matmul(y, w.t(), out=logits)
        else:
            torch.mm(y, w.t(), out=logits, out_dtype=torch.float32)
