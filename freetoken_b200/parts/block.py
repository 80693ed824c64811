"""Arrangement of the parts in one layer.

``prenorm_residual`` (python/freetoken/models/minimax_m3/model.py:53-61): every norm call is
"add the previous sub-layer's output to the residual, then norm the sum":
``r += x; h = N_in(r); a = mixer(h); r += a; h = N_post(r); f = ffn(h)`` and ``f`` travels to
the next layer's first norm.  The residual stream is 32-bit.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ..config.spec import PartSpec
from .base import BLOCKS, NORMS, Block, BuildEnv, FeedForward, Mixer, Part, StepState, as_rows, nvtx_range


@BLOCKS.register("prenorm_residual")
class PreNormResidualBlock(Block):
    """params: ``hidden``, ``norm`` (PartSpec used for both norms),
    ``input_norm_name``, ``post_norm_name`` (weight-name parts)."""

    def __init__(self, spec: PartSpec, env: BuildEnv, mixer: Mixer, ffn: FeedForward,
                 mixer_name: str, ffn_name: str):
        super().__init__(spec, env, mixer, ffn, mixer_name, ffn_name)
        self.hidden = int(spec["hidden"])
        self.input_norm = NORMS.build(spec["norm"], env)
        self.post_norm = NORMS.build(spec["norm"], env)
        self.input_norm_name = spec.get("input_norm_name", "input_layernorm")
        self.post_norm_name = spec.get("post_norm_name", "post_attention_layernorm")

    def children(self) -> Dict[str, Part]:
        return {self.input_norm_name: self.input_norm, self.mixer_name: self.mixer,
                self.post_norm_name: self.post_norm, self.ffn_name: self.ffn}

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        return n_tokens * self.hidden * (2 * item + 4)

    def forward(self, x: Optional[torch.Tensor], residual: torch.Tensor, step: StepState,
                cache: Any, writes_cache: bool) -> torch.Tensor:
        T = residual.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        h = ws.get("block.h", (T, self.hidden), dt, (cap, self.hidden))
        self.input_norm.add_forward(as_rows(x, self.input_norm), residual, h)
        with nvtx_range(f"mixer {self.mixer.kind}"):
            a = self.mixer.forward(h, step, cache, writes_cache)
        h2 = ws.get("block.h2", (T, self.hidden), dt, (cap, self.hidden))
        h32 = None
        if self.ffn.f32_input_needed(T) and dt != torch.float32:
            h32 = ws.get("block.h2_f32", (T, self.hidden), torch.float32, (cap, self.hidden))
        self.post_norm.add_forward(a, residual, h2, out_f32=h32)
        lazy = getattr(self.ffn, "forward_lazy", None)
        with nvtx_range(f"feed-forward {self.ffn.kind}"):
            return lazy(h2, step, h_f32=h32) if lazy is not None else self.ffn.forward(h2, step, h_f32=h32)
