"""Dense gated feed-forward: ``down(act(gate(h), up(h)))``.

``gate_up_proj`` holds the gate rows then the up rows; the activation works on the two
un-interleaved halves (python/freetoken/models/minimax_m3/mlp.py:54-59).  ``silu`` is
``g sigmoid(g) u``; ``swigluoai`` clamps first: ``g' = min(g, limit)``,
``u' = clamp(u, -limit, limit)``, ``g' sigmoid(alpha g') (u' + 1)``
(python/freetoken/kernel/triton/activation.py:96-98,103-107).  The two projections are
library matrix products (python/freetoken/layers/linear.py:31-32), the activation is ours.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import ParamSpec, PartSpec
from ..errors import ConfigError
from ..kernels import ops
from .base import FEED_FORWARDS, BuildEnv, FeedForward, StepState


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """params: ``hidden``, ``inter``, ``act`` ("silu" | "swigluoai"), ``alpha``, ``limit``."""

    def __init__(self, spec: PartSpec, env: BuildEnv, tag: str = "mlp"):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden"])
        self.inter = int(spec["inter"])
        self.act = spec.get("act", "swigluoai")
        if self.act not in ops.ACT_CODES:
            raise ConfigError(f"gated_mlp: unknown activation '{self.act}'")
        self.alpha = float(spec.get("alpha", 1.702))
        self.limit = float(spec.get("limit", 7.0))
        self.tag = tag

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "gate_up_proj.weight": ParamSpec((2 * self.inter, self.hidden)),
            "down_proj.weight": ParamSpec((self.hidden, self.inter)),
        }

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        return n_tokens * (3 * self.inter + self.hidden) * item

    def forward(self, h: torch.Tensor, step: StepState, h_f32: Optional[torch.Tensor] = None) -> torch.Tensor:
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        gu = ws.get(f"{self.tag}.gate_up", (T, 2 * self.inter), dt, (cap, 2 * self.inter))
        ops.linear(h, self.params["gate_up_proj.weight"], gu)
        a = ws.get(f"{self.tag}.act", (T, self.inter), dt, (cap, self.inter))
        ops.act_and_mul(gu, a, self.act, self.alpha, self.limit)
        out = ws.get(f"{self.tag}.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(a, self.params["down_proj.weight"], out)
        return out
