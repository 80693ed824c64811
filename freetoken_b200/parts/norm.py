"""RMSNorm, plain or Gemma form, with the residual sum fused in.

``y = x * rsqrt(mean(x^2) + eps) * (1 + w)`` in 32-bit (python/freetoken/kernel/triton/norm.py:65-75;
``1 + w`` only in the Gemma form, :69-72); the fused variant first adds the sub-layer output
to the residual stream (:101-112, python/freetoken/layers/norm.py:120-147).  The residual
stream itself is kept in 32-bit here, so the sum is never rounded.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import ParamSpec, PartSpec
from ..kernels import ops
from .base import NORMS, BuildEnv, Norm, RouteSum


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``, ``gemma`` (bool: multiply by ``1 + w``)."""

    takes_route_sum = True

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.gemma = bool(spec.get("gemma", True))

    def param_specs(self) -> Dict[str, ParamSpec]:
        init = ("normal", 0.0, 0.02) if self.gemma else ("normal", 1.0, 0.02)
        return {"weight": ParamSpec((self.size,), "float32", init, store="bfloat16")}

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.add_rmsnorm(x, None, self.params["weight"], self.eps, self.gemma, out)
        return out

    def add_forward(self, x: Optional[torch.Tensor], residual: torch.Tensor, out: torch.Tensor,
                    out_f32: Optional[torch.Tensor] = None,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if isinstance(x, RouteSum):
            ops.add_rmsnorm_routes(x.y, x.pos, x.top_k, x.shared, residual, self.params["weight"], self.eps,
                                   self.gemma, out, out_f32=out_f32, rows=rows)
        else:
            ops.add_rmsnorm(x, residual, self.params["weight"], self.eps, self.gemma, out,
                            out_f32=out_f32, rows=rows)
        return out
