"""Mixture-of-experts feed-forward: router, routed experts, optional shared expert.

Router, all in 32-bit (python/freetoken/models/minimax_m3/moe.py:71-81): logits =
``float32(h) @ W_g^T`` with ``W_g`` stored in 32-bit; ``s = sigmoid(logits)``; the choice is
``topk(s + bias)``, the weights are the unbiased ``s`` of the chosen experts divided by their
sum (+1e-20) and multiplied by ``routed_scaling_factor``.  The softmax form takes
``s = softmax(logits)`` (python/freetoken/moe/fused.py:27-31).

Experts (python/freetoken/moe/fused_nvfp4.py:317-344): routes sorted by expert, grouped
product with ``gate_up_proj [E, 2I, H]``, activation on the two halves, grouped product with
``down_proj [E, H, I]`` whose 32-bit accumulator is multiplied by the route weight
(python/freetoken/kernel/triton/fused_moe.py:292-296), then the sum over a token's routes in
route order with a 32-bit accumulator (:111-153).  The shared expert runs on the same input
and is added (moe.py:87-88).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import ParamSpec, PartSpec
from ..errors import ConfigError
from ..kernels import ops
from .base import FEED_FORWARDS, BuildEnv, FeedForward, Part, RouteSum, StepState
from .mlp import GatedMLP


SPLIT_ROUTER_PRODUCT = True  # long bfloat16 steps: router logits as three tensor-core products (see split_in_three)


def split_in_three(w: torch.Tensor) -> Optional[torch.Tensor]:
    """The float32 matrix ``w [E, H]`` as three bfloat16 matrices stacked to ``[3 E, H]`` whose sum is ``w``
    exactly (8 + 8 + 8 bits of its 24-bit mantissas), largest first; None where that is not so (values near
    the end of the exponent range).

    The router's input in a bfloat16 step is the norm's bfloat16 output, so a product of it with a
    bfloat16 piece is exact in 32 bits and ``x W^T`` is the 32-bit sum of three bfloat16 matrix products
    with 32-bit accumulators: the tensor cores take what the float32 product of the reference
    (python/freetoken/models/minimax_m3/moe.py:71-73) does on the CUDA cores, with the same products and
    other rounding of the partial sums only."""
    w = w.float()
    hi = w.to(torch.bfloat16)
    r1 = w - hi.float()
    mid = r1.to(torch.bfloat16)
    r2 = r1 - mid.float()
    lo = r2.to(torch.bfloat16)
    if not torch.equal((hi.float() + mid.float()) + lo.float(), w) or not torch.isfinite(w).all():
        return None
    return torch.cat([hi, mid, lo], dim=0).contiguous()


@FEED_FORWARDS.register("moe")
class MoE(FeedForward):
    """params: ``hidden``, ``inter``, ``n_experts``, ``top_k``, ``scoring`` ("sigmoid" |
    "softmax"), ``bias`` (bool), ``scale``, ``act``, ``alpha``, ``limit``,
    ``shared_inter`` (0 = no shared expert).  ``h_f32`` given to the forward calls of a bfloat16 model
    is ``float32(h)``, as a norm's ``out_f32`` is."""

    wants_f32_input = True

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden"])
        self.inter = int(spec["inter"])
        self.n_experts = int(spec["n_experts"])
        self.top_k = int(spec["top_k"])
        if not 1 <= self.top_k <= self.n_experts:
            raise ConfigError("moe: top_k must be in [1, n_experts]")
        self.scoring = spec.get("scoring", "sigmoid")
        if self.scoring not in ops.SCORE_CODES:
            raise ConfigError(f"moe: unknown scoring '{self.scoring}'")
        self.has_bias = bool(spec.get("bias", False))
        self.scale = float(spec.get("scale", 1.0))
        self.act = spec.get("act", "swigluoai")
        self.alpha = float(spec.get("alpha", 1.702))
        self.limit = float(spec.get("limit", 7.0))
        self.shared_inter = int(spec.get("shared_inter", 0) or 0)
        self._gate_pieces: Optional[torch.Tensor] = None
        self.shared: Optional[GatedMLP] = None
        if self.shared_inter:
            self.shared = GatedMLP(PartSpec("gated_mlp", dict(
                hidden=self.hidden, inter=self.shared_inter, act=self.act, alpha=self.alpha,
                limit=self.limit)), env, tag="moe.shared")

    def param_specs(self) -> Dict[str, ParamSpec]:
        out = {
            "gate.weight": ParamSpec((self.n_experts, self.hidden), "float32"),
            "experts.gate_up_proj": ParamSpec((self.n_experts, 2 * self.inter, self.hidden)),
            "experts.down_proj": ParamSpec((self.n_experts, self.hidden, self.inter)),
        }
        if self.has_bias:
            out["e_score_correction_bias"] = ParamSpec((self.n_experts,), "float32", ("normal", 0.0, 0.01))
        return out

    def children(self) -> Dict[str, Part]:
        return {"shared_experts": self.shared} if self.shared is not None else {}

    def f32_input_needed(self, n_tokens: int) -> bool:
        # long bfloat16 steps take the router product from the bfloat16 rows themselves
        return not (self._gate_pieces is not None and self.env.dtype == torch.bfloat16
                    and not ops.moe_route_fits(n_tokens, self.hidden, self.n_experts, self.top_k))

    def bind(self, tensors) -> None:
        super().bind(tensors)
        self._gate_pieces = None
        if self.env.dtype == torch.bfloat16 and SPLIT_ROUTER_PRODUCT:
            self._gate_pieces = split_in_three(self.params["gate.weight"])

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        T, k, H, I, E = n_tokens, self.top_k, self.hidden, self.inter, self.n_experts
        routed = T * k * ((2 * H + I) * item + 4 * 4)  # expert-ordered input, activation, output; ids, weights, sort
        return routed + T * (H * (4 + item) + E * 4 * 4) + (2 * E + 1) * 4  # (logits, and their three pieces)

    def forward(self, h: torch.Tensor, step: StepState, h_f32: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.forward_lazy(h, step, h_f32).rows()

    def _few_tokens(self, h, h_f32, step, logits, ids, wts, bias) -> RouteSum:
        """Steps of up to four tokens: the routes stay in token order (no sort, no gathered copy of the
        activations) and each route's expert rows are streamed by the few-token kernels."""
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        k, R = self.top_k, T * self.top_k
        ops.moe_route(h_f32, self.params["gate.weight"], bias, k, self.scoring, self.scale, logits, ids, wts)
        record = self.env.shared.get("record_expert_counts")
        if record is not None:
            record.append(torch.bincount(ids.view(-1).long(), minlength=self.n_experts).to(torch.int32))
        if "moe.pos.identity" not in self.env.shared:
            self.env.shared["moe.pos.identity"] = torch.arange(64 * 64, dtype=torch.int32, device=self.env.device)
        pos = self.env.shared["moe.pos.identity"][:R]
        a = ws.get("moe.act", (R, self.inter), dt, (cap * k, self.inter))
        ops.moe_small_gate_up(h, ids, self.params["experts.gate_up_proj"], self.act, self.alpha, self.limit, a)
        y = ws.get("moe.y", (R, self.hidden), dt, (cap * k, self.hidden))
        ops.moe_small_down(a, ids, wts, self.params["experts.down_proj"], y)
        shared = self.shared.forward(h, step) if self.shared is not None else None
        out = ws.get("moe.out", (T, self.hidden), dt, (cap, self.hidden))
        return RouteSum(y, pos, k, shared, T, out)

    def forward_lazy(self, h: torch.Tensor, step: StepState, h_f32: Optional[torch.Tensor] = None) -> RouteSum:
        """The experts' rows and where each token's routes lie among them; the sum over a token's routes
        is left to the consumer (the next norm takes it together with the residual sum)."""
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        k, E, R = self.top_k, self.n_experts, T * self.top_k
        if h_f32 is None and self.f32_input_needed(T):
            if h.dtype == torch.float32:
                h_f32 = h
            else:
                h_f32 = ws.get("moe.h_f32", (T, self.hidden), torch.float32, (cap, self.hidden))
                ops.cast(h, h_f32)
        logits = ws.get("moe.logits", (T, E), torch.float32, (cap, E))
        ids = ws.get("moe.ids", (T, k), torch.int32, (cap, k))
        wts = ws.get("moe.weights", (T, k), torch.float32, (cap, k))
        counts = ws.get("moe.counts", (E,), torch.int32)
        offsets = ws.get("moe.offsets", (E + 1,), torch.int32)
        routes = ws.get("moe.routes", (R,), torch.int32, (cap * k,))
        pos = ws.get("moe.pos", (R,), torch.int32, (cap * k,))
        bias = self.params.get("e_score_correction_bias")
        if (dt == torch.bfloat16 and ops.moe_small_fits(T, self.hidden, self.inter, k)
                and ops.moe_route_fits(T, self.hidden, E, k)):
            return self._few_tokens(h, h_f32, step, logits, ids, wts, bias)
        if ops.moe_route_fits(T, self.hidden, E, k):  # small steps: logits, choice and sort in one launch
            ops.moe_route(h_f32, self.params["gate.weight"], bias, k, self.scoring, self.scale, logits, ids, wts,
                          counts, offsets, routes, pos)
        elif self._gate_pieces is not None and h.dtype == torch.bfloat16:
            # the router reads float32(h): the three products below are exact, their 32-bit sums are the logits
            pieces = ws.get("moe.logit_pieces", (T, 3 * E), torch.float32, (cap, 3 * E))
            torch.mm(h, self._gate_pieces.t(), out_dtype=torch.float32, out=pieces)
            ops.router_topk(pieces, bias, k, self.scoring, self.scale, ids, wts, n_parts=3)
            ops.moe_permute(ids, E, counts, offsets, routes, pos)
        else:
            torch.matmul(h_f32, self.params["gate.weight"].t(), out=logits)
            ops.router_topk(logits, bias, k, self.scoring, self.scale, ids, wts)
            ops.moe_permute(ids, E, counts, offsets, routes, pos)
        record = self.env.shared.get("record_expert_counts")
        if record is not None:  # measurement hook: which experts a step touched, layer by layer
            record.append(counts.clone())
        a = ws.get("moe.act", (R, self.inter), dt, (cap * k, self.inter))
        if ops.moe_gemm1_gather_fits(dt, self.hidden, self.inter, E, R) and h.is_contiguous():
            # the gate/up kernel reads each expert's rows where they lie: no copy into expert order
            ops.moe_gemm1_act_gather(h, routes, k, self.params["experts.gate_up_proj"], offsets, self.act,
                                     self.alpha, self.limit, a)
        else:
            x = ws.get("moe.x", (R, self.hidden), dt, (cap * k, self.hidden))
            ops.moe_gather(h, routes, k, x)
            ops.moe_gemm1_act(x, self.params["experts.gate_up_proj"], offsets, self.act, self.alpha,
                              self.limit, a)
        y = ws.get("moe.y", (R, self.hidden), dt, (cap * k, self.hidden))
        ops.moe_gemm2(a, self.params["experts.down_proj"], offsets, routes, wts.view(-1), y)
        shared = self.shared.forward(h, step) if self.shared is not None else None
        out = ws.get("moe.out", (T, self.hidden), dt, (cap, self.hidden))
        return RouteSum(y, pos, k, shared, T, out)
