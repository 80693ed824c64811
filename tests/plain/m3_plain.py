"""Plain, slow MiniMax-M3: whole sequences, no cache, no batching, one function per part.

Written from the reference's formulas (file:line cited in each function; paths are
relative to the reference project).  The reference's own model code cannot run a
forward pass on a CPU (its norm, rope, attention and expert kernels are Triton or
library CUDA code), so the whole model rests on the formulas; part by part it is
compared with what of the reference does run on a CPU (its router and rope table,
its tests' PyTorch oracles for paged attention, block-sparse attention and fused
experts, and its Triton norm, rope and activation kernels under Triton's CPU
interpreter) in ``tests/golden/make_golden.py``, whose recorded outputs
``tests/test_plain.py`` checks again without the reference.

It shares no code with ``freetoken_b200``: it parses config.json and reads the
safetensors file (through the ``safetensors`` package) itself.

``rounding="bfloat16"`` rounds at the places where the reference's serving path
stores bfloat16 (marked ``rnd`` below); ``rounding=None`` keeps everything in the
working dtype (float32 or float64).
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- config
@dataclass
class PlainConfig:
    vocab: int
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    rotary_dim: int
    theta: float
    eps: float
    qk_norm: bool
    gemma: bool
    tied: bool
    act: str
    alpha: float
    limit: float
    experts: int
    top_k: int
    inter: int
    dense_inter: int
    shared_inter: int
    n_shared: int
    scale: float
    bias: bool
    scoring: str
    moe_layers: List[bool]
    sparse_layers: List[bool]
    sparse_block: int = 0
    sparse_topk: int = 0
    sparse_local: int = 0
    sparse_init: int = 0


def read_config(folder: str) -> PlainConfig:
    """Keys and defaults: python/freetoken/models/minimax_m3/args.py:135-254, config.py:61-198."""
    with open(os.path.join(folder, "config.json")) as f:
        raw = json.load(f)
    c = raw.get("text_config", raw)
    layers = c["num_hidden_layers"]
    heads = c["num_attention_heads"]
    head_dim = c.get("head_dim") or c["hidden_size"] // heads
    rotary = c.get("rotary_dim")
    if rotary is None:
        rotary = int(head_dim * c.get("partial_rotary_factor", 1.0))
    theta = c.get("rope_theta")
    if theta is None:
        theta = (c.get("rope_parameters") or {}).get("rope_theta", 10000.0)
    freq = c.get("moe_layer_freq")
    if freq is None and c.get("mlp_layer_types") is not None:
        freq = [1 if t == "sparse" else 0 for t in c["mlp_layer_types"]]
    experts = c.get("num_local_experts", 0) or 0
    moe_layers = [bool(f) for f in freq[:layers]] if freq else [experts > 0] * layers
    sp = c.get("sparse_attention_config") or {}
    sparse_layers = [False] * layers
    if sp.get("use_sparse_attention"):
        sf = sp.get("sparse_attention_freq")
        sparse_layers = [bool(f) for f in sf[:layers]] if sf else [True] * layers
    inter = c["intermediate_size"]
    act = c.get("hidden_act", "swigluoai")
    if act == "silu" and ("swiglu_alpha" in c or "swiglu_limit" in c):
        act = "swigluoai"  # the native key shape's spelling of the clamped form (config.py:128-145)
    return PlainConfig(
        vocab=c["vocab_size"],
        hidden=c["hidden_size"],
        layers=layers,
        heads=heads,
        kv_heads=c.get("num_key_value_heads") or heads,
        head_dim=head_dim,
        rotary_dim=rotary,
        theta=float(theta),
        eps=float(c["rms_norm_eps"]),
        qk_norm=bool(c.get("use_qk_norm", True)),
        gemma=bool(c.get("use_gemma_norm", True)),
        tied=bool(c.get("tie_word_embeddings", False)),
        act=act,
        alpha=float(c.get("swiglu_alpha", 1.702)),
        limit=float(c.get("swiglu_limit", 7.0)),
        experts=experts,
        top_k=c.get("num_experts_per_tok", 0) or 0,
        inter=inter,
        dense_inter=c.get("dense_intermediate_size") or inter,
        shared_inter=c.get("shared_intermediate_size") or inter,
        n_shared=c.get("n_shared_experts", 0) or 0,
        scale=float(c.get("routed_scaling_factor", 1.0)),
        bias=bool(c.get("use_routing_bias", False)),
        scoring=c.get("scoring_func", "sigmoid"),
        moe_layers=moe_layers,
        sparse_layers=sparse_layers,
        sparse_block=int(sp.get("sparse_block_size", 0) or 0),
        sparse_topk=int(sp.get("sparse_topk_blocks", 0) or 0),
        sparse_local=int(sp.get("sparse_local_block", 0) or 0),
        sparse_init=int(sp.get("sparse_init_block", 0) or 0),
    )


class _WidenOnRead(dict):
    """Tensors kept as the file stores them and widened to the working dtype when read: for models
    whose weights would not fit twice into memory."""

    def __init__(self, dtype: torch.dtype):
        super().__init__()
        self.dtype = dtype

    def __getitem__(self, name):
        return super().__getitem__(name).to(self.dtype)

    def get(self, name, default=None):
        return self[name] if name in self else default


def read_weights(folder: str, dtype: torch.dtype, lazy: bool = False) -> Dict[str, torch.Tensor]:
    """Tensors by checkpoint name (python/freetoken/models/minimax_m3/weight.py:182-246);
    the ``language_model.`` prefix is dropped.  ``lazy`` widens a tensor each time it is read instead
    of once for all."""
    from safetensors.torch import load_file

    out = _WidenOnRead(dtype) if lazy else {}
    for name, t in load_file(os.path.join(folder, "model.safetensors")).items():
        if name.startswith("language_model."):
            name = name[len("language_model."):]
        if lazy:
            dict.__setitem__(out, name, t)
        else:
            out[name] = t.to(dtype)
    return out


# A discrete choice (expert, key block) counts as safe against bfloat16 rounding when its gap is this
# many times the movement that rounding causes in the plain model's own scores.
SAFETY = 4.0


# --------------------------------------------------------------------------- parts
def _rnd(x: torch.Tensor, rounding: Optional[str]) -> torch.Tensor:
    if rounding == "bfloat16":
        return x.to(torch.bfloat16).to(x.dtype)
    return x


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, gemma: bool) -> torch.Tensor:
    """``y = x * rsqrt(mean(x^2) + eps) * (1 + w)`` over the last dim, in that multiply
    order (python/freetoken/kernel/triton/norm.py:65-75; ``1 + w`` at :69-72)."""
    scale = w + 1.0 if gemma else w
    inv = torch.rsqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return x * inv * scale


def rope_table(rotary_dim: int, theta: float, positions: int, dtype: torch.dtype):
    """cos and sin ``[positions, rotary_dim/2]`` (python/freetoken/layers/rotary.py:49-59):
    ``inv_freq_i = 1 / theta^(2i/rotary_dim)``, angle = position * inv_freq, both in float32."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim))
    t = torch.arange(positions, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def apply_rope(u: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Partial NeoX rotation of ``u [T, heads, D]`` (python/freetoken/kernel/triton/rope.py:51-78):
    for ``d < half``: ``o[d] = u[d] cos_d - u[d+half] sin_d``, ``o[d+half] = u[d+half] cos_d + u[d] sin_d``;
    dims >= rotary_dim pass through."""
    if rotary_dim == 0:
        return u
    half = rotary_dim // 2
    a, b, rest = u[..., :half], u[..., half:rotary_dim], u[..., rotary_dim:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: int,
                     rounding: Optional[str] = None, allowed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(q k^T / sqrt(D))`` over keys ``j <= t`` of the same sequence; q head ``h``
    reads kv head ``h // group`` (python/freetoken/kernel/triton/attention.py:74,102,118-137;
    scale python/freetoken/attention/triton.py:163).  ``allowed [kv_heads, T, T]`` further
    restricts the keys (block-sparse layers).  Probabilities are rounded before ``P V`` in the
    serving path (attention.py:252,573)."""
    T, H, D = q.shape
    out = torch.empty_like(q)
    causal = torch.ones(T, T, dtype=torch.bool).tril()
    for h in range(H):
        kh = h // group
        s = (q[:, h] @ k[:, kh].T) * (D ** -0.5)
        mask = causal if allowed is None else causal & allowed[kh]
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = _rnd(p, rounding) @ v[:, kh]
    return out


def sparse_block_selection(iq: torch.Tensor, ik: torch.Tensor, block: int, topk: int,
                           local: int, init: int, margins: Optional[list] = None) -> torch.Tensor:
    """Which keys each (kv head, query) may read in a block-sparse layer -> bool ``[Hi, T, T]``.

    Block score = max over the block's visible positions of ``iq . ik``, unscaled
    (python/freetoken/kernel/triton/minimax_m3_sparse.py:152-170); the first ``init`` blocks
    score 1e30, the newest ``local`` blocks 1e29 (local wins), the ``min(topk, visible)``
    highest are taken (:232-244,269-284).  Ties go to the lower block index."""
    T, Hi, _ = iq.shape
    scores = torch.einsum("thd,sd->hts", iq, ik)
    pos = torch.arange(T)
    scores = scores.masked_fill(pos[None, None, :] > pos[None, :, None], float("-inf"))
    nblocks = (T + block - 1) // block
    pad = nblocks * block - T
    if pad:
        scores = torch.nn.functional.pad(scores, (0, pad), value=float("-inf"))
    bscore = scores.view(Hi, T, nblocks, block).amax(-1)
    allowed = torch.zeros(Hi, T, T, dtype=torch.bool)
    for h in range(Hi):
        for t in range(T):
            nb = t // block + 1
            s = bscore[h, t, :nb].clone()
            s = torch.where(torch.isnan(s), torch.full_like(s, -1e30), s)
            if init:
                s[: min(init, nb)] = 1e30
            s[max(0, nb - local):] = 1e29
            order = sorted(range(nb), key=lambda b: (-float(s[b]), b))
            for b in order[: min(topk, nb)]:
                allowed[h, t, b * block: min((b + 1) * block, T)] = True
            if margins is not None and nb > topk:  # gap between the last taken and the first dropped block
                margins.append((t, float(s[order[topk - 1]] - s[order[topk]])))
    if margins is not None:
        margins.append(("scores", bscore.clone()))
    return allowed


def activation(g: torch.Tensor, u: torch.Tensor, act: str, alpha: float, limit: float) -> torch.Tensor:
    """``silu``: ``g sigmoid(g) u``; ``swigluoai``: ``g' = min(g, limit)``, ``u' = clamp(u, +-limit)``,
    ``g' sigmoid(alpha g') (u' + 1)`` (python/freetoken/kernel/triton/activation.py:96-98,103-107)."""
    if act == "silu":
        return g * torch.sigmoid(g) * u
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    return g * torch.sigmoid(alpha * g) * (u + 1.0)


def gated_mlp(h, w_gate, w_up, w_down, cfg: PlainConfig, rounding):
    """``down(act(gate(h), up(h)))`` (python/freetoken/models/minimax_m3/mlp.py:54-59)."""
    g = _rnd(h @ w_gate.T, rounding)
    u = _rnd(h @ w_up.T, rounding)
    a = _rnd(activation(g, u, cfg.act, cfg.alpha, cfg.limit), rounding)
    return _rnd(a @ w_down.T, rounding)


def router(h: torch.Tensor, w_gate: torch.Tensor, bias: Optional[torch.Tensor], cfg: PlainConfig):
    """Expert choice and weights, all in float32
    (python/freetoken/models/minimax_m3/moe.py:71-81; softmax form python/freetoken/moe/fused.py:27-31).
    Ties go to the lower expert index."""
    logits = h.float() @ w_gate.float().T
    if cfg.scoring == "sigmoid":
        scores = torch.sigmoid(logits)
    else:
        scores = torch.softmax(logits, dim=-1)
    choice = scores + bias.float() if bias is not None else scores
    ids = torch.argsort(choice, dim=-1, descending=True, stable=True)[:, : cfg.top_k]
    w = scores.gather(-1, ids)
    if cfg.scoring == "sigmoid":
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    else:
        w = w / w.sum(-1, keepdim=True)
    return w * cfg.scale, ids


def router_margin(h: torch.Tensor, w_gate: torch.Tensor, bias: Optional[torch.Tensor], cfg: PlainConfig):
    """Per token, the gap between the last chosen and the first rejected expert's choice score,
    expressed in units of the router logit (the gap divided by the score's slope there:
    ``s (1 - s)`` for sigmoid, ``p`` for softmax).  A gap below the noise that reduced
    precision puts on the logits means that run may legitimately pick another expert."""
    logits = h.float() @ w_gate.float().T
    scores = torch.sigmoid(logits) if cfg.scoring == "sigmoid" else torch.softmax(logits, dim=-1)
    choice = scores + bias.float() if bias is not None else scores
    if cfg.top_k >= choice.shape[-1]:
        return torch.full((h.shape[0],), float("inf"))
    srt, idx = torch.sort(choice, dim=-1, descending=True)
    gap = srt[:, cfg.top_k - 1] - srt[:, cfg.top_k]
    s = scores.gather(-1, idx[:, cfg.top_k - 1: cfg.top_k])[:, 0]
    slope = s * (1 - s) if cfg.scoring == "sigmoid" else s
    return gap / slope.clamp_min(1e-12)


def routed_experts(h, ids, w, W, prefix: str, cfg: PlainConfig, rounding):
    """``out_t = sum_j (act(h_t W1[e]^T) W2[e]^T) w[t, j]`` with ``e = ids[t, j]``: the weight multiplies
    the unrounded product, the sum runs over the routes in route order
    (python/freetoken/moe/fused_nvfp4.py:317-344; python/freetoken/kernel/triton/fused_moe.py:287-296,142-152)."""
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        acc = torch.zeros(h.shape[1], dtype=h.dtype)
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            x = h[t: t + 1]
            g = _rnd(x @ W[f"{prefix}experts.{e}.w1.weight"].T, rounding)
            u = _rnd(x @ W[f"{prefix}experts.{e}.w3.weight"].T, rounding)
            a = _rnd(activation(g, u, cfg.act, cfg.alpha, cfg.limit), rounding)
            y = _rnd((a @ W[f"{prefix}experts.{e}.w2.weight"].T) * w[t, j].to(h.dtype), rounding)
            acc = acc + y[0]
        out[t] = _rnd(acc, rounding)
    return out


def moe_block(h, W, prefix: str, cfg: PlainConfig, rounding, margins: Optional[list] = None):
    """Router, routed experts (:func:`routed_experts`), plus the shared expert on the same input
    (python/freetoken/models/minimax_m3/moe.py:83-88)."""
    bias = W.get(prefix + "e_score_correction_bias") if cfg.bias else None
    w, ids = router(h, W[prefix + "gate.weight"], bias, cfg)
    if margins is not None:
        margins.append((router_margin(h, W[prefix + "gate.weight"], bias, cfg),
                        h.float() @ W[prefix + "gate.weight"].float().T))
    out = routed_experts(h, ids, w, W, prefix, cfg, rounding)
    if cfg.n_shared > 0:
        sh = gated_mlp(h, W[prefix + "shared_experts.gate_proj.weight"],
                       W[prefix + "shared_experts.up_proj.weight"],
                       W[prefix + "shared_experts.down_proj.weight"], cfg, rounding)
        out = _rnd(out + sh, rounding)
    return out


def attention_layer(h, W, prefix: str, cfg: PlainConfig, cos, sin, sparse: bool, rounding,
                    sel_margins: Optional[list] = None):
    """qkv projection, per-head q/k norm, partial rope, causal softmax attention, output
    projection (python/freetoken/models/minimax_m3/attention.py:79-119)."""
    T = h.shape[0]
    q = _rnd(h @ W[prefix + "q_proj.weight"].T, rounding).view(T, cfg.heads, cfg.head_dim)
    k = _rnd(h @ W[prefix + "k_proj.weight"].T, rounding).view(T, cfg.kv_heads, cfg.head_dim)
    v = _rnd(h @ W[prefix + "v_proj.weight"].T, rounding).view(T, cfg.kv_heads, cfg.head_dim)
    if cfg.qk_norm:
        q = rms_norm(q, W[prefix + "q_norm.weight"], cfg.eps, cfg.gemma)
        k = rms_norm(k, W[prefix + "k_norm.weight"], cfg.eps, cfg.gemma)
    q = _rnd(apply_rope(q, cos, sin, cfg.rotary_dim), rounding)
    k = _rnd(apply_rope(k, cos, sin, cfg.rotary_dim), rounding)
    allowed = None
    if sparse:
        iq = _rnd(h @ W[prefix + "index_q_proj.weight"].T, rounding).view(T, cfg.kv_heads, cfg.head_dim)
        ik = _rnd(h @ W[prefix + "index_k_proj.weight"].T, rounding).view(T, 1, cfg.head_dim)
        iq = rms_norm(iq, W[prefix + "index_q_norm.weight"], cfg.eps, cfg.gemma)
        ik = rms_norm(ik, W[prefix + "index_k_norm.weight"], cfg.eps, cfg.gemma)
        iq = _rnd(apply_rope(iq, cos, sin, cfg.rotary_dim), rounding)
        ik = _rnd(apply_rope(ik, cos, sin, cfg.rotary_dim), rounding)
        allowed = sparse_block_selection(iq, ik[:, 0], cfg.sparse_block, cfg.sparse_topk,
                                         cfg.sparse_local, cfg.sparse_init, sel_margins)
    o = _rnd(causal_attention(q, k, v, cfg.heads // cfg.kv_heads, rounding, allowed), rounding)
    return _rnd(o.reshape(T, -1) @ W[prefix + "o_proj.weight"].T, rounding)


# --------------------------------------------------------------------------- model
class PlainM3:
    def __init__(self, folder: str, dtype: torch.dtype = torch.float32, rounding: Optional[str] = None,
                 lazy: bool = False):
        self.cfg = read_config(folder)
        self.W = read_weights(folder, dtype, lazy)
        self.dtype = dtype
        self.rounding = rounding

    def router_margins(self, tokens: Sequence[int]) -> torch.Tensor:
        """``[T]``: how safe each token's discrete choices are against bfloat16 rounding; values at or
        below ``tests.helpers.NEAR_TIE`` mean "may legitimately differ in bfloat16".

        The model is run twice, in the working precision and with bfloat16 rounding.  Per MoE layer
        the router gap of a token (in logit units) is set against how far the rounding moved that
        token's router logits; per block-sparse layer the gap between the last taken and the first
        dropped block score against how far its block scores moved.  A choice whose gap is less than
        ``SAFETY`` times that movement (the engine rounds in another order than this emulation, so
        its noise is of the same size but not the same sign) is reported as 0, otherwise as the gap."""
        exact_r, exact_s, rough_r, rough_s = [], [], [], []
        self.hidden_states(tokens, margins=exact_r, sel_margins=exact_s)
        keep = self.rounding
        self.rounding = "bfloat16"
        try:
            self.hidden_states(tokens, margins=rough_r, sel_margins=rough_s)
        finally:
            self.rounding = keep
        T = len(tokens)
        out = torch.full((T,), float("inf"))
        for (gap, logits), (_, logits_b) in zip(exact_r, rough_r):
            noise = (logits - logits_b).abs().max(-1).values
            safe = gap > SAFETY * noise + 1e-4
            out = torch.minimum(out, torch.where(safe, gap, torch.zeros_like(gap)))
        scores = [x[1] for x in exact_s if x[0] == "scores"]
        scores_b = [x[1] for x in rough_s if x[0] == "scores"]
        gaps = [x for x in exact_s if x[0] != "scores"]
        layer = 0
        per_layer = len(gaps) // max(1, len(scores))
        for i, (t, gap) in enumerate(gaps):
            layer = min(i // max(1, per_layer), len(scores) - 1)
            a, b = scores[layer][:, t], scores_b[layer][:, t]
            ok = torch.isfinite(a) & torch.isfinite(b)
            noise = float((a[ok] - b[ok]).abs().max()) if ok.any() else 0.0
            if gap <= SAFETY * noise + 1e-3:
                out[t] = 0.0
        return out

    def hidden_states(self, tokens: Sequence[int], return_layers: bool = False, margins: Optional[list] = None,
                      sel_margins: Optional[list] = None):
        """Residual stream after the last layer, before the final norm, ``[T, hidden]``.

        Pre-norm with the residual carried beside the sub-layer output
        (python/freetoken/models/minimax_m3/model.py:53-61,75-80): ``r <- r + x``; ``h = norm(r)``.
        The sum is kept unrounded here (the reference stores it in bfloat16 but norms the
        unrounded sum, python/freetoken/kernel/triton/norm.py:101-112)."""
        cfg, W, rd = self.cfg, self.W, self.rounding
        ids = torch.as_tensor(list(tokens), dtype=torch.long)
        T = ids.shape[0]
        cos, sin = rope_table(cfg.rotary_dim, cfg.theta, T, self.dtype) if cfg.rotary_dim else (None, None)
        r = W["model.embed_tokens.weight"][ids]  # no scaling (model.py:76)
        per_layer = []
        for l in range(cfg.layers):
            p = f"model.layers.{l}."
            h = _rnd(rms_norm(r, W[p + "input_layernorm.weight"], cfg.eps, cfg.gemma), rd)
            a = attention_layer(h, W, p + "self_attn.", cfg, cos, sin, cfg.sparse_layers[l], rd, sel_margins)
            r = r + a
            h = _rnd(rms_norm(r, W[p + "post_attention_layernorm.weight"], cfg.eps, cfg.gemma), rd)
            if cfg.moe_layers[l]:
                f = moe_block(h, W, p + "block_sparse_moe.", cfg, rd, margins)
            else:
                f = gated_mlp(h, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                              W[p + "mlp.down_proj.weight"], cfg, rd)
            r = r + f
            per_layer.append(r.clone())
        return (r, per_layer) if return_layers else r

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """Logits at every position ``[T, vocab]`` (final norm + head,
        python/freetoken/layers/embedding.py:103-113; tied head uses the embedding, :81-90)."""
        cfg, W = self.cfg, self.W
        r = self.hidden_states(tokens)
        y = _rnd(rms_norm(r, W["model.norm.weight"], cfg.eps, cfg.gemma), self.rounding)
        head = W["model.embed_tokens.weight"] if cfg.tied else W["lm_head.weight"]
        return y @ head.T

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        """``n`` greedy tokens; the lowest index wins a tie (python/freetoken/engine/sample.py:78-79)."""
        toks = list(prompt)
        out = []
        for _ in range(n):
            nxt = int(torch.argmax(self.logits(toks)[-1]))
            out.append(nxt)
            toks.append(nxt)
        return out


# --------------------------------------------------------------------------- sampling
def sample_reference(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """Temperature sampling by inverse CDF (python/freetoken/engine/sample.py:63-73;
    python/freetoken/kernel/triton/sampling.py:123-143,342-425): ``p = softmax(logits / max(T, 1e-6))``;
    top-k keeps the k largest, then top-p keeps the smallest prefix of the sorted probabilities whose
    mass reaches p (:576-618); the kept probabilities are walked in index order and the first index
    whose running sum exceeds ``u * total`` is drawn."""
    x = logits.double() / max(temperature, 1e-6)
    p = torch.softmax(x, dim=-1)
    keep = torch.ones_like(p, dtype=torch.bool)
    order = torch.argsort(p, descending=True, stable=True)
    if 0 < top_k < p.numel():
        keep[order[top_k:]] = False
    if top_p < 1.0:
        ps = p[order] * keep[order]
        csum = torch.cumsum(ps, 0)
        total = ps.sum()
        # smallest prefix whose mass reaches top_p * total
        n = int((csum < top_p * total).sum()) + 1
        keep[order[n:]] = False
    p = p * keep
    target = u * float(p.sum())
    run = 0.0
    last = 0
    for i in range(p.numel()):
        if p[i] > 0:
            run += float(p[i])
            last = i
            if run > target:
                return i
    return last
