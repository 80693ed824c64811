"""Seeded random weights.

Two forms.  :func:`write_model_folder` makes a model folder (``config.json`` and
``model.safetensors`` with the architecture's checkpoint names) on the CPU from a
configuration and a seed; the engine, the replay tool and the plain test implementation
then read the same file.  :func:`random_tensors_on_device` fills the model's tensors on
the device without touching the disk, for models too large to write (the benchmark's
90 GB); it is the counterpart of the reference's dummy weights
(python/freetoken/engine/engine.py:241-267), seeded per tensor instead of globally so the
values do not depend on creation order.

Distributions come from each parameter's ``init``: weights ``N(0, 0.02)``, norm scales
``N(0, 0.02)`` in the Gemma (1+w) form or ``1 + N(0, 0.02)`` otherwise, router bias
``N(0, 0.01)``.
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping, Optional

import torch

from ..config.spec import ParamSpec
from .binder import FusionRule, target_dtype, unfuse
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "int32": torch.int32}


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def _draw(ps: ParamSpec, gen: torch.Generator, device, dtype: torch.dtype) -> torch.Tensor:
    kind = ps.init[0]
    if kind == "zeros":
        return torch.zeros(ps.shape, dtype=dtype, device=device)
    if kind == "ones":
        return torch.ones(ps.shape, dtype=dtype, device=device)
    if kind == "normal":
        _, mean, std = ps.init
        if not dtype.is_floating_point:
            return torch.zeros(ps.shape, dtype=dtype, device=device)
        t = torch.empty(ps.shape, dtype=torch.float32 if dtype != torch.bfloat16 else dtype, device=device)
        t.normal_(mean, std, generator=gen)
        return t.to(dtype)
    raise ValueError(f"unknown init {ps.init!r}")


def random_tensors_cpu(expected: Mapping[str, ParamSpec], seed: int, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Every expected tensor in its storage dtype, drawn in float32 and rounded.  ``device`` may name
    a CUDA device to draw there (large models; the values then differ from the CPU's draws)."""
    out = {}
    for name, ps in expected.items():
        gen = torch.Generator(device=device).manual_seed(tensor_seed(seed, name))
        t = _draw(ps, gen, device, torch.float32 if ps.dtype != "int32" else torch.int32)
        out[name] = t.to(_STORE[ps.storage_dtype()])
    return out


def random_tensors_on_device(expected: Mapping[str, ParamSpec], seed: int, compute_dtype: torch.dtype,
                             device: torch.device) -> Dict[str, torch.Tensor]:
    out = {}
    for name, ps in expected.items():
        gen = torch.Generator(device=device).manual_seed(tensor_seed(seed, name))
        out[name] = _draw(ps, gen, device, target_dtype(ps, compute_dtype))
    return out


def write_model_folder(config: Mapping[str, Any], folder: str, seed: int, fused_names: bool = False,
                       device: str = "cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` for the architecture ``config`` names.

    ``config`` is the config.json content.  Tensors carry the checkpoint's per-part names
    (``q_proj``, ``experts.3.w1`` ...) unless ``fused_names`` asks for the model's own.  ``device``:
    where the values are drawn (a CUDA device makes gigabytes of weights in seconds; the file is the
    reference either way, whoever reads it)."""
    from ..engine.build import describe_model  # late import: engine imports weights

    arch, typed, spec, expected = describe_model(config)
    tensors = random_tensors_cpu(expected, seed, device)
    if not fused_names:
        for rule in arch.fusion_rules(typed):
            if rule.target in tensors:
                tensors.update(unfuse(rule, tensors.pop(rule.target)))  # views: the writer copies tensor by tensor
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config), f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
