"""Binds checkpoint tensors to the model's tensors by name.

The model states what it expects (full name -> shape and dtype policy); the architecture
states how checkpoint tensors combine into them (:class:`FusionRule`) and which name
prefixes to drop.  Everything wrong with a folder is collected and reported in ONE
:class:`WeightError` that lists missing tensors, unexpected tensors and wrong shapes.
The reference reports these three as a ``KeyError``, a ``RuntimeError`` and an
``AssertionError`` from three places (python/freetoken/layers/base.py:32-53).

dtype policy: ``"compute"`` tensors are converted to the engine's dtype (bfloat16 in the
serving path); ``"float32"`` tensors (router matrix and bias, norm scales) stay or become
32-bit in both paths, like the reference's router (python/freetoken/models/minimax_m3/moe.py:39-49);
``"int32"`` tables stay integers.  A float parameter cannot be bound from an integer tensor.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..config.spec import ParamSpec
from ..errors import WeightError
from .safetensors_io import ModelFolder


@dataclass
class FusionRule:
    """``target`` is built from ``sources``.

    ``how``: ``"cat0"`` concatenates along dim 0; ``"stack"`` stacks ``[n, ...]``;
    ``"stack_pairs"`` takes sources two by two (gate, up), concatenates each pair along dim 0
    and stacks the results (``[E, 2I, H]`` from ``w1``/``w3`` per expert)."""

    target: str
    sources: List[str]
    how: str
    sizes: Optional[List[int]] = None  # dim-0 sizes of a cat0's parts (equal parts when None)


def _norm_name(name: str, prefixes: Sequence[str]) -> str:
    for p in prefixes:
        if name.startswith(p):
            return name[len(p):]
    return name


def _is_float(dt: torch.dtype) -> bool:
    return dt in (torch.float32, torch.bfloat16, torch.float16, torch.float64)


def target_dtype(ps: ParamSpec, compute: torch.dtype) -> torch.dtype:
    if ps.dtype == "compute":
        return compute
    return {"float32": torch.float32, "int32": torch.int32}[ps.dtype]


def bind_folder(folder: str, expected: Mapping[str, ParamSpec], rules: Sequence[FusionRule],
                compute_dtype: torch.dtype, device: torch.device,
                prefixes: Sequence[str] = (), ignorable: Callable[[str], bool] = lambda n: False,
                optional: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Read every expected tensor from ``folder`` onto ``device``.

    ``optional`` names may be present in the folder without being expected (a tied model's
    stray ``lm_head.weight``)."""
    mf = ModelFolder(folder)
    file_names: Dict[str, str] = {}  # normalised -> name in the file
    for raw in mf.names():
        n = _norm_name(raw, prefixes)
        if ignorable(n) or ignorable(raw):
            continue
        file_names[n] = raw
    rule_of = {r.target: r for r in rules}
    missing: List[str] = []
    wrong: List[str] = []
    used = set()
    plan: List[Tuple[str, ParamSpec, Optional[FusionRule]]] = []

    for name, ps in expected.items():
        if name in file_names:
            shape = mf.shape(file_names[name])
            if tuple(shape) != tuple(ps.shape):
                wrong.append(f"{name}: file has {list(shape)}, model expects {list(ps.shape)}")
            elif _is_float(target_dtype(ps, compute_dtype)) != _is_float(mf.dtype(file_names[name])):
                wrong.append(f"{name}: file dtype {mf.dtype(file_names[name])} cannot become "
                             f"{target_dtype(ps, compute_dtype)}")
            else:
                plan.append((name, ps, None))
            used.add(name)
            continue
        rule = rule_of.get(name)
        if rule is None or not any(s in file_names for s in rule.sources):
            missing.append(name)
            continue
        absent = [s for s in rule.sources if s not in file_names]
        used.update(s for s in rule.sources if s in file_names)
        if absent:
            missing.extend(absent)
            continue
        err = _check_fusion(rule, ps, {s: tuple(mf.shape(file_names[s])) for s in rule.sources})
        if err:
            wrong.extend(err)
            continue
        bad_dtype = [s for s in rule.sources
                     if _is_float(target_dtype(ps, compute_dtype)) != _is_float(mf.dtype(file_names[s]))]
        if bad_dtype:
            wrong.extend(f"{s}: file dtype {mf.dtype(file_names[s])} cannot become "
                         f"{target_dtype(ps, compute_dtype)}" for s in bad_dtype)
            continue
        plan.append((name, ps, rule))

    unexpected = sorted(n for n in file_names if n not in used and n not in optional)
    if missing or unexpected or wrong:
        lines = [f"{folder}: the weight files do not match the model"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(_clip(sorted(missing))))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(_clip(unexpected)))
        if wrong:
            lines.append(f"  wrong shapes or dtypes ({len(wrong)}): " + "; ".join(_clip(wrong)))
        err = WeightError("\n".join(lines))
        err.missing, err.unexpected, err.wrong = sorted(missing), unexpected, wrong
        raise err

    out: Dict[str, torch.Tensor] = {}
    for name, ps, rule in plan:
        dt = target_dtype(ps, compute_dtype)
        if rule is None:
            out[name] = mf.read(file_names[name]).to(device=device, dtype=dt).contiguous()
            continue
        target = torch.empty(ps.shape, dtype=dt, device=device)
        for src, index in _fusion_indices(rule, {s: tuple(mf.shape(file_names[s])) for s in rule.sources}):
            target[index].copy_(mf.read(file_names[src]))
        out[name] = target
    return out


def _clip(items: List[str], limit: int = 40) -> List[str]:
    if len(items) <= limit:
        return items
    return items[:limit] + [f"... and {len(items) - limit} more"]


def _check_fusion(rule: FusionRule, ps: ParamSpec, shapes: Dict[str, Tuple[int, ...]]) -> List[str]:
    want = tuple(ps.shape)
    srcs = rule.sources
    errs: List[str] = []
    if rule.how == "cat0":
        rows = sum(shapes[s][0] if shapes[s] else 0 for s in srcs)
        tails = {shapes[s][1:] for s in srcs}
        if rows != want[0] or tails != {want[1:]}:
            errs.append(f"{rule.target}: parts {[list(shapes[s]) for s in srcs]} do not concatenate "
                        f"to {list(want)}")
    elif rule.how == "stack":
        if len(srcs) != want[0]:
            errs.append(f"{rule.target}: {len(srcs)} parts for a first dim of {want[0]}")
        for s in srcs:
            if shapes[s] != want[1:]:
                errs.append(f"{s}: file has {list(shapes[s])}, model expects {list(want[1:])}")
    elif rule.how == "stack_pairs":
        if len(srcs) != 2 * want[0]:
            errs.append(f"{rule.target}: {len(srcs)} parts for {want[0]} pairs")
        for i in range(0, len(srcs) - 1, 2):
            a, b = shapes[srcs[i]], shapes[srcs[i + 1]]
            if a[1:] != want[2:] or b[1:] != want[2:] or len(a) != len(want) - 1 \
                    or a[0] + b[0] != want[1]:
                errs.append(f"{srcs[i]} / {srcs[i + 1]}: file has {list(a)} and {list(b)}, model "
                            f"expects two parts that concatenate to {list(want[1:])}")
    else:
        errs.append(f"{rule.target}: unknown fusion '{rule.how}'")
    return errs


def _fusion_indices(rule: FusionRule, shapes: Dict[str, Tuple[int, ...]]):
    if rule.how == "cat0":
        r = 0
        for s in rule.sources:
            n = shapes[s][0]
            yield s, (slice(r, r + n),)
            r += n
    elif rule.how == "stack":
        for i, s in enumerate(rule.sources):
            yield s, (i,)
    elif rule.how == "stack_pairs":
        for i in range(0, len(rule.sources), 2):
            a, b = rule.sources[i], rule.sources[i + 1]
            na = shapes[a][0]
            yield a, (i // 2, slice(0, na))
            yield b, (i // 2, slice(na, na + shapes[b][0]))


def unfuse(rule: FusionRule, tensor: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Inverse of a fusion, for writing checkpoints with per-part names."""
    out: Dict[str, torch.Tensor] = {}
    n = len(rule.sources)
    if rule.how == "cat0":
        sizes = list(rule.sizes) if rule.sizes is not None else [tensor.shape[0] // n] * n
        r = 0
        for s, k in zip(rule.sources, sizes):
            out[s] = tensor[r:r + k]
            r += k
    elif rule.how == "stack":
        for i, s in enumerate(rule.sources):
            out[s] = tensor[i]
    elif rule.how == "stack_pairs":
        half = tensor.shape[1] // 2
        for i in range(0, n, 2):
            out[rule.sources[i]] = tensor[i // 2, :half]
            out[rule.sources[i + 1]] = tensor[i // 2, half:]
    return out
