"""From a model folder (or a config dict) to a bound :class:`Model`.

Mirrors the reference's engine start-up (python/freetoken/engine/engine.py:321-323,452-467):
resolve the architecture from ``architectures[0]``, build the model, then fill it either from
the folder's safetensors files or with seeded random tensors made on the device.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from ..config.spec import ModelSpec, ParamSpec
from ..models.model import Model
from ..parts import BuildEnv, Workspace
from ..registry import Architecture, architecture_of
from ..weights.binder import bind_folder
from ..weights.random_init import random_tensors_on_device


def describe_model(raw_config: Mapping[str, Any], num_layers: Optional[int] = None
                   ) -> Tuple[Architecture, Any, ModelSpec, Dict[str, ParamSpec]]:
    """Architecture, typed config, model description and expected tensors of a config.json,
    without touching a GPU."""
    arch = architecture_of(raw_config)
    typed = arch.parse_config(raw_config, num_layers=num_layers)
    spec = arch.build_spec(typed)
    cpu = torch.device("cpu")
    env = BuildEnv(dtype=torch.bfloat16, device=cpu, max_seq_len=1, max_step_tokens=1,
                   workspace=Workspace(cpu))
    return arch, typed, spec, Model(spec, env).param_specs()


def build_model(spec: ModelSpec, env: BuildEnv) -> Model:
    return Model(spec, env)


def load_weights(model: Model, arch: Architecture, typed: Any, folder: str) -> None:
    expected = model.param_specs()
    optional = (f"{model.spec.head_name}.weight",) if model.tied else ()
    tensors = bind_folder(folder, expected, arch.fusion_rules(typed), model.env.dtype,
                          model.env.device, prefixes=arch.name_prefixes,
                          ignorable=arch.ignorable, optional=optional)
    model.bind(tensors)


def random_weights(model: Model, seed: int) -> None:
    tensors = random_tensors_on_device(model.param_specs(), seed, model.env.dtype, model.env.device)
    model.bind(tensors)
