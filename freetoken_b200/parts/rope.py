"""Position encodings.

``rope_neox``: partial NeoX rotary embedding.  ``inv_freq_i = 1 / theta^(2i / rotary_dim)``,
angle = ``float32(position) * inv_freq_i``, table ``cos || sin`` of shape
``[positions, rotary_dim]`` in float32 (python/freetoken/layers/rotary.py:49-59).  The table is
computed once on the host with the same float32 operations as the reference and uploaded,
so every consumer (and a CPU check) sees identical angles; it covers the engine's longest
sequence rather than the checkpoint's ``max_position_embeddings``.  Mixers rotate inside
their own kernels (``norm_rope_store``); one table serves all layers with equal parameters
(``get_rope`` is cached the same way, rotary.py:211-231).

``none``: no position encoding (a mixer that needs none asks for this kind).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import PartSpec
from ..errors import ConfigError
from .base import POSITIONS, BuildEnv, PositionEncoding


@POSITIONS.register("rope_neox")
class NeoxRope(PositionEncoding):
    """params: ``rotary_dim`` (even, <= head_dim; 0 disables), ``theta``."""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ConfigError(f"rope_neox: rotary_dim={self.rotary_dim} must be even and >= 0")
        self._table: Optional[torch.Tensor] = None

    def table(self) -> Optional[torch.Tensor]:
        """Built at the first call: by then the engine has settled its longest sequence
        (``env.max_seq_len`` may shrink between a part's construction and the first step, once
        the cache has been sized)."""
        if self._table is None and self.rotary_dim:
            rd = self.rotary_dim
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, rd, 2, dtype=torch.float) / rd))
            t = torch.arange(self.env.max_seq_len, dtype=torch.float)
            freqs = torch.einsum("i,j -> ij", t, inv_freq)
            self._table = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(self.env.device)
        return self._table


@POSITIONS.register("none")
class NoPosition(PositionEncoding):
    rotary_dim = 0

    def table(self) -> Optional[torch.Tensor]:
        return None


def shared_position(spec: PartSpec, env: BuildEnv) -> PositionEncoding:
    """One instance per distinct spec for the whole model."""
    key = ("position", spec.key())
    if key not in env.shared:
        env.shared[key] = POSITIONS.build(spec, env)
    return env.shared[key]
