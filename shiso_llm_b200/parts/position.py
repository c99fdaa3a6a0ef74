"""Position encodings.

``rope_half_split`` rotates pairs ``(i, i + rotary_dim/2)`` of a head by the angle
``pos * theta^(-2i / rotary_dim)`` (kernels/cuda/dense/dense_common.cuh:166-180).
The inverse frequencies are computed once in float64 and rounded to float32; the
angle ``pos * inv_freq`` and its sine and cosine are evaluated in float32 inside
the fused norm + rotate + store kernel (the reference calls ``powf`` per element
on the device; the ladder is the same).
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from .base import POSITION_ENCODINGS, PositionEncoding


@POSITION_ENCODINGS.register("rope_half_split")
class RopeHalfSplit(PositionEncoding):
    def __init__(self, spec, env, head_dim: int):
        super().__init__(spec, env)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params.get("rotary_dim") or head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise UnsupportedShape("rotary_dim", self.rotary_dim, f"must be even and at most the head size {head_dim}")
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-2.0 * i / self.rotary_dim)).to(torch.float32).to(env.device)

    def rotary(self):
        return self.inv_freq, self.rotary_dim


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries and keys as they are."""

    def __init__(self, spec, env, head_dim: int):
        super().__init__(spec, env)

    def rotary(self):
        return None, 0
