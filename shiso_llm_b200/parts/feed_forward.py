"""SwiGLU feed-forward: ``W_down (silu(W_gate x) * (W_up x))``.

The gate and up matrices are stored apart in the checkpoint and run as one paired
projection (crates/shiso-engine/src/ffn.rs:234-239); here they are joined into one
``[2I, H]`` matrix when bound, so one product yields ``[gate | up]`` rows; the activation
(kernels/cuda/generic/glu.cuh:35-57: alpha 1, no clamp) is applied in the product's epilogue
for decode-sized batches and by a kernel of its own otherwise.
"""

from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import FEED_FORWARDS, DeferredLinear, FeedForward, project


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.names = (p["gate"], p["up"], p["down"])
        self.gate_up = None
        self.down = None

    def tensor_specs(self):
        gate, up, down = self.names
        return [
            TensorSpec(gate, (self.inter, self.hidden)),
            TensorSpec(up, (self.inter, self.hidden)),
            TensorSpec(down, (self.hidden, self.inter)),
        ]

    def bind(self, tensors):
        gate, up, down = self.names
        g, u = tensors[gate], tensors[up]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.gate_up = torch.cat([g, u], dim=0).contiguous()
        self.down = tensors[down]

    def forward(self, x, step):
        ops = self.env.ops
        mid = project(ops, x, self.gate_up, self.env.dtype, glu=True)
        return DeferredLinear(ops, mid, self.down, self.env.dtype)
