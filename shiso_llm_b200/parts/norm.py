"""RMS normalisation: ``y = x * rsqrt(mean(x^2) + eps) * w`` with the statistics in float32.

The weight multiplies directly, not as ``1 + w`` (kernels/cuda/generic/norm.cuh:86-93).
``add_apply`` is the fused residual-add + norm that closes every block
(norm.cuh:105-165; crates/shiso-engine/src/layers.rs:2476-2498): the stored sum is
what is normalised.
"""

from __future__ import annotations

from ..weights.spec import ONES, VECTOR, TensorSpec
from .base import NORMS, Norm


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.tensor_name = spec.params["tensor"]
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.tensor_name, (self.size,), VECTOR, ONES)]

    def bind(self, tensors):
        self.weight = tensors[self.tensor_name]

    def rms_params(self):
        """``(weight, eps)``: what a kernel that normalises inside a product needs."""
        return self.weight, self.eps

    def apply(self, x):
        return self.env.ops.rmsnorm(x, self.weight, self.eps, self.env.dtype)

    def add_apply(self, residual, delta, rows=None):
        return self.env.ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.env.dtype, rows)

    def add_apply_linear(self, residual, deferred):
        """``residual += deferred.x @ deferred.w^T`` and the norm of the sum, fused where the
        kernel table can (decode-sized bfloat16 steps)."""
        return self.env.ops.linear_add_rmsnorm(deferred.x, deferred.w, residual, self.weight, self.eps, self.env.dtype)
