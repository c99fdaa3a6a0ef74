"""Gated short convolution: ``out = W_out (c * conv(b * x))``.

``p = W_in n`` is split ``[b | c | x]``; the gate is applied BEFORE the
convolution and the request's state keeps the last ``taps - 1`` gated inputs
``u = b * x``, oldest first, in float32 - never ``x`` alone
(kernels/metal/dense/dense_short_conv.metal:5-15,45-67).  ``y_t = c_t * (sum_j
w[:, j] * u_{t-(taps-1)+j} + bias)`` with ``w[:, taps-1]`` on the current token
(crates/shiso-models/src/lfm2/model.rs:227-232); ``u`` before the request's first
token is zero.  The reference walks a portion's tokens serially, one thread a
channel, and launches once per row for a decode batch
(crates/shiso-engine/src/short_conv.rs:171-182); here one launch covers every
sequence of the step, parallel over tokens, each sequence with its own state slot.
"""

from __future__ import annotations

from ..config.errors import UnsupportedShape
from ..weights.spec import VECTOR, ZEROS, TensorSpec
from .base import MIXERS, DeferredLinear, DeferredNorm, FixedState, Mixer

MAX_TAPS = 8


@MIXERS.register("short_conv")
class ShortConv(Mixer):
    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.taps = int(p["taps"])
        if not 2 <= self.taps <= MAX_TAPS:
            raise UnsupportedShape("conv taps", self.taps, f"the short-conv kernels take 2 to {MAX_TAPS} taps")
        self.has_bias = bool(p.get("bias", False))
        self.names = {k: p[k] for k in ("in_proj", "conv", "out_proj")}
        self.bias_name = p.get("conv_bias")
        self.in_proj = self.conv = self.out_proj = self.bias = None

    def tensor_specs(self):
        h, l = self.hidden, self.taps
        specs = [
            TensorSpec(self.names["in_proj"], (3 * h, h)),
            TensorSpec(self.names["conv"], (h, l), VECTOR, alt_shapes=((h, 1, l),)),
            TensorSpec(self.names["out_proj"], (h, h)),
        ]
        if self.has_bias:
            specs.append(TensorSpec(self.bias_name, (h,), VECTOR))
        return specs

    def bind(self, tensors):
        self.in_proj = tensors[self.names["in_proj"]]
        self.conv = tensors[self.names["conv"]]
        self.out_proj = tensors[self.names["out_proj"]]
        self.bias = tensors[self.bias_name] if self.has_bias else None

    def cache_spec(self):
        return FixedState((self.taps - 1, self.hidden))

    def forward(self, x, step, cache):
        ops = self.env.ops
        if isinstance(x, DeferredNorm):
            y = x.linear_short_conv(self.in_proj, self.conv, self.bias, cache.state, step)
        else:
            y = ops.linear_short_conv(x, self.in_proj, self.conv, self.bias, cache.state, step)
        return DeferredLinear(ops, y, self.out_proj, self.env.dtype)
