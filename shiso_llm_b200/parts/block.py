"""Arrangements of norm, mixer, feed-forward and the residual stream in one layer.

``pre_norm``: ``h = x + mixer(norm(x))``, ``x' = h + ff(norm(h))`` with no
post-norms (crates/shiso-models/src/lfm2/config.rs:184; the layer loop at
crates/shiso-engine/src/layers.rs:2003-2294).  A block only marks its outputs as
pending on the stream; the next norm adds them while it normalises.
"""

from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec, env, layer):
        super().__init__(spec, env)
        self.name = layer.name
        self.mixer_norm = NORMS.build(layer.mixer_norm, env)
        self.mixer = MIXERS.build(layer.mixer, env)
        self.feed_forward = None
        self.ff_norm = None
        if layer.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, env)
            self.ff_norm = NORMS.build(layer.feed_forward_norm, env)

    def sub_parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        specs = []
        for part in self.sub_parts():
            specs += part.tensor_specs()
        return specs

    def bind(self, tensors):
        for part in self.sub_parts():
            part.bind(tensors)

    def mixer_part(self):
        return self.mixer

    def forward(self, stream, step, cache):
        x = stream.normed(self.mixer_norm, getattr(self.mixer, "takes_deferred_norm", False))
        stream.add(self.mixer.forward(x, step, cache))
        if self.feed_forward is not None:
            x = stream.normed(self.ff_norm, getattr(self.feed_forward, "takes_deferred_norm", False))
            stream.add(self.feed_forward.forward(x, step))
