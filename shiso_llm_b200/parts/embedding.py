"""Token embedding and the output head.

Embedding: ``x_t = E[id_t]`` with no scale (crates/shiso-engine/src/layers.rs:1341-1357).
Head: logits for the requested rows only, against the embedding table when tied or a
matrix of its own otherwise (layers.rs:2616-2681).  Logits are float32.
"""

from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import EMBEDDINGS, HEADS, Embedding, Head, project


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.tensor_name = spec.params["tensor"]
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.tensor_name, (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.weight = tensors[self.tensor_name]

    def table(self):
        return self.weight

    def forward(self, step):
        feed = getattr(step, "feed_index", None)
        if feed is None:
            return self.env.ops.embed(step.token_ids, self.weight)
        return self.env.ops.embed(step.token_ids, self.weight, feed, step.fed_tokens)


@HEADS.register("linear_head")
class LinearHead(Head):
    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.vocab = int(p["vocab_size"])
        self.hidden = int(p["hidden_size"])
        self.tied_to = p.get("tied_to")
        self.tensor_name = p.get("tensor")
        if (self.tied_to is None) == (self.tensor_name is None):
            raise ValueError("a head is either tied to a table or has a tensor of its own")
        self.weight = None

    def tensor_specs(self):
        if self.tied_to is not None:
            return []
        return [TensorSpec(self.tensor_name, (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.weight = tensors[self.tied_to if self.tied_to is not None else self.tensor_name]

    def forward(self, x):
        """Float32 logits of the rows ``x``, a tensor or a ``DeferredNorm``."""
        return project(self.env.ops, x, self.weight, torch.float32)
