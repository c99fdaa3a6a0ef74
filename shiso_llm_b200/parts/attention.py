"""Grouped-query attention over a paged cache.

Order of operations, as the reference launches them
(crates/shiso-engine/src/dense/attn.rs:497-546): q/k/v projections without bias;
per-head RMS norm of q and k with a ``[head_dim]`` weight, before the rotation
(kernels/cuda/dense/dense_norm_rope.cuh:42-53,96-106); position encoding; the
normalised, rotated key and the raw value are stored in the cache at the row the
block table names - before any score is taken, so a portion's tokens see their own
keys (dense/attn.rs:28-33); scores ``(q . k) * scale`` over positions
``max(0, pos + 1 - window) .. pos`` with the KV head of query head ``h`` being
``h // (heads / kv_heads)`` (kernels/cuda/dense/dense_attn.cuh:32-34,60,87-88,110);
softmax in float32; output projection.

q, k and v are stored apart in the checkpoint and joined into one ``[(heads +
2 kv_heads) * head_dim, hidden]`` matrix when bound, so one product feeds the fused
norm + rotate + store kernel.  A run entry that borrows another entry's cache
projects queries only and stores nothing.
"""

from __future__ import annotations

import math

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import TensorSpec
from .base import MIXERS, NORMS, POSITION_ENCODINGS, DeferredLinear, Mixer, PagedKV, project

MAX_HEAD_DIM = 256  # what the general attention kernel keeps of a head in a warp's registers


@MIXERS.register("gqa_attention")
class GqaAttention(Mixer):
    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        if self.heads % self.kv_heads:
            raise UnsupportedShape("num_kv_heads", self.kv_heads, f"does not divide {self.heads} query heads")
        # Any head size up to 256 runs: the tensor-core kernels take sizes in steps of 16 (the
        # kernel table sends other sizes, in either compute type, to the general kernel).
        if not 0 < self.head_dim <= MAX_HEAD_DIM:
            raise UnsupportedShape("head_dim", self.head_dim, f"the attention kernels take head sizes up to {MAX_HEAD_DIM}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = int(p["window"]) if p.get("window") else None
        self.borrows_cache = bool(p.get("borrows_cache", False))
        self.names = {k: p[k] for k in ("q_proj", "k_proj", "v_proj", "out_proj")}
        self.q_norm = NORMS.build(p["q_norm"], env) if p.get("q_norm") is not None else None
        self.k_norm = NORMS.build(p["k_norm"], env) if p.get("k_norm") is not None else None
        for norm in (self.q_norm, self.k_norm):
            if norm is not None and norm.size != self.head_dim:
                raise UnsupportedShape("qk norm size", norm.size, f"must equal the head size {self.head_dim}")
        if self.q_norm is not None and self.k_norm is not None and self.q_norm.eps != self.k_norm.eps:
            raise UnsupportedShape("qk norm eps", (self.q_norm.eps, self.k_norm.eps), "q and k norms share one kernel and one eps")
        self.position = POSITION_ENCODINGS.build(p["position"], env, self.head_dim)
        self.qkv = None
        self.out = None

    def sub_parts(self):
        return [x for x in (self.q_norm, self.k_norm, self.position) if x is not None]

    def tensor_specs(self):
        q_rows = self.heads * self.head_dim
        kv_rows = self.kv_heads * self.head_dim
        specs = [TensorSpec(self.names["q_proj"], (q_rows, self.hidden))]
        if not self.borrows_cache:
            specs += [
                TensorSpec(self.names["k_proj"], (kv_rows, self.hidden)),
                TensorSpec(self.names["v_proj"], (kv_rows, self.hidden)),
            ]
        specs.append(TensorSpec(self.names["out_proj"], (self.hidden, q_rows)))
        for part in self.sub_parts():
            specs += part.tensor_specs()
        return specs

    def bind(self, tensors):
        mats = [tensors[self.names["q_proj"]]]
        if not self.borrows_cache:
            mats += [tensors[self.names["k_proj"]], tensors[self.names["v_proj"]]]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.qkv = torch.cat(mats, dim=0).contiguous()
        self.out = tensors[self.names["out_proj"]]
        for part in self.sub_parts():
            part.bind(tensors)

    def cache_spec(self):
        if self.borrows_cache:
            return None
        return PagedKV(self.kv_heads, self.head_dim, self.window)  # values as wide as keys, in the compute type

    def forward(self, x, step, cache):
        ops = self.env.ops
        store = cache.owner and not self.borrows_cache
        qkv = project(ops, x, self.qkv, self.env.dtype)
        inv_freq, rotary_dim = self.position.rotary()
        interleaved = bool(getattr(self.position, "interleaved", False))
        pairing = {"interleaved": True} if interleaved else {}  # handed on only when it is not the usual one
        from_qkv = getattr(ops, "decode_attention_from_qkv", None)
        if from_qkv is not None and not interleaved and not self.borrows_cache and self.q_norm is not None and self.k_norm is not None:
            # steps of single tokens: norm, rotation, cache store and attention in one launch
            attn = from_qkv(
                qkv, self.heads, self.kv_heads, self.head_dim, self.q_norm.weight, self.k_norm.weight, self.q_norm.eps,
                inv_freq, rotary_dim, step, cache.k, cache.v, step.block_tables[cache.group], cache.page_size, store,
                self.scale, self.window or 0,
            )
            if attn is not None:
                return DeferredLinear(ops, attn, self.out, self.env.dtype)
        q = ops.qk_norm_rope_store(
            qkv,
            self.heads,
            0 if self.borrows_cache else self.kv_heads,
            self.head_dim,
            self.q_norm.weight if self.q_norm is not None else None,
            self.k_norm.weight if self.k_norm is not None else None,
            self.q_norm.eps if self.q_norm is not None else (self.k_norm.eps if self.k_norm is not None else 0.0),
            inv_freq,
            rotary_dim,
            step,
            cache.k,
            cache.v,
            step.block_tables[cache.group],
            cache.page_size,
            store,
            **pairing,
        )
        attn = ops.paged_attention(
            q,
            self.heads,
            cache.kv_heads,
            self.head_dim,
            cache.k,
            cache.v,
            step.block_tables[cache.group],
            cache.page_size,
            self.scale,
            self.window or 0,
            step,
        )
        return DeferredLinear(ops, attn, self.out, self.env.dtype)
