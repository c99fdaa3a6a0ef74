"""LFM2 (``Lfm2ForCausalLM``): typed configuration and model plan.

A decoder that interleaves gated short-convolution layers with GQA attention
layers (per-head RMS QK-norm, half-split RoPE), each followed by a SwiGLU
feed-forward, pre-RMSNorm everywhere, a final norm named after the embedding and
a tied or untied output head.

The reference reads this family's geometry from GGUF metadata and uses
``config.json`` only to recognise ``model_type`` and cross-check five widths
plus ``layer_types`` (crates/shiso-models/src/lfm2/config.rs:34,63-73,131-220,
223-274).  Here config.json is the single source, read by its own keys; the
checks kept from the reference are: ``len(layer_types) == num_hidden_layers``
and only ``conv`` / ``full_attention`` values (config.rs:252-271), ``hidden``
divisible by the head count (config.rs:142-147), query heads divisible by KV
heads (crates/shiso-engine/src/dense/mod.rs:101-110), at least two conv taps
(crates/shiso-engine/src/short_conv.rs:58), and a refusal of rope scaling
(crates/shiso-models/src/llama/config.rs:254-259).
"""

from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Mapping, Optional

from ..parts.plan import LayerSpec, ModelPlan, PartSpec, sequential_order
from .errors import ConfigMissing, InvalidValue
from .registry import register_architecture

ARCHITECTURE = "Lfm2ForCausalLM"
MODEL_TYPES = ("lfm2",)
CONV = "conv"
FULL_ATTENTION = "full_attention"


def _need(document: Mapping[str, Any], key: str):
    if key not in document or document[key] is None:
        raise ConfigMissing(key)
    return document[key]


def _positive_int(document, key) -> int:
    value = _need(document, key)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise InvalidValue(key, value, "expected a positive integer")
    return value


def _number(document, key, default=None) -> float:
    value = document.get(key, default)
    if value is None:
        raise ConfigMissing(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise InvalidValue(key, value, "expected a number")
    return float(value)


def _boolean(document, key, default=None) -> bool:
    value = document.get(key, default)
    if value is None:
        raise ConfigMissing(key)
    if not isinstance(value, bool):
        raise InvalidValue(key, value, "expected true or false")
    return value


def feed_forward_width(block_ff_dim: int, auto_adjust: bool, multiplier: float, multiple_of: int) -> int:
    """The SwiGLU intermediate width the configuration describes.

    With auto-adjust on the stated width is scaled by 2/3 (the usual SwiGLU
    parameter-parity rule), by ``multiplier``, and rounded up to ``multiple_of``:
    8192 -> 5632 and 10752 -> 7168 at 256; 384 -> 256 at 64.  With it off the
    stated width is used as is.  The reference reads the final width from GGUF
    (crates/shiso-models/src/lfm2/config.rs:177), so this rule has no twin there.
    """
    if not auto_adjust:
        return block_ff_dim
    width = int(2 * block_ff_dim / 3)
    width = int(multiplier * width)
    return multiple_of * ((width + multiple_of - 1) // multiple_of)


@dataclass(frozen=True)
class Lfm2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    layer_types: tuple[str, ...]
    conv_L_cache: int
    conv_bias: bool
    block_ff_dim: int
    block_auto_adjust_ff_dim: bool
    block_multiple_of: int
    block_ffn_dim_multiplier: float
    norm_eps: float
    rope_theta: float
    tie_embedding: bool
    max_position_embeddings: Optional[int] = None
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    @property
    def head_dim(self) -> int:
        # Derived, never stored (crates/shiso-models/src/lfm2/config.rs:148-150).
        return self.hidden_size // self.num_attention_heads

    @property
    def intermediate_size(self) -> int:
        return feed_forward_width(
            self.block_ff_dim,
            self.block_auto_adjust_ff_dim,
            self.block_ffn_dim_multiplier,
            self.block_multiple_of,
        )

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "Lfm2Config":
        names = document.get("architectures")
        model_type = document.get("model_type")
        if names is not None and (not isinstance(names, list) or not names or names[0] != ARCHITECTURE):
            raise InvalidValue("architectures", names, f"expected [{ARCHITECTURE!r}]")
        if names is None and model_type not in MODEL_TYPES:
            raise InvalidValue("model_type", model_type, f"expected one of {MODEL_TYPES}")

        hidden = _positive_int(document, "hidden_size")
        layers = _positive_int(document, "num_hidden_layers")
        heads = _positive_int(document, "num_attention_heads")
        kv_heads = _positive_int(document, "num_key_value_heads")
        vocab = _positive_int(document, "vocab_size")

        kinds = _need(document, "layer_types")
        if not isinstance(kinds, list) or not all(isinstance(k, str) for k in kinds):
            raise InvalidValue("layer_types", kinds, "expected a list of layer kind names")
        if len(kinds) != layers:
            raise InvalidValue(
                "layer_types", kinds, f"{len(kinds)} entries for num_hidden_layers = {layers}"
            )
        for i, kind in enumerate(kinds):
            if kind not in (CONV, FULL_ATTENTION):
                raise InvalidValue(
                    f"layer_types[{i}]", kind, f"expected {CONV!r} or {FULL_ATTENTION!r}"
                )

        if hidden % heads != 0:
            raise InvalidValue(
                "num_attention_heads", heads, f"does not divide hidden_size = {hidden}"
            )
        if heads % kv_heads != 0:
            raise InvalidValue(
                "num_key_value_heads", kv_heads, f"does not divide num_attention_heads = {heads}"
            )
        if (hidden // heads) % 2 != 0:
            raise InvalidValue(
                "hidden_size", hidden, "the head size hidden_size / num_attention_heads must be even for RoPE"
            )

        taps = _positive_int(document, "conv_L_cache")
        if taps < 2:
            raise InvalidValue("conv_L_cache", taps, "a short convolution needs at least 2 taps")

        ff_dim = _positive_int(document, "block_ff_dim")
        auto_adjust = _boolean(document, "block_auto_adjust_ff_dim")
        multiplier = _number(document, "block_ffn_dim_multiplier", 1.0)
        if multiplier <= 0:
            raise InvalidValue("block_ffn_dim_multiplier", multiplier, "expected a positive number")
        if auto_adjust:
            multiple_of = _positive_int(document, "block_multiple_of")
        else:
            multiple_of = document.get("block_multiple_of", 1)
            if isinstance(multiple_of, bool) or not isinstance(multiple_of, int) or multiple_of <= 0:
                raise InvalidValue("block_multiple_of", multiple_of, "expected a positive integer")

        eps = _number(document, "norm_eps")
        if not 0.0 < eps < 1.0:
            raise InvalidValue("norm_eps", eps, "expected a small positive number")
        theta = _number(document, "rope_theta")
        if theta <= 1.0:
            raise InvalidValue("rope_theta", theta, "expected a base above 1")
        if document.get("rope_scaling") is not None:
            raise InvalidValue("rope_scaling", document["rope_scaling"], "rope scaling is not part of this architecture")

        tie_keys = [k for k in ("tie_embedding", "tie_word_embeddings") if k in document]
        if len(tie_keys) == 2 and document[tie_keys[0]] != document[tie_keys[1]]:
            raise InvalidValue("tie_word_embeddings", document["tie_word_embeddings"], "disagrees with tie_embedding")
        tie = _boolean(document, tie_keys[0], True) if tie_keys else True

        def optional_int(key):
            value = document.get(key)
            if value is None:
                return None
            if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                raise InvalidValue(key, value, "expected a non-negative integer")
            return value

        eos = optional_int("eos_token_id")
        if eos is not None and eos >= vocab:
            raise InvalidValue("eos_token_id", eos, f"outside the vocabulary of {vocab}")

        return cls(
            vocab_size=vocab,
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            layer_types=tuple(kinds),
            conv_L_cache=taps,
            conv_bias=_boolean(document, "conv_bias", False),
            block_ff_dim=ff_dim,
            block_auto_adjust_ff_dim=auto_adjust,
            block_multiple_of=multiple_of,
            block_ffn_dim_multiplier=multiplier,
            norm_eps=eps,
            rope_theta=theta,
            tie_embedding=tie,
            max_position_embeddings=optional_int("max_position_embeddings"),
            eos_token_id=eos,
            bos_token_id=optional_int("bos_token_id"),
            pad_token_id=optional_int("pad_token_id"),
        )

    def to_dict(self) -> dict:
        document = {"architectures": [ARCHITECTURE], "model_type": MODEL_TYPES[0]}
        for key, value in asdict(self).items():
            if value is None:
                continue
            document[key] = list(value) if isinstance(value, tuple) else value
        return document


def build_plan(config: Lfm2Config) -> ModelPlan:
    """LFM2 as a list of parts.

    Layer order and wiring follow the reference's layer loop
    (crates/shiso-engine/src/layers.rs:1952-2301): pre-norm, mixer, residual,
    feed-forward norm, SwiGLU, residual; the final norm is the tensor named
    after the embedding (crates/shiso-models/src/lfm2/model.rs:9-14).
    """
    hidden = config.hidden_size

    def norm(name: str, size: int = hidden) -> PartSpec:
        return PartSpec("rmsnorm", {"tensor": name, "size": size, "eps": config.norm_eps})

    layers = []
    for i, kind in enumerate(config.layer_types):
        prefix = f"model.layers.{i}"
        if kind == CONV:
            mixer = PartSpec(
                "short_conv",
                {
                    "hidden_size": hidden,
                    "taps": config.conv_L_cache,
                    "bias": config.conv_bias,
                    "in_proj": f"{prefix}.conv.in_proj.weight",
                    "conv": f"{prefix}.conv.conv.weight",
                    "conv_bias": f"{prefix}.conv.conv.bias",
                    "out_proj": f"{prefix}.conv.out_proj.weight",
                },
            )
        else:
            head_dim = config.head_dim
            mixer = PartSpec(
                "gqa_attention",
                {
                    "hidden_size": hidden,
                    "num_heads": config.num_attention_heads,
                    "num_kv_heads": config.num_key_value_heads,
                    "head_dim": head_dim,
                    "scale": None,
                    "window": None,
                    "q_proj": f"{prefix}.self_attn.q_proj.weight",
                    "k_proj": f"{prefix}.self_attn.k_proj.weight",
                    "v_proj": f"{prefix}.self_attn.v_proj.weight",
                    "out_proj": f"{prefix}.self_attn.out_proj.weight",
                    "q_norm": norm(f"{prefix}.self_attn.q_layernorm.weight", head_dim),
                    "k_norm": norm(f"{prefix}.self_attn.k_layernorm.weight", head_dim),
                    "position": PartSpec(
                        "rope_half_split", {"theta": config.rope_theta, "rotary_dim": head_dim}
                    ),
                },
            )
        layers.append(
            LayerSpec(
                name=prefix,
                block=PartSpec("pre_norm"),
                mixer=mixer,
                mixer_norm=norm(f"{prefix}.operator_norm.weight"),
                feed_forward=PartSpec(
                    "swiglu",
                    {
                        "hidden_size": hidden,
                        "intermediate_size": config.intermediate_size,
                        "gate": f"{prefix}.feed_forward.w1.weight",
                        "up": f"{prefix}.feed_forward.w3.weight",
                        "down": f"{prefix}.feed_forward.w2.weight",
                    },
                ),
                feed_forward_norm=norm(f"{prefix}.ffn_norm.weight"),
            )
        )

    return ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=hidden,
        vocab_size=config.vocab_size,
        embedding=PartSpec(
            "token_embedding",
            {"tensor": "model.embed_tokens.weight", "vocab_size": config.vocab_size, "hidden_size": hidden},
        ),
        layers=tuple(layers),
        order=sequential_order(len(layers)),
        final_norm=norm("model.embedding_norm.weight"),
        head=PartSpec(
            "linear_head",
            {
                "vocab_size": config.vocab_size,
                "hidden_size": hidden,
                "tied_to": "model.embed_tokens.weight" if config.tie_embedding else None,
                "tensor": None if config.tie_embedding else "lm_head.weight",
            },
        ),
        eos_token_ids=(config.eos_token_id,) if config.eos_token_id is not None else (),
        max_position=config.max_position_embeddings,
    )


register_architecture(ARCHITECTURE, Lfm2Config, build_plan, MODEL_TYPES)
