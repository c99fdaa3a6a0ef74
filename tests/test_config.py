"""Configuration: keys read, derived sizes, every refusal, the registry."""

import copy
import json

import pytest

import helpers
from shiso_llm_b200.config import (
    ConfigMissing, InvalidValue, Lfm2Config, UnknownArchitecture, architecture_of, feed_forward_width,
    load_config, plan_from_document, register_architecture, registered_architectures, unregister_architecture,
)
from shiso_llm_b200.parts import ModelPlan


def test_reads_every_key_of_both_tiny_configurations():
    a = Lfm2Config.from_dict(helpers.TINY_A)
    b = Lfm2Config.from_dict(helpers.TINY_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 3, 1, 32)
    assert a.intermediate_size == 192 and b.intermediate_size == 256
    assert a.tie_embedding and not b.tie_embedding
    assert (a.conv_L_cache, b.conv_L_cache) == (3, 4) and (a.conv_bias, b.conv_bias) == (False, True)
    assert (a.norm_eps, b.norm_eps) == (1e-5, 1e-6) and (a.rope_theta, b.rope_theta) == (1e4, 1e6)
    assert Lfm2Config.from_dict(a.to_dict()) == a and Lfm2Config.from_dict(b.to_dict()) == b


@pytest.mark.parametrize("ff,mult,want", [(8192, 256, 5632), (6656, 256, 4608), (10752, 256, 7168), (384, 64, 256)])
def test_feed_forward_width_rule(ff, mult, want):
    assert feed_forward_width(ff, True, 1.0, mult) == want
    assert feed_forward_width(ff, False, 1.0, mult) == ff


def test_presets_match_the_published_shapes():
    from shiso_llm_b200.cli import preset_path

    for name, inter, attn in (("lfm2-1.2b", 5632, [2, 5, 8, 10, 12, 14]), ("lfm2-350m", 4608, [2, 5, 8, 10, 12, 14]),
                              ("lfm2-2.6b", 7168, [2, 6, 10, 14, 18, 22, 25, 28])):
        cfg = Lfm2Config.from_dict(json.load(open(preset_path(name))))
        assert cfg.intermediate_size == inter
        assert [i for i, k in enumerate(cfg.layer_types) if k == "full_attention"] == attn


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                                 "vocab_size", "layer_types", "conv_L_cache", "block_ff_dim",
                                 "block_auto_adjust_ff_dim", "norm_eps", "rope_theta"])
def test_missing_key_is_named(key):
    doc = copy.deepcopy(helpers.TINY_B)
    del doc[key]
    with pytest.raises(ConfigMissing) as e:
        Lfm2Config.from_dict(doc)
    assert e.value.key == key


@pytest.mark.parametrize("key,value", [
    ("layer_types", ["conv"] * 5), ("layer_types", ["conv", "conv", "sliding", "conv", "conv", "conv"]),
    ("num_attention_heads", 5), ("num_key_value_heads", 2), ("conv_L_cache", 1), ("norm_eps", 0.0),
    ("rope_theta", 1.0), ("rope_scaling", {"type": "linear", "factor": 2.0}), ("hidden_size", -4),
    ("vocab_size", True), ("conv_bias", "yes"), ("block_ffn_dim_multiplier", 0),
])
def test_invalid_value_is_refused(key, value):
    doc = copy.deepcopy(helpers.TINY_B)
    doc[key] = value
    with pytest.raises(InvalidValue):
        Lfm2Config.from_dict(doc)


def test_tie_alias_and_conflict():
    doc = copy.deepcopy(helpers.TINY_A)
    del doc["tie_embedding"]
    doc["tie_word_embeddings"] = False
    assert Lfm2Config.from_dict(doc).tie_embedding is False
    doc["tie_embedding"] = True
    with pytest.raises(InvalidValue):
        Lfm2Config.from_dict(doc)


def test_registry_picks_by_name_and_refuses_unknown():
    assert "Lfm2ForCausalLM" in registered_architectures()
    assert architecture_of(helpers.TINY_A).name == "Lfm2ForCausalLM"
    assert architecture_of({"model_type": "lfm2"}).name == "Lfm2ForCausalLM"
    with pytest.raises(UnknownArchitecture):
        architecture_of({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigMissing):
        architecture_of({})


def test_plan_lists_parts_layer_by_layer():
    _, config, plan = plan_from_document(helpers.TINY_B)
    assert isinstance(plan, ModelPlan)
    kinds = [layer.mixer.kind for layer in plan.layers]
    assert kinds == ["short_conv", "short_conv", "gqa_attention", "short_conv", "gqa_attention", "gqa_attention"]
    assert [e.layer for e in plan.order] == list(range(6)) and all(e.cache_of is None for e in plan.order)
    assert plan.head.params["tensor"] == "lm_head.weight" and plan.head.params["tied_to"] is None
    assert plan.layers[2].mixer.params["position"].params["theta"] == 1e6
    assert plan.layers[0].feed_forward.params["intermediate_size"] == 256


def test_another_architecture_can_be_registered(tmp_path):
    class ToyConfig:
        @classmethod
        def from_dict(cls, d):
            return cls()

    register_architecture("ToyForCausalLM", ToyConfig, lambda c: "plan")
    try:
        (tmp_path / "config.json").write_text(json.dumps({"architectures": ["ToyForCausalLM"]}))
        arch, cfg = load_config(str(tmp_path))
        assert arch.name == "ToyForCausalLM" and isinstance(cfg, ToyConfig) and arch.build_plan(cfg) == "plan"
    finally:
        unregister_architecture("ToyForCausalLM")
