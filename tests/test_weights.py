"""Weights: the safetensors container, loading by name with one clear error, random folders."""

import json
import os

import pytest
import torch

import helpers
from shiso_llm_b200.weights import (
    SafetensorsError, SafetensorsFile, WeightError, load_weights, random_tensors, write_model_folder, write_safetensors,
)


def test_container_round_trip(tmp_path):
    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
        "d": torch.randn(2, 1, 4).to(torch.float16),
    }
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, {"k": "v"})
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(tensors) and f.metadata == {"k": "v"}
    for name, t in tensors.items():
        assert f.tensor(name).dtype == t.dtype and torch.equal(f.tensor(name), t)
    raw = open(path, "rb").read()
    header_len = int.from_bytes(raw[:8], "little")
    assert header_len % 8 == 0 and json.loads(raw[8 : 8 + header_len])["a"]["dtype"] == "F32"


def test_container_refuses_bad_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes((10**9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    header = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))


def test_random_folder_is_deterministic_and_loads_by_name(tmp_path):
    a = helpers.make_folder(tmp_path / "a", helpers.TINY_B, 1)
    b = helpers.make_tensors(helpers.TINY_B, 1)
    c = helpers.make_tensors(helpers.TINY_B, 2)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert os.path.isfile(tmp_path / "a" / "config.json") and os.path.isfile(tmp_path / "a" / "model.safetensors")
    specs = helpers.tensor_specs_of(helpers.TINY_B)
    assert {s.name for s in specs} == set(a)
    assert "lm_head.weight" in a and "model.layers.0.conv.conv.bias" in a
    assert "lm_head.weight" not in helpers.make_tensors(helpers.TINY_A, 0)
    bf = load_weights(str(tmp_path / "a"), specs, torch.bfloat16, "cpu")
    fp = load_weights(str(tmp_path / "a"), specs, torch.float32, "cpu")
    assert bf["model.layers.0.conv.in_proj.weight"].dtype == torch.bfloat16
    assert bf["model.layers.0.operator_norm.weight"].dtype == torch.float32  # vectors are read in 32-bit
    assert bf["model.layers.0.conv.conv.weight"].shape == (96, 4)
    assert all(t.dtype == torch.float32 for t in fp.values())
    assert torch.equal(fp["lm_head.weight"], bf["lm_head.weight"].float())


def test_a_matrix_stored_in_32_bit_stays_so(tmp_path):
    tensors = {k: v.clone() for k, v in helpers.make_tensors(helpers.TINY_A, 0).items()}
    name = "model.layers.1.self_attn.q_proj.weight"
    tensors[name] = tensors[name].float() + 1e-4  # not representable in bfloat16
    write_model_folder(str(tmp_path), helpers.TINY_A, tensors)
    got = load_weights(str(tmp_path), helpers.tensor_specs_of(helpers.TINY_A), torch.bfloat16, "cpu")
    assert got[name].dtype == torch.float32 and torch.equal(got[name], tensors[name])


def test_one_error_lists_everything_wrong(tmp_path):
    tensors = dict(helpers.make_tensors(helpers.TINY_B, 1))
    del tensors["model.layers.2.self_attn.k_layernorm.weight"]
    del tensors["model.embedding_norm.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(2)
    tensors["model.layers.0.feed_forward.w1.weight"] = torch.zeros(255, 96, dtype=torch.bfloat16)
    tensors["model.layers.1.ffn_norm.weight"] = torch.zeros(96, dtype=torch.int32)
    write_model_folder(str(tmp_path), helpers.TINY_B, tensors)
    with pytest.raises(WeightError) as e:
        load_weights(str(tmp_path), helpers.tensor_specs_of(helpers.TINY_B), torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["model.embedding_norm.weight", "model.layers.2.self_attn.k_layernorm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.feed_forward.w1.weight", (256, 96), (255, 96))]
    assert err.wrong_dtype[0][0] == "model.layers.1.ffn_norm.weight"
    text = str(err)
    for piece in ("missing (2)", "unexpected (1)", "expected [256, 96], file has [255, 96]", "model.layers.9.extra.weight"):
        assert piece in text


def test_tied_model_refuses_a_head_of_its_own(tmp_path):
    tensors = dict(helpers.make_tensors(helpers.TINY_A, 0))
    tensors["lm_head.weight"] = torch.zeros(512, 64, dtype=torch.bfloat16)
    write_model_folder(str(tmp_path), helpers.TINY_A, tensors)
    with pytest.raises(WeightError) as e:
        load_weights(str(tmp_path), helpers.tensor_specs_of(helpers.TINY_A), torch.bfloat16, "cpu")
    assert e.value.unexpected == ["lm_head.weight"]


def test_empty_folder(tmp_path):
    with pytest.raises(WeightError):
        load_weights(str(tmp_path), helpers.tensor_specs_of(helpers.TINY_A), torch.bfloat16, "cpu")
