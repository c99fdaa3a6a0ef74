"""The command line: ``init-random`` and ``info`` need no GPU; ``generate`` has no CPU path and
says so; on a GPU ``bin/shiso generate`` runs as a user runs it, in a process of its own."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_lfm2
from shiso_llm_b200 import cli
from shiso_llm_b200.kernels.library import KernelLibraryError
from shiso_llm_b200.weights.safetensors_io import SafetensorsFile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def write_config(path, document):
    with open(path, "w") as f:
        json.dump(document, f)
    return str(path)


def test_init_random_writes_a_folder_that_info_reads(tmp_path, capsys):
    config = write_config(tmp_path / "tiny_b.json", helpers.TINY_B)
    out = tmp_path / "model"
    assert cli.main(["init-random", "--config", config, "--seed", "1", "--out", str(out)]) == 0
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    assert json.load(open(out / "config.json")) == helpers.TINY_B
    # the same (configuration, seed) gives the same bytes; another seed does not
    again, other = tmp_path / "again", tmp_path / "other"
    cli.main(["init-random", "--config", config, "--seed", "1", "--out", str(again)])
    cli.main(["init-random", "--config", config, "--seed", "2", "--out", str(other)])
    data = open(out / "model.safetensors", "rb").read()
    assert data == open(again / "model.safetensors", "rb").read() != open(other / "model.safetensors", "rb").read()
    names = set(SafetensorsFile(str(out / "model.safetensors")).names())
    assert names == {s.name for s in helpers.tensor_specs_of(helpers.TINY_B)}
    capsys.readouterr()
    assert cli.main(["info", "-m", str(out)]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["architecture"] == "Lfm2ForCausalLM"
    assert info["layers"] == ["short_conv", "short_conv", "gqa_attention", "short_conv", "gqa_attention", "gqa_attention"]
    assert info["derived"] == {"intermediate_size": 256, "head_dim": 32} and info["config"]["conv_L_cache"] == 4


def test_init_random_from_a_preset_keeps_fewer_layers(tmp_path, capsys):
    out = tmp_path / "cut"
    assert cli.main(["init-random", "--preset", "lfm2-350m", "--num-layers", "1", "--out", str(out)]) == 0
    document = json.load(open(out / "config.json"))
    assert document["num_hidden_layers"] == 1 and document["layer_types"] == ["conv"]
    with pytest.raises(SystemExit, match="unknown preset"):
        cli.main(["init-random", "--preset", "no-such-model", "--out", str(tmp_path / "x")])


@pytest.mark.skipif(torch.cuda.is_available(), reason="this is about a machine without a GPU")
def test_generate_has_no_cpu_path(tmp_path):
    helpers.make_folder(tmp_path, helpers.TINY_A, 0)
    with pytest.raises(KernelLibraryError, match="no CUDA device"):
        cli.main(["generate", "-m", str(tmp_path), "--prompt-ids", "1,2,3"])
    with pytest.raises(SystemExit):
        cli.main(["generate", "--prompt-ids", "1,2,3"])  # neither a folder nor a preset


@pytest.mark.gpu
def test_bin_shiso_generate_in_a_process_of_its_own(tmp_path):
    """Greedy ids printed by ``bin/shiso generate`` equal the plain implementation's; the dumped
    logits row of each prompt's last position matches it; the layer dump names every entry."""
    doc, seed = helpers.TINY["B"]
    folder = tmp_path / "model"
    tensors = helpers.make_folder(folder, doc, seed)
    prompts = [helpers.random_prompt(n, doc["vocab_size"], 50 + n) for n in (4, 23)]
    rows = tmp_path / "rows"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "shiso"), "generate", "-m", str(folder), "--dtype", "float32",
           "--max-tokens", "10", "--ctx", "128", "--max-num-batched-tokens", "16", "--dump-logits", str(rows),
           "--dump-layers", "1", "--bad-token-ids", "0"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")]
    assert [o["finish_reason"] for o in lines] == ["length", "length"]
    for p, o in zip(prompts, lines):
        want = plain_lfm2.plain_greedy(doc, tensors, p, 10)
        assert 0 not in want, "choose prompts whose continuation does not need the suppressed id"
        assert o["token_ids"] == want
    index = json.load(open(rows / "index.json"))["rows"]
    assert [r["prompt_tokens"] for r in index] == [4, 23]
    for p, r in zip(prompts, index):
        row = torch.from_numpy(np.load(rows / r["file"])).double()
        ref = plain_lfm2.plain_forward(doc, tensors, p)[-1]
        ref[0] = row[0]  # the suppressed id is written before the dump is taken or after; either is fine
        assert (row - ref).abs().max() <= 2e-5 * max(1.0, ref.abs().max().item())
    dump = [line for line in proc.stderr.splitlines() if " entry " in line and "rms=" in line]
    assert any("entry -1 (embedding)" in line for line in dump) and any("entry 5 (gqa_attention)" in line for line in dump)
    assert all("non_finite=0" in line for line in dump)
    # a second dump into the same folder replaces nothing
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "not empty" in proc.stderr


@pytest.mark.gpu
def test_generate_with_random_weights_of_a_preset(capsys):
    assert cli.main(["generate", "--random-config", "lfm2-350m", "--weights-seed", "3", "--prompt-len", "40", "--prompt-len", "9",
                     "--max-tokens", "5", "--ctx", "256", "--max-num-seqs", "2", "--max-num-batched-tokens", "64",
                     "--temperature", "0.8", "--top-k", "50", "--seed", "4"]) == 0
    outs = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert [len(o["token_ids"]) for o in outs] == [5, 5] and all(o["finish_reason"] == "length" for o in outs)
