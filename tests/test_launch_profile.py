"""The launch profiler: rows add up, and a profiled run computes what an unprofiled one does."""

import json
import os
import subprocess
import sys

import pytest
import torch

import helpers
from shiso_llm_b200.kernels.profile import LaunchTable, StepProfiler

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rows_add_up_by_kernel_and_shape(tmp_path):
    table = LaunchTable("decode steps")
    table.add_step([("linear", "8x64x32", 1, 4.0), ("rmsnorm", "8x32", 1, 1.0), ("linear", "8x64x32", 1, 6.0)], 30.0, 16.0)
    table.add_step([("linear", "8x64x32", 1, 5.0), ("linear", "8x16x32", 1, 2.0), ("short_conv", "8x32", 2, 2.0)], 20.0, 12.0)
    report = table.report()
    assert report["steps"] == 2
    assert report["device_us_per_step"] == pytest.approx(10.0)
    assert report["wall_us_per_step"] == pytest.approx(25.0)
    assert report["span_us_per_step"] == pytest.approx(14.0)
    rows = {(r["kernel"], r["shape"]): r for r in report["rows"]}
    assert rows[("linear", "8x64x32")]["us_per_step"] == pytest.approx(7.5)
    assert rows[("linear", "8x64x32")]["mean_us"] == pytest.approx(5.0)
    assert rows[("linear", "8x64x32")]["launches_per_step"] == pytest.approx(1.5)
    assert rows[("short_conv", "8x32")]["launches_per_step"] == pytest.approx(1.0)  # two launches, one of two steps
    assert report["rows"][0]["kernel"] == "linear" and report["rows"][0]["shape"] == "8x64x32"  # largest share first
    assert sum(r["share"] for r in report["rows"]) == pytest.approx(1.0)
    profiler = StepProfiler(str(tmp_path / "out"))
    profiler.add("decode", [("linear", "1x2x3", 1, 1.0)], 2.0)
    profiler.write()
    written = json.load(open(tmp_path / "out" / "launches.json"))
    assert list(written) == ["decode"] and written["decode"]["rows"][0]["kernel"] == "linear"
    assert "decode steps: 1 steps" in open(tmp_path / "out" / "launches.txt").read()


@pytest.mark.gpu
def test_profiled_generation_matches_and_counts_every_launch(tmp_path):
    from shiso_llm_b200 import LLM, SamplingParams
    from shiso_llm_b200.kernels import ops

    document, seed = helpers.TINY["A"]
    folder = str(tmp_path / "model")
    helpers.make_folder(folder, document, seed)
    prompts = [helpers.random_prompt(n, document["vocab_size"], 60 + n) for n in (21, 6)]
    params = SamplingParams(temperature=0.0, max_new_tokens=6)
    plain = LLM(folder, dtype="bfloat16", ctx=128, page_size=16, max_num_seqs=2, max_num_batched_tokens=32)
    want = [o.token_ids for o in plain.generate(prompts, params)]
    llm = LLM(folder, dtype="bfloat16", ctx=128, page_size=16, max_num_seqs=2, max_num_batched_tokens=32)
    profiler = llm.engine.enable_launch_profile(str(tmp_path / "profile"))
    before = ops.launch_count
    got = [o.token_ids for o in llm.generate(prompts, params)]
    launched = ops.launch_count - before
    llm.engine.disable_launch_profile()
    assert got == want
    report = profiler.report()
    assert set(report) == {"decode", "prompt"}
    counted = sum(r["launches_per_step"] * report[k]["steps"] for k in report for r in report[k]["rows"])
    # the picking kernels run after the step, outside the region: one or two launches a step
    steps = report["decode"]["steps"] + report["prompt"]["steps"]
    assert launched - 2 * steps <= round(counted) <= launched
    for kind in report:
        assert report[kind]["device_us_per_step"] > 0
        assert report[kind]["device_us_per_step"] <= report[kind]["span_us_per_step"] * 1.02
        assert report[kind]["span_us_per_step"] <= report[kind]["wall_us_per_step"] * 1.05
        assert any(r["kernel"].startswith("linear") and r["shape"] for r in report[kind]["rows"])
    # a step after the region is closed is replayed from its graph again and leaves no row
    steps_before = steps
    llm.generate([prompts[1]], params)
    assert sum(t.steps for t in profiler.tables.values()) == steps_before
    profiler.write()
    assert os.path.isfile(tmp_path / "profile" / "launches.txt")


@pytest.mark.gpu
def test_generate_profile_dir_from_the_command_line(tmp_path):
    document, seed = helpers.TINY["B"]
    folder = str(tmp_path / "model")
    helpers.make_folder(folder, document, seed)
    out = str(tmp_path / "profile")
    run = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "shiso"), "generate", "-m", folder, "--ctx", "128", "--prompt-ids", "5,6,7,8,9",
         "--max-tokens", "4", "--max-num-seqs", "1", "--profile-dir", out],
        capture_output=True, text=True, timeout=600,
    )
    assert run.returncode == 0, run.stderr[-2000:]
    report = json.load(open(os.path.join(out, "launches.json")))
    assert report["prompt"]["steps"] == 1 and report["decode"]["steps"] == 3
    assert "us/step" in run.stderr
