"""Replay through bin/trace_run on the GPU, compared with the plain implementation.

For each tiny configuration and each compute type ONE trace_run process replays, one
after the other over the same small pool: every request alone and whole; most of a
request in one step and its last 32 tokens one by one; portions of changing size down
to two tokens (and single tokens); and a mixed trace with up to four live requests,
portions of some beside decoded tokens of others, with so few pages that they are used
again.  All wanted rows are compared with the plain implementation run on each whole
sequence.
"""

import pytest
import torch

import helpers
import plain_lfm2
import replay
from tolerances import check_logits

pytestmark = pytest.mark.gpu

LENGTHS = [70, 100, 40, 64, 7, 33, 1]
MAX_TOKENS = 320


def build_steps(requests):
    """(label, request id in trace, source request, steps) for every way of cutting."""
    steps, expect = [], []
    for rid, toks in requests.items():
        steps += helpers.whole(f"w-{rid}", toks)
        expect.append((f"whole {rid}", f"w-{rid}", rid))
    for rid in ("r0", "r1", "r3"):
        steps += helpers.tail_one_by_one(f"t-{rid}", requests[rid], 32)
        expect.append((f"tail {rid}", f"t-{rid}", rid))
    for rid, sizes in (("r1", [13, 2, 7, 64, 3]), ("r0", [2, 3, 1, 2, 5, 1, 1, 17]), ("r2", [2]), ("r5", [16, 1, 16])):
        steps += helpers.portions(f"p-{rid}", requests[rid], sizes)
        expect.append((f"portions {rid} {sizes}", f"p-{rid}", rid))
    mixed = replay.mixed_trace({f"m-{k}": v for k, v in requests.items()}, 5, MAX_TOKENS)
    steps += mixed
    expect += [(f"mixed {rid}", f"m-{rid}", rid) for rid in requests]
    mixed2 = replay.mixed_trace({f"n-{k}": v for k, v in reversed(list(requests.items()))}, 11, MAX_TOKENS, tail=3)
    steps += mixed2
    expect += [(f"mixed-b {rid}", f"n-{rid}", rid) for rid in requests]
    return steps, expect


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_all_cuts(tmp_path, name, dtype):
    doc, seed = helpers.TINY[name]
    model_dir = tmp_path / "model"
    tensors = helpers.make_folder(model_dir, doc, seed)
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab_size"], 10 + i) for i, n in enumerate(LENGTHS)}
    steps, expect = build_steps(requests)
    rows = replay.run_trace_run(model_dir, dtype, steps, MAX_TOKENS, tmp_path / "out", doc["vocab_size"])
    reference = {rid: plain_lfm2.plain_forward(doc, tensors, toks) for rid, toks in requests.items()}
    failures = []
    for label, trace_id, rid in expect:
        got = replay.stack_rows(rows, trace_id, len(requests[rid]))
        try:
            check_logits(got, reference[rid], dtype, f"{name} {dtype} {label}")
        except AssertionError as e:
            failures.append(str(e))
    assert not failures, "\n".join(failures)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuts_agree_with_each_other(tmp_path, dtype):
    """The same request whole, by single tokens and in portions, through the engine in one
    process: rows must agree far more closely than with the reference's budget."""
    doc, seed = helpers.TINY["B"]
    model_dir = tmp_path / "model"
    helpers.make_folder(model_dir, doc, seed)
    engine = helpers.make_engine(model_dir, dtype, page_size=16, kv_cache_tokens=256, ctx=256, max_num_batched_tokens=256)
    toks = helpers.random_prompt(90, doc["vocab_size"], 77)
    whole = replay.stack_rows(helpers.run_steps(engine, helpers.whole("a", toks)), "a", len(toks))
    single = replay.stack_rows(helpers.run_steps(engine, helpers.portions("b", toks, [1])), "b", len(toks))
    cut = replay.stack_rows(helpers.run_steps(engine, helpers.portions("c", toks, [5, 2, 31, 3])), "c", len(toks))
    scale = whole.std().item()
    bound = 1e-5 if dtype == "float32" else 0.05 * scale
    assert (whole - single).abs().max().item() <= bound
    assert (whole - cut).abs().max().item() <= bound
