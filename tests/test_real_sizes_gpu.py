"""The engine at LFM2-1.2B layer sizes (hidden 2048, 32/8 heads of 64, intermediate 5632,
vocabulary 65536) with random weights, against the plain implementation: the first three
layers (conv, conv, attention), so that the float64 reference stays within seconds.  Every
tensor-core and weight-streaming kernel runs at the shapes the benchmark uses: a portion long
enough for the persistent product and the tiled attention (200 rows), the cluster split-K
product (40 rows), and single tokens for the skinny product and the decode attention.
"""

import json

import pytest
import torch

import helpers
import plain_lfm2
import replay
from shiso_llm_b200.cli import preset_path
from shiso_llm_b200.config import plan_from_document
from shiso_llm_b200.engine import Engine, EngineOptions
from shiso_llm_b200.parts import BuildEnv, Model
from shiso_llm_b200.weights import random_tensors
from shiso_llm_b200.weights.loader import target_dtype
from tolerances import check_logits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sized():
    document = json.load(open(preset_path("lfm2-1.2b")))
    document["layer_types"] = document["layer_types"][:3]
    document["num_hidden_layers"] = 3
    _, _, plan = plan_from_document(document)
    specs = Model(plan, BuildEnv(torch.float32, torch.device("cpu"), None)).tensor_specs()
    stored = random_tensors(specs, 7, 0.02, "bfloat16", 0.1)
    tokens = helpers.random_prompt(248, document["vocab_size"], 3)
    reference = plain_lfm2.plain_forward(document, stored, tokens)
    return document, plan, specs, stored, tokens, reference


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_every_kernel_route(sized, dtype):
    from shiso_llm_b200.kernels import ops

    document, plan, specs, stored, tokens, reference = sized
    compute = torch.float32 if dtype == "float32" else torch.bfloat16
    by = {s.name: s for s in specs}
    tensors = {k: v.to("cuda", target_dtype(by[k], v.dtype, compute)) for k, v in stored.items()}
    options = EngineOptions(dtype=dtype, ctx=512, page_size=16, kv_cache_tokens=1024, max_num_seqs=2,
                            max_num_batched_tokens=256)
    engine = Engine.from_plan(plan, tensors, options, ops)
    steps = helpers.portions("a", tokens, [200, 40] + [1] * 8)
    rows = helpers.run_steps(engine, steps)
    ops.check_kernel_status()
    got = replay.stack_rows(rows, "a", len(tokens))
    check_logits(got, reference, dtype, f"1.2B layer sizes, {dtype}")
    whole = replay.stack_rows(helpers.run_steps(engine, helpers.whole("b", tokens)), "b", len(tokens))
    check_logits(whole, reference, dtype, f"1.2B layer sizes whole, {dtype}")


@pytest.fixture(scope="module")
def sized_long(sized):
    document, plan, specs, stored, _, _ = sized
    a = helpers.random_prompt(640, document["vocab_size"], 5)
    b = helpers.random_prompt(290, document["vocab_size"], 6)
    return a, b, plain_lfm2.plain_forward(document, stored, a), plain_lfm2.plain_forward(document, stored, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_long_portions_and_mixed_steps(sized, sized_long, dtype):
    """Two requests at the same layer sizes through the routes only long steps take: a 600-row
    portion (products on SM pairs, attention in tensor memory, the short conv over runs of rows),
    a mixed step of a 20-row portion deep in one sequence beside the first 260 rows of another,
    decode steps of two rows (the weight-streaming products with the row scale applied to their
    accumulators) with one request further along than the other, and a 12-row portion."""
    from shiso_llm_b200.kernels import ops

    document, plan, specs, stored, _, _ = sized
    a, b, ref_a, ref_b = sized_long
    compute = torch.float32 if dtype == "float32" else torch.bfloat16
    by = {s.name: s for s in specs}
    tensors = {k: v.to("cuda", target_dtype(by[k], v.dtype, compute)) for k, v in stored.items()}
    options = EngineOptions(dtype=dtype, ctx=1024, page_size=16, kv_cache_tokens=1024, max_num_seqs=2,
                            max_num_batched_tokens=640)
    engine = Engine.from_plan(plan, tensors, options, ops)

    def every(n):
        return list(range(n))

    steps = [
        ([("a", a[:600], every(600))], []),
        ([("a", a[600:620], every(20)), ("b", b[:260], every(260))], []),
    ]
    for i in range(8):
        steps.append(([("b", [b[260 + i]], [0]), ("a", [a[620 + i]], [0])], []))
    steps.append(([("a", a[628:640], every(12))], ["a"]))
    steps.append(([("b", b[268:290], every(22))], ["b"]))
    rows = helpers.run_steps(engine, steps)
    ops.check_kernel_status()
    check_logits(replay.stack_rows(rows, "a", len(a)), ref_a, dtype, f"long request, {dtype}")
    check_logits(replay.stack_rows(rows, "b", len(b)), ref_b, dtype, f"second request, {dtype}")
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_a_dozen_decoding_requests(sized, dtype):
    """Twelve requests of different lengths decoding together at the same layer sizes: steps of
    twelve single tokens (products with tokens as the MMA's N operand and the residual add and
    norm in their epilogues, the decode attention over twelve block tables, the serial short
    conv), after their prompts went in as one mixed step; then nine of them go on (a step of
    nine rows) while three have ended and given their pages back."""
    from shiso_llm_b200.kernels import ops

    document, plan, specs, stored, _, _ = sized
    compute = torch.float32 if dtype == "float32" else torch.bfloat16
    by = {s.name: s for s in specs}
    tensors = {k: v.to("cuda", target_dtype(by[k], v.dtype, compute)) for k, v in stored.items()}
    options = EngineOptions(dtype=dtype, ctx=256, page_size=16, kv_cache_tokens=12 * 80, max_num_seqs=12,
                            max_num_batched_tokens=512)
    engine = Engine.from_plan(plan, tensors, options, ops)
    names = [f"r{i}" for i in range(12)]
    prompts = {n: helpers.random_prompt(30 + 3 * i, document["vocab_size"], 40 + i) for i, n in enumerate(names)}
    starts = {n: 17 + 2 * i for i, n in enumerate(names)}  # rows that go in with the first step
    references = {n: plain_lfm2.plain_forward(document, stored, prompts[n]) for n in names}
    steps = [([(n, prompts[n][: starts[n]], list(range(starts[n]))) for n in names], [])]
    for k in range(8):
        steps.append(([(n, [prompts[n][starts[n] + k]], [0]) for n in names], names[:3] if k == 7 else []))
    for k in range(8, 13):
        steps.append(([(n, [prompts[n][starts[n] + k]], [0]) for n in names[3:]], names[3:] if k == 12 else []))
    rows = helpers.run_steps(engine, steps)
    ops.check_kernel_status()
    for i, n in enumerate(names):
        seen = starts[n] + (8 if i < 3 else 13)
        check_logits(replay.stack_rows(rows, n, seen), references[n][:seen], dtype, f"request {n} of twelve, {dtype}")
    engine.cache.check()


@pytest.mark.parametrize("live", [40, 80])
def test_real_layer_sizes_dozens_of_decoding_requests(sized, live):
    """Forty and eighty requests decoding together in bfloat16 at the same layer sizes: one
    token tile of 64 and two of them in the products whose K is split over a cluster (the
    residual add and norm in their epilogues, above 64 rows the gate/up pair as product and
    activation kernel), attention from the qkv rows (forty) and from queries (eighty), captured
    steps; a third of the requests end on the way and the rest go on in a smaller step."""
    from shiso_llm_b200.kernels import ops

    document, plan, specs, stored, _, _ = sized
    by = {s.name: s for s in specs}
    tensors = {k: v.to("cuda", target_dtype(by[k], v.dtype, torch.bfloat16)) for k, v in stored.items()}
    options = EngineOptions(dtype="bfloat16", ctx=128, page_size=16, kv_cache_tokens=live * 48, max_num_seqs=live,
                            max_num_batched_tokens=1024)
    engine = Engine.from_plan(plan, tensors, options, ops)
    names = [f"r{i}" for i in range(live)]
    prompts = {n: helpers.random_prompt(20 + i % 9, document["vocab_size"], 140 + i) for i, n in enumerate(names)}
    starts = {n: 6 + i % 5 for i, n in enumerate(names)}  # rows that go in with the first step
    references = {n: plain_lfm2.plain_forward(document, stored, prompts[n]) for n in names}
    early = names[: live // 3]
    steps = [([(n, prompts[n][: starts[n]], list(range(starts[n]))) for n in names], [])]
    for k in range(4):
        steps.append(([(n, [prompts[n][starts[n] + k]], [0]) for n in names], early if k == 3 else []))
    for k in range(4, 8):
        steps.append(([(n, [prompts[n][starts[n] + k]], [0]) for n in names[live // 3:]], names[live // 3:] if k == 7 else []))
    rows = helpers.run_steps(engine, steps)
    ops.check_kernel_status()
    for i, n in enumerate(names):
        seen = starts[n] + (4 if n in early else 8)
        check_logits(replay.stack_rows(rows, n, seen), references[n][:seen], "bfloat16", f"request {n} of {live}")
    engine.cache.check()
