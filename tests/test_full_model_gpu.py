"""The whole LFM2-1.2B-shaped model - the unmodified preset, all 16 layers - at the context the
benchmark runs, against the plain implementation evaluated in float64 on the GPU.

One schedule, run in float32 and in bfloat16, over 21 token sequences with random weights:

1. a 2,048-token prompt as ONE step (the products on SM pairs, attention in tensor memory,
   the short convolution over runs of rows), logits at rows spread over the prompt;
2. twenty more 2,048-token prompts, then decode steps at positions >= 2,048 with 20 live
   requests (22 steps), 8 live (21 steps) and 1 live (21 steps): captured graphs, the
   tensor-memory products with tokens as the N operand, the weight-streaming products, the
   split-key decode attention over block tables of 130 pages;
3. the first prompt again under another name, read in 512-token portions beside three requests
   that decode (steps of 515 rows), its last 64 tokens as a step of 67 rows beside the same three
   (the 65..192-row route: two token tiles, K split over a cluster);
4. the pool holds 20 requests and a few pages more, so the requests of (2) take the pages that
   (1) gave back and the request of (3) takes pages of requests that ended in (2).

The comparison is teacher-forced: every request's tokens are fixed in advance, so a wrong
logit cannot hide behind a different continuation.  Budgets: ``tolerances.check_logits`` for
float32 and ``tolerances.check_logits_deep`` for bfloat16 (top-64 overlap and worst change of
log-probability over the plain implementation's top 64, after the reference's parity budgets,
crates/shiso-bench/src/compare.rs:66-118, and its split and batch bounds,
crates/shiso-models/tests/lfm2_forward.rs:259-289,302-380).
"""

import json

import pytest
import torch

import helpers
import plain_lfm2
from shiso_llm_b200.cli import preset_path
from shiso_llm_b200.config import plan_from_document
from shiso_llm_b200.engine import Engine, EngineOptions
from shiso_llm_b200.parts import BuildEnv, Model
from shiso_llm_b200.weights.spec import VECTOR
from tolerances import check_logits, check_logits_deep

pytestmark = pytest.mark.gpu

PROMPT = 2048
LIVE = 20
PHASES = ((20, 22), (8, 21), (1, 21))  # (live requests, decode steps): 64 steps for request 0
SPREAD_ROWS = [0, 1, 2, 15, 16, 17, 63, 64, 127, 128, 129, 511, 512, 1023, 1024, 1500, 2046, 2047]


def device_weights(specs, seed, std=0.02, jitter=0.1):
    """Random weights made on the GPU whose values are exact in bfloat16 (so that both engines
    and the plain implementation see the same numbers); norm weights are jittered around 1."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    out = {}
    for spec in sorted(specs, key=lambda s: s.name):
        if spec.init == "normal":
            t = torch.empty(spec.shape, dtype=torch.float32, device="cuda").normal_(0.0, std, generator=gen)
        elif spec.init == "ones":
            t = 1.0 + jitter * torch.empty(spec.shape, dtype=torch.float32, device="cuda").normal_(0.0, 1.0, generator=gen)
        else:
            t = torch.zeros(spec.shape, dtype=torch.float32, device="cuda")
        out[spec.name] = t.to(torch.bfloat16)
    return out


def schedule(tokens):
    """The steps (as ``helpers.run_steps`` takes them) and, per request, the positions whose
    logits they ask for.  ``tokens[name]`` is each request's full token list."""
    steps, wanted = [], {}

    def want(name, at, places):
        wanted.setdefault(name, []).extend(at + p for p in places)

    # 1. one 2,048-row step
    steps.append(([("whole", tokens["whole"][:PROMPT], SPREAD_ROWS)], ["whole"]))
    want("whole", 0, SPREAD_ROWS)
    # 2. twenty prompts, then decoding with 20, 8 and 1 live requests
    names = [f"r{i}" for i in range(LIVE)]
    for n in names:
        steps.append(([(n, tokens[n][:PROMPT], [PROMPT - 1])], []))
        want(n, 0, [PROMPT - 1])
    at = {n: PROMPT for n in names}

    def decode(group, count, end_after=()):
        for k in range(count):
            entries = []
            for n in group:
                entries.append((n, [tokens[n][at[n]]], [0]))
                want(n, at[n], [0])
                at[n] += 1
            steps.append((entries, list(end_after) if k == count - 1 else []))

    decode(names, PHASES[0][1], names[8:])
    decode(names[:8], PHASES[1][1], names[4:8])
    # 3. the first prompt again in 512-row portions beside r1..r3 decoding; r0 sits these steps out
    beside = names[1:4]
    portion_rows = [0, 1, 255, 510, 511]
    for start in range(0, PROMPT, 512):
        entries = [("again", tokens["whole"][start : start + 512], portion_rows)]
        want("again", start, portion_rows)
        for n in beside:
            entries.append((n, [tokens[n][at[n]]], [0]))
            want(n, at[n], [0])
            at[n] += 1
        steps.append((entries, []))
    tail = list(range(0, 64, 9)) + [63]
    entries = [(n, [tokens[n][at[n]]], [0]) for n in beside]
    for n in beside:
        want(n, at[n], [0])
        at[n] += 1
    entries.insert(1, ("again", tokens["whole"][PROMPT : PROMPT + 64], tail))  # 67 rows, the portion in the middle
    want("again", PROMPT, tail)
    steps.append((entries, ["again"] + beside))
    # request 0 alone
    decode(names[:1], PHASES[2][1], names[:1])
    return steps, wanted


@pytest.fixture(scope="module")
def full():
    document = json.load(open(preset_path("lfm2-1.2b")))
    assert document["num_hidden_layers"] == 16 and len(document["layer_types"]) == 16
    _, _, plan = plan_from_document(document)
    specs = Model(plan, BuildEnv(torch.float32, torch.device("cpu"), None)).tensor_specs()
    stored = device_weights(specs, 11)
    vocab = document["vocab_size"]
    tokens = {"whole": helpers.random_prompt(PROMPT + 64, vocab, 100)}
    for i in range(LIVE):
        tokens[f"r{i}"] = helpers.random_prompt(PROMPT + 64, vocab, 200 + i)
    steps, wanted = schedule(tokens)
    wanted["whole"] = sorted(set(wanted["whole"]) | set(wanted.pop("again")))
    as_double = {k: v.double() for k, v in stored.items()}
    reference = {}
    for name, places in wanted.items():
        places = sorted(set(places))
        length = max(places) + 1
        logits = plain_lfm2.plain_forward(document, as_double, tokens[name][:length], device="cuda", rows=places)
        reference[name] = {p: logits[i].float().cpu() for i, p in enumerate(places)}  # float32 holds the comparison's digits
    del as_double
    torch.cuda.empty_cache()
    return document, plan, specs, stored, steps, reference


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_sixteen_layers_at_the_benchmark_context(full, dtype):
    from shiso_llm_b200.kernels import ops

    document, plan, specs, stored, steps, reference = full
    compute = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = {s.name: stored[s.name].to(torch.float32 if s.role == VECTOR else compute) for s in specs}
    pool_tokens = LIVE * (-(-(PROMPT + PHASES[0][1]) // 16) * 16) + 8 * 16
    options = EngineOptions(dtype=dtype, ctx=4096, page_size=16, kv_cache_tokens=pool_tokens, max_num_seqs=LIVE,
                            max_num_batched_tokens=PROMPT, cuda_graphs=True)
    engine = Engine.from_plan(plan, tensors, options, ops)
    rows = helpers.run_steps(engine, steps)
    ops.check_kernel_status()
    assert engine.graphs is not None and engine.graphs.replays >= sum(n for _, n in PHASES)
    engine.cache.check()
    assert engine.cache.free_pages() == [engine.cache.num_pages] and engine.cache.slots.free_slots == LIVE
    check = check_logits if dtype == "float32" else check_logits_deep
    for name, got in rows.items():
        ref_name = "whole" if name == "again" else name
        places = sorted(got)
        check(torch.stack([got[p] for p in places]), torch.stack([reference[ref_name][p] for p in places]), dtype,
              f"all 16 layers, {dtype}, request {name} at positions {places[0]}..{places[-1]}")
    # the same positions of the same tokens, once as one step and once in portions beside other requests
    both = sorted(set(rows["whole"]) & set(rows["again"]))
    assert len(both) >= 8
    a = torch.stack([rows["whole"][p] for p in both])
    b = torch.stack([rows["again"][p] for p in both])
    check(b, a, dtype, f"all 16 layers, {dtype}: the prompt in portions beside other requests against the prompt as one step")
