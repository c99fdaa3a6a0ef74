"""The engine end to end, twice: on the CPU with the plain stand-in kernels (which checks the
step function, the cache and the scheduler), and on the GPU with the CUDA kernels
(``-m gpu``).  Same bodies, same tolerances.
"""

import pytest
import torch

import fake_kernels
import helpers
import plain_lfm2
import replay
import toy_parts
from shiso_llm_b200 import LLM, SamplingParams
from shiso_llm_b200.cache import OutOfPages
from shiso_llm_b200.config import register_architecture, unregister_architecture
from shiso_llm_b200.engine import Engine, EngineOptions, StepEntry
from shiso_llm_b200.sampling import host as host_sampling
from shiso_llm_b200.weights import random_tensors
from tolerances import check_logits


def _fake_sample(logits, temperature, top_k, top_p, min_p, keys, positions, out=None, status_out=None):
    fake_kernels.hand_over_status(status_out)
    picks = []
    for r in range(logits.shape[0]):
        p = SamplingParams(temperature=float(temperature[r]), top_k=int(top_k[r]), top_p=float(top_p[r]), min_p=float(min_p[r]))
        picks.append(host_sampling.keyed_sample(logits[r].numpy(), p, int(keys[r]), int(positions[r])))
    picks = torch.tensor(picks, dtype=torch.int32)
    if out is None:
        return picks
    out.copy_(picks)
    return out


fake_kernels.sample = _fake_sample

BACKENDS = [pytest.param("cpu", id="plain-kernels-cpu"), pytest.param("cuda", id="cuda", marks=pytest.mark.gpu)]


def backend_args(backend):
    if backend == "cpu":
        return {"ops": fake_kernels, "device": "cpu"}
    return {"ops": None, "device": "cuda:0"}


def dtypes(backend):
    return ["float32"] if backend == "cpu" else ["float32", "bfloat16"]


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["A", "B"])
def test_every_cut_matches_the_plain_implementation(tmp_path, backend, name):
    doc, seed = helpers.TINY[name]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    lengths = [70, 40, 7, 33, 1]
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab_size"], 10 + i) for i, n in enumerate(lengths)}
    reference = {rid: plain_lfm2.plain_forward(doc, tensors, toks) for rid, toks in requests.items()}
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=4, kv_cache_tokens=192, ctx=128,
                                     max_num_batched_tokens=128, **backend_args(backend))
        steps, expect = [], []
        for rid, toks in requests.items():
            steps += helpers.whole(f"w-{rid}", toks)
            expect.append((f"w-{rid}", rid))
        steps += helpers.tail_one_by_one("t-r0", requests["r0"], 32)
        steps += helpers.portions("p-r0", requests["r0"], [13, 2, 7, 1, 3])
        steps += helpers.portions("p-r3", requests["r3"], [2])
        expect += [("t-r0", "r0"), ("p-r0", "r0"), ("p-r3", "r3")]
        steps += replay.mixed_trace({f"m-{k}": v for k, v in requests.items()}, 3, 192)
        expect += [(f"m-{rid}", rid) for rid in requests]
        rows = helpers.run_steps(engine, steps)
        for trace_id, rid in expect:
            got = replay.stack_rows(rows, trace_id, len(requests[rid]))
            check_logits(got, reference[rid], dtype, f"{name} {dtype} {trace_id}")
        assert engine.cache.free_pages() == [48] and engine.cache.slots.free_slots == 4


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_and_first_tokens(tmp_path, backend):
    """400 tokens one by one (pages cross, the rotation reaches large angles), and the very
    first positions of a sequence (conv state still empty, a single key)."""
    doc, seed = helpers.TINY["B"]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    toks = helpers.random_prompt(400, doc["vocab_size"], 5)
    ref = plain_lfm2.plain_forward(doc, tensors, toks)
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=16, kv_cache_tokens=512, ctx=512,
                                     max_num_batched_tokens=64, **backend_args(backend))
        rows = helpers.run_steps(engine, helpers.portions("a", toks, [1]))
        check_logits(replay.stack_rows(rows, "a", 400), ref, dtype, f"long decode {dtype}")
        rows = helpers.run_steps(engine, helpers.portions("b", toks[:6], [1, 2, 3]))
        check_logits(replay.stack_rows(rows, "b", 6), ref[:6], dtype, f"first tokens {dtype}")


@pytest.mark.parametrize("backend", BACKENDS)
def test_greedy_generation_through_the_entry_point(tmp_path, backend):
    for name in ("A", "B"):
        doc, seed = helpers.TINY[name]
        folder = tmp_path / name
        tensors = helpers.make_folder(folder, doc, seed)
        prompts = [helpers.random_prompt(n, doc["vocab_size"], 20 + n) for n in (5, 17, 33)]
        want = [plain_lfm2.plain_greedy(doc, tensors, p, 16) for p in prompts]
        llm = LLM(str(folder), dtype="float32", ctx=128, page_size=16, max_num_seqs=4, max_num_batched_tokens=32,
                  prefill_chunk=13, **backend_args(backend))
        seen = {}  # (request, position) -> the logits row a token was picked from

        def tap(plan, logits, seen=seen):
            rows = logits.float().cpu()
            for row, entry in zip(rows, [e for e in plan.entries if e.samples]):
                seen[(entry.request.id, entry.start + entry.count - 1)] = row

        llm.logits_tap = tap
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=16))
        assert [o.token_ids for o in outs] == want and all(o.finish_reason == "length" for o in outs)
        # equal ids say little where the tiny model repeats itself: every row a token was picked from
        # is compared too
        for out, prompt in zip(outs, prompts):
            ref = plain_lfm2.plain_forward(doc, tensors, prompt + out.token_ids[:-1])
            places = range(len(prompt) - 1, len(prompt) + 15)
            got = torch.stack([seen[(out.request_id, p)] for p in places])
            check_logits(got, ref[len(prompt) - 1 :], "float32", f"rows that generation picked from, tiny {name}")
        llm.engine.cache.check()
        assert llm.engine.cache.slots.free_slots == 4


@pytest.mark.parametrize("backend", BACKENDS)
def test_sampling_is_the_same_under_every_cut_and_after_preemption(tmp_path, backend):
    """Tiny B's workload: prompts of 1, 7, 40, 64 and 100 tokens as a mixed batch with 13-token
    portions beside decode, 24 steps at temperature 0.8 with seed 1; then again with a pool
    so small that requests are preempted and recomputed."""
    doc, seed = helpers.TINY["B"]
    helpers.make_folder(tmp_path, doc, seed)
    prompts = [helpers.random_prompt(n, doc["vocab_size"], 30 + n) for n in (1, 7, 40, 64, 100)]
    params = SamplingParams(temperature=0.8, seed=1, max_new_tokens=24, top_k=200, top_p=0.95)
    roomy = LLM(str(tmp_path), dtype="float32", ctx=256, page_size=16, max_num_seqs=5, max_num_batched_tokens=256,
                lookahead=False, **backend_args(backend))
    base = roomy.generate(prompts, params)
    assert all(len(o.token_ids) == 24 and o.preemptions == 0 for o in base)
    assert len({tuple(o.token_ids) for o in base}) == 5
    cut = LLM(str(tmp_path), dtype="float32", ctx=256, page_size=16, max_num_seqs=4, max_num_batched_tokens=32,
              prefill_chunk=13, **backend_args(backend))
    assert [o.token_ids for o in cut.generate(prompts, params)] == [o.token_ids for o in base]
    tight = LLM(str(tmp_path), dtype="float32", ctx=256, page_size=16, kv_cache_tokens=208, allow_small_pool=True, max_num_seqs=4,
                max_num_batched_tokens=32, prefill_chunk=13, **backend_args(backend))
    outs = tight.generate(prompts, params)
    assert [o.token_ids for o in outs] == [o.token_ids for o in base]
    assert tight.scheduler.stats["preempted"] > 0
    tight.engine.cache.check()
    failing = LLM(str(tmp_path), dtype="float32", ctx=256, page_size=16, kv_cache_tokens=208, allow_small_pool=True, max_num_seqs=4,
                  max_num_batched_tokens=32, prefill_chunk=13, on_exhaustion="fail", **backend_args(backend))
    outs = failing.generate(prompts, params)
    assert any(o.finish_reason == "error" and "kv pool" in o.error for o in outs)
    for o, b in zip(outs, base):
        if o.finish_reason == "length":
            assert o.token_ids == b.token_ids
    assert failing.engine.cache.free_pages() == [13]


@pytest.mark.parametrize("backend", BACKENDS)
def test_lookahead_gives_the_same_tokens_and_stops(tmp_path, backend):
    """Planning a step before the last one's tokens have reached the host changes no token: greedy
    and sampled requests side by side, one of which ends on a stop token (found in the output of
    a first run), through a pool small enough to preempt."""
    doc, seed = helpers.TINY["A"]
    helpers.make_folder(tmp_path, doc, seed)
    prompts = [helpers.random_prompt(n, doc["vocab_size"], 60 + n) for n in (3, 21, 50, 9)]

    def run(lookahead, stop, **kw):
        params = [
            SamplingParams(temperature=1.0, seed=6, top_k=50, max_new_tokens=20, stop_token_ids=stop),
            SamplingParams(temperature=0.7, seed=5, max_new_tokens=12),
            SamplingParams(temperature=0.0, max_new_tokens=1),
            SamplingParams(temperature=0.0, max_new_tokens=20),
        ]
        llm = LLM(str(tmp_path), dtype="float32", ctx=128, page_size=16, max_num_seqs=4, max_num_batched_tokens=24,
                  prefill_chunk=11, lookahead=lookahead, **kw, **backend_args(backend))
        outs = llm.generate(prompts, params)
        llm.engine.cache.check()
        assert llm.engine.cache.slots.free_slots == 4 and not llm.has_unfinished()
        return [(o.token_ids, o.finish_reason) for o in outs], llm

    free_run, _ = run(False, ())
    first = free_run[0][0]
    cut = next((i for i in range(3, len(first)) if first[i] not in first[:i]), None)
    assert cut is not None, "the tiny model repeats itself too early for this test"
    stop = (first[cut],)  # a token the first request reaches after a few steps ends it from now on
    waited, _ = run(False, stop)
    ahead, llm = run(True, stop)
    assert waited == ahead
    assert ahead[0] == (first[:cut], "stop") and ahead[1:] == free_run[1:]
    # one row was computed past the stop before the host knew of it
    assert llm.scheduler.stats["decode_tokens"] == run(False, stop)[1].scheduler.stats["decode_tokens"] + 1


@pytest.mark.parametrize("backend", BACKENDS)
def test_step_refusals_leave_the_cache_as_it_was(tmp_path, backend):
    doc, seed = helpers.TINY["A"]
    helpers.make_folder(tmp_path, doc, seed)
    engine = helpers.make_engine(tmp_path, "float32", page_size=4, kv_cache_tokens=32, ctx=32, max_num_seqs=2,
                                 max_num_batched_tokens=64, **backend_args(backend))
    engine.step([StepEntry("a", [1, 2, 3, 4, 5], [4])])
    before = (engine.cache.free_pages(), engine.cache.length("a"))
    with pytest.raises(ValueError):
        engine.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    with pytest.raises(ValueError):
        engine.step([StepEntry("a", [512], [0])])
    with pytest.raises(ValueError):
        engine.step([StepEntry("a", [], [])])
    with pytest.raises(ValueError):
        engine.step([StepEntry("a", [1, 2], [2])])
    with pytest.raises(OutOfPages):
        engine.step([StepEntry("a", [1] * 20, []), StepEntry("b", [1] * 12, [])])
    assert (engine.cache.free_pages(), engine.cache.length("a")) == before and not engine.cache.has("b")
    engine.step([StepEntry("b", [1, 2], []), StepEntry("a", [7], [0])])
    with pytest.raises(OutOfPages):
        engine.step([StepEntry("c", [1], [0])])  # no state slot left
    engine.finish("a")
    engine.finish("b")
    engine.cache.check()
    assert engine.cache.free_pages() == [8]


@pytest.mark.parametrize("backend", BACKENDS)
def test_toy_parts_register_build_and_step_without_touching_the_framework(backend):
    """A mixer with state of its own, a routed feed-forward and another position encoding,
    defined in tests/toy_parts.py; a run order that names a layer twice and lets a layer read
    another entry's cache; a windowed cache group whose pages come back."""
    toy_parts.register()
    try:
        plan = toy_parts.toy_plan()
        args = backend_args(backend)
        from shiso_llm_b200.parts import BuildEnv, Model

        specs = Model(plan, BuildEnv(torch.float32, torch.device("cpu"), None)).tensor_specs()
        stored = random_tensors(specs, 3, 0.08, "bfloat16", 0.1)
        ids = helpers.random_prompt(45, toy_parts.VOCAB, 9)
        ref = toy_parts.toy_reference(stored, ids)
        options = EngineOptions(dtype="float32", ctx=64, page_size=4, kv_cache_tokens=64, max_num_seqs=2,
                                max_num_batched_tokens=64, device=args["device"])
        ops = args["ops"]
        if ops is None:
            from shiso_llm_b200.kernels import ops
        from shiso_llm_b200.weights.loader import target_dtype

        by_name = {s.name: s for s in specs}
        tensors = {k: v.to(args["device"], target_dtype(by_name[k], v.dtype, torch.float32)) for k, v in stored.items()}
        engine = Engine.from_plan(plan, tensors, options, ops)
        assert engine.graphs is None  # the toy mixer is not graph-safe
        needs = engine.model.cache_needs()
        assert [type(n).__name__ for n in needs] == ["FixedState", "PagedKV", "FixedState", "NoneType"]
        for cut in ([45], [1], [7, 2, 1, 13]):
            rows = helpers.run_steps(engine, helpers.portions("t", ids, cut))
            check_logits(replay.stack_rows(rows, "t", 45), ref, "float32", f"toy model cut {cut}")
        # a window of 6 with pages of 4: at most 3 pages of the 12 a full cache would need
        engine.step([StepEntry("w", ids, [])])
        assert sum(p >= 0 for p in engine.cache.block_table("w", 0)) <= 3
        engine.finish("w")
        engine.cache.check()
    finally:
        toy_parts.unregister()


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_plan_with_a_portion_grid_typed_state_and_narrow_values(backend):
    """A toy model whose plan names ``portion_multiple`` 4, whose first mixer keeps float64
    state and refuses portions that start off the grid, and whose second mixer caches values
    narrower than its keys in float32: built and generated with through the scheduler, which
    must cut every prompt on the grid, without a change to the package."""
    toy_parts.register()
    try:
        plan = toy_parts.grid_plan()
        args = backend_args(backend)
        from shiso_llm_b200.parts import BuildEnv, Model
        from shiso_llm_b200.weights.loader import target_dtype

        specs = Model(plan, BuildEnv(torch.float32, torch.device("cpu"), None)).tensor_specs()
        stored = random_tensors(specs, 5, 0.08, "bfloat16", 0.1)
        ops = args["ops"]
        if ops is None:
            from shiso_llm_b200.kernels import ops
        by_name = {s.name: s for s in specs}
        tensors = {k: v.to(args["device"], target_dtype(by_name[k], v.dtype, torch.float32)) for k, v in stored.items()}
        options = EngineOptions(dtype="float32", ctx=64, page_size=4, max_num_seqs=3, max_num_batched_tokens=16, device=args["device"])
        engine = Engine.from_plan(plan, tensors, options, ops)
        needs = engine.model.cache_needs()
        assert needs[0].dtype == torch.float64 and needs[1].value_dim == toy_parts.V_DIM and needs[1].dtype == torch.float32
        ids = helpers.random_prompt(30, toy_parts.VOCAB, 12)
        ref = toy_parts.grid_reference(stored, ids)
        rows = helpers.run_steps(engine, helpers.portions("g", ids, [8, 4, 12, 4, 2]))  # every start on the grid
        check_logits(replay.stack_rows(rows, "g", 30), ref, "float32", "grid model in portions")
        with pytest.raises(AssertionError, match="off the grid"):
            helpers.run_steps(engine, helpers.portions("bad", ids, [5, 3]))
        engine.finish("bad")

        def greedy(prompt, steps):
            out, seq = [], list(prompt)
            for _ in range(steps):
                out.append(int(toy_parts.grid_reference(stored, seq)[-1].argmax()))
                seq.append(out[-1])
            return out

        prompts = [helpers.random_prompt(n, toy_parts.VOCAB, 20 + n) for n in (3, 13, 22, 9)]
        # 16 tokens a step, portions of at most 10: cut to 8 beside decode rows; lengths 13 and 22 end off the grid
        llm = LLM(engine, prefill_chunk=10)
        assert llm.scheduler.config.portion_multiple == 4
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=6))
        assert [o.token_ids for o in outs] == [greedy(p, 6) for p in prompts]
        assert llm.scheduler.stats["steps"] > 6
        engine.cache.check()
        with pytest.raises(ValueError, match="could never advance"):
            LLM(engine, prefill_chunk=3)
    finally:
        toy_parts.unregister()


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_head_size_that_is_no_multiple_of_16(tmp_path, backend):
    """hidden 96 with 4 heads gives heads of 24: legal for the architecture, and run by the
    general kernels in both compute types."""
    doc = dict(helpers.TINY_B, num_attention_heads=4, num_key_value_heads=2)
    tensors = helpers.make_folder(tmp_path, doc, 4)
    toks = helpers.random_prompt(50, doc["vocab_size"], 8)
    ref = plain_lfm2.plain_forward(doc, tensors, toks)
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=8, kv_cache_tokens=128, ctx=128, max_num_batched_tokens=64,
                                     **backend_args(backend))
        assert engine.config.head_dim == 24
        steps = helpers.whole("w", toks) + helpers.portions("p", toks, [7, 1, 20, 2]) + helpers.tail_one_by_one("t", toks, 12)
        rows = helpers.run_steps(engine, steps)
        for name in "wpt":
            check_logits(replay.stack_rows(rows, name, 50), ref, dtype, f"head size 24, {dtype}, {name}")


@pytest.mark.gpu
def test_more_decode_batch_sizes_than_captured_graphs_are_kept(tmp_path):
    """Thirty requests that end one after the other: decode steps of 30, 29, .. 1 rows run as
    the captured sizes 32, 24, 16 (made-up rows behind the step's own) and 8 .. 1; only four
    graphs are kept here, so the graph for 32 is dropped meanwhile and captured anew when 30
    rows come again.  Logits stay those of the plain implementation throughout."""
    doc, seed = helpers.TINY["A"]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    count = 30
    for dtype in ("float32", "bfloat16"):
        engine = helpers.make_engine(tmp_path, dtype, page_size=16, ctx=64, max_num_seqs=count, max_num_batched_tokens=256)
        assert engine.graphs is not None
        engine.graphs.max_graphs = 4
        names = [f"r{i}" for i in range(count)]
        tokens = {n: helpers.random_prompt(6 + count + 3, doc["vocab_size"], 300 + i) for i, n in enumerate(names)}
        steps = [([(n, tokens[n][:6], [5]) for n in names], [])]
        at = 6
        for live in range(count, 0, -1):  # after a step of `live` rows the last of them ends
            steps.append(([(n, [tokens[n][at]], [0]) for n in names[:live]], [names[live - 1]]))
            at += 1
        rows = helpers.run_steps(engine, steps)
        assert sorted(engine.graphs._graphs) == [1, 2, 3, 4]
        again = [f"s{i}" for i in range(count)]
        steps = [([(n, tokens[f"r{i}"][:6], [5]) for i, n in enumerate(again)], []),
                 ([(n, [tokens[f"r{i}"][6]], [0]) for i, n in enumerate(again)], again)]
        rows.update(helpers.run_steps(engine, steps))
        assert 32 in engine.graphs._graphs and len(engine.graphs._graphs) == 4
        for i, n in enumerate(names):
            decoded = count - i  # request i took part in the steps of 30 .. i + 1 rows
            ref = plain_lfm2.plain_forward(doc, tensors, tokens[n][: 6 + decoded])
            places = sorted(rows[n])
            assert places == list(range(5, 6 + decoded))
            check_logits(torch.stack([rows[n][p] for p in places]), ref[5:], dtype, f"request {n} through {decoded} batch sizes, {dtype}")
            check_logits(torch.stack([rows[f"s{i}"][p] for p in (5, 6)]), ref[5:7], dtype, f"request s{i} after the graph came back")
        engine.cache.check()


def test_a_padded_step_leaves_the_entries_rows_as_they_are(tmp_path):
    """The padding of a captured shape - made-up sequences on scratch pages and a scratch slot,
    wanted rows filled up - changes nothing for the step's own rows, sequences and state: the
    same trace through padded steps and through plain steps gives the same logits, with the
    plain stand-in kernels on the CPU."""
    from shiso_llm_b200.engine.batch import StepBuilder
    from shiso_llm_b200.engine.graphs import padded_shape

    assert padded_shape(2048, 1) == (2048, 1) and padded_shape(512, 4) == (512, 4)  # on the grid already: taken as they are
    assert padded_shape(2049, 1) == (2112, 2) and padded_shape(512, 3) == (576, 4) and padded_shape(70, 4) == (128, 8)
    assert padded_shape(549, 38) == (576, 64) and padded_shape(5, 2) == (16, 4) and padded_shape(16, 2) == (16, 2)

    doc, seed = helpers.TINY["B"]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab_size"], 40 + i) for i, n in enumerate((37, 21, 9, 50))}
    reference = {rid: plain_lfm2.plain_forward(doc, tensors, toks) for rid, toks in requests.items()}
    engine = helpers.make_engine(tmp_path, "float32", ops=fake_kernels, page_size=4, kv_cache_tokens=256, ctx=64,
                                 max_num_seqs=4, max_num_batched_tokens=64)
    assert engine.cache.scratch_slot == 4 and len(engine.cache.scratch_pages) == 16
    builder = StepBuilder(engine.cache, "cpu", 128, 8, fixed_table_width=engine.cache.max_blocks)
    rows, consumed = {}, {}
    for entries, end in replay.mixed_trace(requests, 7, 256):
        batch = [StepEntry(r, t, w[-1:]) for r, t, w in entries]  # at most one wanted row per sequence
        padded_rows, seqs = padded_shape(sum(len(e.tokens) for e in batch), len(batch))
        shape = (padded_rows, seqs, seqs)
        starts = [engine.cache.append(e.request, len(e.tokens)) for e in batch]
        meta = builder.build(batch, starts, pad=shape)
        assert (meta.num_tokens, meta.num_seqs, meta.num_wanted) == shape and not meta.h_q_start
        logits = engine.model.forward(meta, engine.cache)
        at = 0
        for e in batch:
            engine.cache.commit(e.request)
            base = consumed.get(e.request, 0)
            for w in e.want:
                rows.setdefault(e.request, {})[base + w] = logits[at].clone()
                at += 1
            consumed[e.request] = base + len(e.tokens)
        for r in end:
            engine.finish(r)
        engine.cache.check()
    for rid, toks in requests.items():
        places = sorted(rows[rid])
        assert len(places) > 5
        check_logits(torch.stack([rows[rid][p] for p in places]), reference[rid][places], "float32", f"padded steps, {rid}")
    assert engine.cache.free_pages() == [64] and engine.cache.slots.free_slots == 4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_steps_replayed_from_captured_graphs(tmp_path, dtype):
    """The same mixed trace twice under other names: every shape of the first pass that comes
    again is captured and replayed (portions beside decoded tokens, padded to the shape), pages
    and slots are reused between the passes, and every logits row is the plain implementation's."""
    doc, seed = helpers.TINY["B"]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    lengths = [70, 40, 7, 33, 90, 64]
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab_size"], 60 + i) for i, n in enumerate(lengths)}
    reference = {rid: plain_lfm2.plain_forward(doc, tensors, toks) for rid, toks in requests.items()}
    engine = helpers.make_engine(tmp_path, dtype, page_size=16, kv_cache_tokens=320, ctx=128, max_num_seqs=4,
                                 max_num_batched_tokens=128)
    assert engine.step_graphs is not None
    for round_ in range(3):
        trace = replay.mixed_trace({f"{round_}-{k}": v for k, v in requests.items()}, 5, 320, portion_sizes=(2, 3, 16, 31, 13))
        trace = [([(r, t, w[-1:]) for r, t, w in entries], end) for entries, end in trace]
        rows = helpers.run_steps(engine, trace)
        for rid, toks in requests.items():
            places = sorted(rows[f"{round_}-{rid}"])
            got = torch.stack([rows[f"{round_}-{rid}"][p] for p in places])
            check_logits(got, reference[rid][places], dtype, f"round {round_} {dtype} {rid}")
    from shiso_llm_b200.kernels import ops

    ops.check_kernel_status()
    assert engine.step_graphs.captures >= 3 and engine.step_graphs.replays > 20
    engine.cache.check()


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_model_that_reads_a_further_per_row_input(backend):
    """A plan may name further int arrays with one value per row (``row_inputs``): entries bring
    them (``StepEntry.extras``), requests bring them for their prompt (``add_request(..,
    extras=..)``), rows without a value get their position, and a toy mixer reads them from the
    step - cut into portions and mixed with other requests like everything else."""
    toy_parts.register()
    try:
        plan = toy_parts.segment_plan()
        args = backend_args(backend)
        from shiso_llm_b200.parts import BuildEnv, Model
        from shiso_llm_b200.weights.loader import target_dtype

        specs = Model(plan, BuildEnv(torch.float32, torch.device("cpu"), None)).tensor_specs()
        stored = random_tensors(specs, 8, 0.3, "bfloat16", 0.1)
        ops = args["ops"]
        if ops is None:
            from shiso_llm_b200.kernels import ops
        by_name = {s.name: s for s in specs}
        tensors = {k: v.to(args["device"], target_dtype(by_name[k], v.dtype, torch.float32)) for k, v in stored.items()}
        options = EngineOptions(dtype="float32", ctx=64, page_size=4, max_num_seqs=3, max_num_batched_tokens=32, device=args["device"])
        engine = Engine.from_plan(plan, tensors, options, ops)
        ids_a, ids_b = helpers.random_prompt(20, toy_parts.VOCAB, 1), helpers.random_prompt(9, toy_parts.VOCAB, 2)
        seg_a = [(7 * i) % 11 for i in range(20)]
        ref_a = toy_parts.segment_reference(stored, ids_a, seg_a)
        ref_b = toy_parts.segment_reference(stored, ids_b, list(range(9)))  # no values given: the positions
        steps = [
            [StepEntry("a", ids_a[:6], list(range(6)), extras={"segment": seg_a[:6]}), StepEntry("b", ids_b[:4], list(range(4)))],
            [StepEntry("b", ids_b[4:], list(range(5))), StepEntry("a", ids_a[6:19], list(range(13)), extras={"segment": seg_a[6:19]})],
            [StepEntry("a", ids_a[19:], [0], extras={"segment": seg_a[19:]})],
        ]
        got_a, got_b = [], []
        for entries in steps:
            logits = engine.step(entries).cpu()
            at = 0
            for e in entries:
                (got_a if e.request == "a" else got_b).append(logits[at : at + len(e.want)])
                at += len(e.want)
        check_logits(torch.cat(got_a), ref_a, "float32", "per-row input given by the entries")
        check_logits(torch.cat(got_b), ref_b, "float32", "per-row input left to the positions")
        with pytest.raises(ValueError, match="no per-row input named"):
            engine.step([StepEntry("c", [1, 2], [], extras={"colour": [0, 0]})])
        with pytest.raises(ValueError, match="values of 'segment' for 2 tokens"):
            engine.step([StepEntry("c", [1, 2], [], extras={"segment": [0]})])
        assert not engine.cache.has("c")
        engine.finish("a"), engine.finish("b")

        # through the entry point: the prompt's values come with the request, produced tokens get their position
        def greedy(prompt, segments, steps):
            seq, seg, out = list(prompt), list(segments), []
            for _ in range(steps):
                out.append(int(toy_parts.segment_reference(stored, seq, seg)[-1].argmax()))
                seg.append(len(seq))
                seq.append(out[-1])
            return out

        llm = LLM(engine, prefill_chunk=7)
        llm.add_request(ids_a, SamplingParams(temperature=0.0, max_new_tokens=5), extras={"segment": seg_a})
        llm.add_request(ids_b, SamplingParams(temperature=0.0, max_new_tokens=5))
        done = []
        while llm.has_unfinished():
            done += llm.step()
        done += llm.drain()
        by_id = {o.request_id: o.token_ids for o in done}
        assert by_id[0] == greedy(ids_a, seg_a, 5) and by_id[1] == greedy(ids_b, list(range(9)), 5)
        with pytest.raises(ValueError, match="no per-row input"):
            llm.add_request(ids_b, extras={"colour": [0] * 9})
        refused = llm.add_request(ids_b, extras={"segment": [1, 2]})
        assert refused.finish_reason == "error" and "values of 'segment'" in refused.error
    finally:
        toy_parts.unregister()


@pytest.mark.gpu
def test_lookahead_stop_and_preemption_in_bfloat16_with_graphs_of_twelve(tmp_path):
    """Twelve requests in bfloat16 with captured decode steps of up to twelve rows, a pool so small
    that requests are preempted and recomputed, one request that ends on a stop token: with and
    without lookahead the tokens are the same, and along every request's own sequence each token
    is the plain implementation's best wherever that one leads clearly."""
    doc, seed = helpers.TINY["B"]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    prompts = [helpers.random_prompt(n, doc["vocab_size"], 90 + n) for n in (3, 21, 50, 9, 33, 17, 5, 40, 12, 28, 7, 45)]

    def run(lookahead, stop):
        params = [SamplingParams(temperature=0.0, max_new_tokens=14 if i else 20, stop_token_ids=stop if i == 0 else ())
                  for i in range(len(prompts))]
        llm = LLM(str(tmp_path), dtype="bfloat16", ctx=128, page_size=16, kv_cache_tokens=448, allow_small_pool=True,
                  max_num_seqs=12, max_num_batched_tokens=48, prefill_chunk=19, lookahead=lookahead, device="cuda:0")
        outs = llm.generate(prompts, params)
        llm.engine.cache.check()
        assert not llm.has_unfinished() and llm.engine.cache.slots.free_slots == 12
        return outs, llm

    free_run, _ = run(False, ())
    first = free_run[0].token_ids
    cut = next((i for i in range(3, len(first)) if first[i] not in first[:i]), None)
    assert cut is not None, "the tiny model repeats itself too early for this test"
    stop = (first[cut],)
    waited, llm_waited = run(False, stop)
    ahead, llm_ahead = run(True, stop)
    assert llm_waited.scheduler.stats["preempted"] > 0 and llm_ahead.scheduler.stats["preempted"] > 0
    assert llm_ahead.engine.graphs is not None and max(llm_ahead.engine.graphs._graphs) >= 8
    assert [(o.token_ids, o.finish_reason) for o in waited] == [(o.token_ids, o.finish_reason) for o in ahead]
    assert ahead[0].finish_reason == "stop" and ahead[0].token_ids == first[:cut]
    checked = 0
    for prompt, out in zip(prompts, ahead):
        logits = plain_lfm2.plain_forward(doc, tensors, prompt + out.token_ids[:-1])[len(prompt) - 1:] if len(out.token_ids) > 1 else \
            plain_lfm2.plain_forward(doc, tensors, prompt)[len(prompt) - 1:]
        top2 = logits.topk(2, dim=-1)
        clear = (top2.values[:, 0] - top2.values[:, 1]) > 0.2 * logits.std()
        picked = torch.tensor(out.token_ids)
        assert (picked[clear] == top2.indices[clear, 0]).all(), (out.token_ids, top2.indices[:, 0].tolist())
        checked += int(clear.sum())
    assert checked >= 40


def test_the_steps_block_goes_by_the_kernel_table_when_it_offers_a_way(tmp_path):
    """``StepBuilder`` hands its block to ``ops.words_from_host`` when the kernel table has one and
    the block is small; a table that declines, a large block and a table without the entry leave
    it to the copy.  Either way the step's arrays on the device are those of the staging block."""
    from shiso_llm_b200.engine.batch import StepBuilder

    doc, seed = helpers.TINY["A"]
    helpers.make_folder(tmp_path, doc, seed)
    engine = helpers.make_engine(tmp_path, "float32", ops=fake_kernels, page_size=4, kv_cache_tokens=256, ctx=64,
                                 max_num_seqs=4, max_num_batched_tokens=64)

    class Table:
        def __init__(self, accept):
            self.accept, self.calls = accept, []

        def words_from_host(self, host, dst):
            self.calls.append(dst.numel())
            if self.accept:
                dst.copy_(host[: dst.numel()])
            return self.accept

    tokens = [7, 8, 9, 10, 11]
    seen = []
    for number, table in enumerate((Table(True), Table(False), None)):
        builder = StepBuilder(engine.cache, "cpu", 64, 4)
        builder.ops = table
        request = f"r{number}"
        start = engine.cache.append(request, len(tokens))
        meta = builder.build([StepEntry(request, tokens, [4])], [start])
        assert meta.token_ids.tolist() == tokens and meta.positions.tolist() == [0, 1, 2, 3, 4]
        engine.cache.cancel(request)
        engine.cache.release(request)
        seen.append(table.calls if table is not None else None)
    assert len(seen[0]) == 1 and len(seen[1]) == 1 and seen[0] == seen[1] and seen[2] is None
    big = StepBuilder(engine.cache, "cpu", 64, 4)
    big.KERNEL_COPY_MAX_WORDS = 4  # every block is a large one now
    big.ops = Table(True)
    start = engine.cache.append("large", len(tokens))
    meta = big.build([StepEntry("large", tokens, [4])], [start])
    assert meta.token_ids.tolist() == tokens and big.ops.calls == []
    engine.cache.cancel("large")
    engine.cache.release("large")
    engine.cache.check()
