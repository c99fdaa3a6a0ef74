"""The scheduler's decisions, on the host, over a real cache manager (CPU tensors) and no model."""

import pytest
import torch

from shiso_llm_b200.cache import CacheManager
from shiso_llm_b200.engine.scheduler import FINISHED, RUNNING, WAITING, Scheduler, SchedulerConfig
from shiso_llm_b200.parts import FixedState, PagedKV
from shiso_llm_b200.sampling import SamplingParams


def make(num_pages=16, page=4, slots=4, eos=(), **cfg):
    cache = CacheManager([PagedKV(1, 16), FixedState((2, 4))], page, num_pages, slots, torch.float32, "cpu")
    config = SchedulerConfig(**{"max_num_seqs": slots, "max_num_batched_tokens": 16, "ctx": 64, **cfg})
    return Scheduler(cache, config, eos), cache


def run_plan(s, cache, plan, token=7):
    """Does what the engine does with a plan: claim, commit, hand back sampled tokens."""
    for e in plan.entries:
        assert cache.append(e.request.id, e.count) == e.start
    for e in plan.entries:
        cache.commit(e.request.id)
    done = s.step_done(plan, [token] * sum(e.samples for e in plan.entries))
    cache.check()
    return done


def test_budget_cuts_prompts_and_decodes_go_first():
    s, cache = make(num_pages=32, max_num_batched_tokens=16, prefill_chunk=10)
    a = s.add("a", list(range(25)), SamplingParams(max_new_tokens=4))
    b = s.add("b", list(range(6)), SamplingParams(max_new_tokens=4))
    p = s.plan()
    assert [(e.request.id, e.start, e.count, e.samples) for e in p.entries] == [("a", 0, 10, False), ("b", 0, 6, True)]
    run_plan(s, cache, p)
    assert b.output == [7] and b.decoding and not a.decoding
    p = s.plan()  # b's decode row first, then a's next portion within the budget and the chunk
    assert [(e.request.id, e.start, e.count, e.samples) for e in p.entries] == [("b", 6, 1, True), ("a", 10, 10, False)]
    run_plan(s, cache, p)
    p = s.plan()
    assert [(e.request.id, e.count, e.samples) for e in p.entries] == [("b", 1, True), ("a", 5, True)]
    run_plan(s, cache, p)
    assert a.decoding and a.output == [7]
    assert s.stats["prefill_tokens"] == 31 and s.stats["decode_tokens"] == 2


def test_admission_respects_sequence_and_slot_limits_in_arrival_order():
    s, cache = make(num_pages=64, slots=2, max_num_batched_tokens=64)
    for name in "abc":
        s.add(name, [1, 2, 3], SamplingParams(max_new_tokens=2))
    p = s.plan()
    assert [e.request.id for e in p.entries] == ["a", "b"] and len(s.waiting) == 1
    run_plan(s, cache, p)
    run_plan(s, cache, s.plan())  # second token: a and b reach their budget
    assert {r.id for r in s.take_finished()} == {"a", "b"} and cache.slots.free_slots == 2
    p = s.plan()
    assert [e.request.id for e in p.entries] == ["c"]


def test_finish_reasons_and_freeing():
    s, cache = make(eos=(9,))
    a = s.add("a", [1, 2], SamplingParams(max_new_tokens=3))
    b = s.add("b", [1, 2], SamplingParams(max_new_tokens=3, stop_token_ids=(5,)))
    c = s.add("c", [1, 2], SamplingParams(max_new_tokens=3, ignore_eos=True))
    run_plan(s, cache, s.plan(), token=9)  # eos: a stops, b stops, c ignores it
    assert (a.finish_reason, a.output) == ("stop", []) and b.finish_reason == "stop" and c.output == [9]
    assert not cache.has("a") and not cache.has("b") and cache.has("c")
    run_plan(s, cache, s.plan(), token=5)
    run_plan(s, cache, s.plan(), token=5)
    assert (c.finish_reason, c.output) == ("length", [9, 5, 5]) and not cache.has("c")
    assert cache.free_pages() == [16] and cache.slots.free_slots == 4 and not s.has_work()


def test_refusals_up_front():
    s, cache = make(num_pages=4)
    assert s.add("empty", [], SamplingParams()).finish_reason == "error"
    assert "context" in s.add("long", list(range(64)), SamplingParams()).error
    assert "pool" in s.add("wide", list(range(20)), SamplingParams()).error
    assert s.add("zero", [1], SamplingParams(max_new_tokens=0)).finish_reason == "length"
    assert not s.has_work() and len(s.take_finished()) == 4


def test_context_limit_caps_the_budget():
    s, cache = make(num_pages=32, ctx=8, max_num_batched_tokens=8)
    a = s.add("a", [1] * 6, SamplingParams(max_new_tokens=100))
    assert a.budget == 2
    while s.has_work():
        run_plan(s, cache, s.plan())
    assert a.finish_reason == "length" and len(a.output) == 2


def fill_to_exhaustion(policy):
    s, cache = make(num_pages=4, page=4, slots=3, max_num_batched_tokens=16, on_exhaustion=policy)
    a = s.add("a", [1] * 7, SamplingParams(max_new_tokens=20))
    b = s.add("b", [1] * 7, SamplingParams(max_new_tokens=20))
    run_plan(s, cache, s.plan())  # both prompts: 2 pages each, pool full
    assert cache.free_pages() == [0]
    run_plan(s, cache, s.plan())  # position 7 still fits page 1 of each
    return s, cache, a, b


def test_pages_run_out_preempt_the_youngest_and_recompute():
    s, cache, a, b = fill_to_exhaustion("preempt")
    p = s.plan()  # position 8 needs a third page: b (younger) gives way to a
    assert [r.id for r in p.preempted] == ["b"] and [e.request.id for e in p.entries] == ["a"]
    assert b.state == WAITING and b.computed == 0 and b.preemptions == 1 and not cache.has("b")
    assert list(s.waiting)[0] is b and b.output == [7, 7]
    run_plan(s, cache, p)
    # b comes back only when pages for all it has so far are free, reads its prompt and its
    # own output again in one portion, and continues from there
    while True:
        p = s.plan()
        mine = [e for e in p.entries if e.request is b]
        if mine:
            break
        assert not cache.has("b")
        run_plan(s, cache, p)
    assert mine[0].start == 0 and mine[0].count == 9 and mine[0].samples and b.preemptions == 1
    run_plan(s, cache, p)
    assert b.output == [7, 7, 7]
    cache.check()


def test_pages_run_out_fail_policy_fails_the_one_that_cannot_grow():
    s, cache, a, b = fill_to_exhaustion("fail")
    p = s.plan()
    assert [r.id for r in p.failed] == ["a"] and a.finish_reason == "error" and "kv pool" in a.error
    assert not cache.has("a") and [e.request.id for e in p.entries] == ["b"]  # a's pages let b go on
    run_plan(s, cache, p)
    cache.check()


def test_a_lone_request_that_cannot_grow_fails_in_both_modes():
    for policy in ("preempt", "fail"):
        s, cache = make(num_pages=2, page=4, slots=2, max_num_batched_tokens=16, on_exhaustion=policy)
        a = s.add("a", [1] * 8, SamplingParams(max_new_tokens=5))
        run_plan(s, cache, s.plan())
        p = s.plan()
        assert a.finish_reason == "error" and p.failed == [a] and not p.entries
        assert cache.free_pages() == [2] and not s.has_work()


def test_portion_shrinks_to_the_free_pages_and_admission_waits_for_room():
    s, cache = make(num_pages=6, page=4, slots=3, max_num_batched_tokens=8)
    a = s.add("a", [1] * 16, SamplingParams(max_new_tokens=2))
    b = s.add("b", [1] * 8, SamplingParams(max_new_tokens=2))
    p = s.plan()  # a's first portion fills the budget
    assert [(e.request.id, e.count) for e in p.entries] == [("a", 8)]
    run_plan(s, cache, p)
    cache.append("other", 12)  # somebody else takes three pages: one is left
    cache.commit("other")
    p = s.plan()  # a wants 8 more tokens but only one page is free; b needs two and waits
    assert [(e.request.id, e.count, e.samples) for e in p.entries] == [("a", 4, False)] and len(s.waiting) == 1
    run_plan(s, cache, p)
    cache.release("other")
    p = s.plan()
    assert [(e.request.id, e.count, e.samples) for e in p.entries] == [("a", 4, True), ("b", 4, False)]
    run_plan(s, cache, p)
    cache.check()


def test_abort_frees_everything_mid_prompt():
    s, cache = make(max_num_batched_tokens=4)
    a = s.add("a", [1] * 10, SamplingParams())
    s.add("b", [1] * 3, SamplingParams())
    run_plan(s, cache, s.plan())
    assert cache.has("a") and s.abort("a") and a.finish_reason == "abort" and not cache.has("a")
    assert s.abort("b") and not s.abort("nobody") and not s.has_work()
    assert cache.free_pages() == [16] and cache.slots.free_slots == 4


def test_invariant_prefilling_or_standing_on_a_token():
    s, cache = make(num_pages=64, max_num_batched_tokens=5)
    reqs = [s.add(i, [1] * n, SamplingParams(max_new_tokens=3)) for i, n in enumerate((9, 2, 6, 4))]
    while s.has_work():
        p = s.plan()
        assert p.num_tokens <= 5 and len({e.request.id for e in p.entries}) == len(p.entries)
        run_plan(s, cache, p)
        for r in s.running:
            assert r.remaining >= 1 and (r.decoding or r.remaining >= 1)
    assert all(r.finish_reason == "length" and len(r.output) == 3 for r in reqs)


# --------------------------------------------------------------------------- tokens that arrive a step late


def drive_late(s, cache, token_of, max_steps=200):
    """The lookahead loop without a model: each step's tokens arrive after the next step was
    planned and launched.  ``token_of(request, output_index)`` is the token the "model" picks.
    Returns the plans, in order."""
    plans, in_flight = [], None
    for _ in range(max_steps):
        if not s.has_work() and in_flight is None:
            break
        plan = s.plan()
        for e in plan.entries:
            assert cache.append(e.request.id, e.count) == e.start
        for e in plan.entries:
            cache.commit(e.request.id)
        s.launched(plan)
        tokens = [token_of(e.request, e.output_index) for e in plan.entries if e.samples]
        if in_flight is not None:
            s.arrived(*in_flight)
        in_flight = (plan, tokens) if plan.entries else None
        cache.check()
        plans.append(plan)
    assert not s.has_work()
    return plans


def test_late_tokens_give_the_same_outputs_as_waiting_for_each_step():
    def pick(req, idx):
        return 100 + 10 * req.id + idx

    outputs = []
    for late in (False, True):
        s, cache = make(num_pages=64, max_num_batched_tokens=6, prefill_chunk=4)
        reqs = [s.add(i, [1] * n, SamplingParams(max_new_tokens=m)) for i, (n, m) in enumerate([(9, 5), (2, 1), (6, 3), (4, 7)])]
        if late:
            plans = drive_late(s, cache, pick)
            # a request standing on a token the host has not seen is planned again, fed from the device
            assert any(e.feed is not None for p in plans for e in p.entries)
        else:
            while s.has_work():
                p = s.plan()
                for e in p.entries:
                    cache.append(e.request.id, e.count)
                    cache.commit(e.request.id)
                s.launched(p)
                s.arrived(p, [pick(e.request, e.output_index) for e in p.entries if e.samples])
        outputs.append([(r.output, r.finish_reason) for r in reqs])
        assert cache.free_pages() == [64] and cache.slots.free_slots == 4
    assert outputs[0] == outputs[1]
    assert [len(o) for o, _ in outputs[0]] == [5, 1, 3, 7] and all(why == "length" for _, why in outputs[0])


def test_a_stop_token_that_arrives_late_drops_the_row_computed_past_it():
    s, cache = make(num_pages=32, eos=(9,))
    a = s.add("a", [1] * 5, SamplingParams(max_new_tokens=10))
    b = s.add("b", [1] * 3, SamplingParams(max_new_tokens=10, ignore_eos=True))

    def pick(req, idx):
        return 9 if idx == 2 else 50 + idx  # the third token is the stop token

    plans = drive_late(s, cache, pick)
    assert a.finish_reason == "stop" and a.output == [50, 51]
    assert b.finish_reason == "length" and b.output == [50, 51, 9] + [50 + i for i in range(3, 10)]
    # "a" was planned once more before its stop token was known
    rows_a = [e for p in plans for e in p.entries if e.request is a]
    assert len(rows_a) == 1 + 3  # the prompt, two decode rows, and the one past the stop
    assert cache.free_pages() == [32] and cache.slots.free_slots == 4 and not s.running and not s.waiting


def test_preemption_and_abort_while_a_token_is_on_its_way():
    """With 6 pages of 4, two requests of 8 tokens each outgrow the pool while decoding: the
    younger is preempted standing on a token the host has not seen, takes it when it arrives,
    and recomputes with it; an abort in the same situation frees everything at once."""
    s, cache = make(num_pages=6, page=4, max_num_batched_tokens=16)
    a = s.add("a", [1] * 8, SamplingParams(max_new_tokens=8))
    b = s.add("b", [2] * 8, SamplingParams(max_new_tokens=8))
    drive_late(s, cache, lambda req, idx: 30 + idx)
    assert a.output == b.output == [30 + i for i in range(8)]
    assert s.stats["preempted"] > 0 and b.preemptions > 0
    assert cache.free_pages() == [6] and cache.slots.free_slots == 4

    s, cache = make(num_pages=16)
    c = s.add("c", [1] * 4, SamplingParams(max_new_tokens=8))
    p1 = s.plan()
    for e in p1.entries:
        cache.append(e.request.id, e.count)
        cache.commit(e.request.id)
    s.launched(p1)
    assert c.output == [-1] and c.decoding
    assert s.abort("c") and cache.free_pages() == [16]
    assert s.arrived(p1, [5]) == [] and c.finish_reason == "abort" and not s.has_work()
