"""What a request sees when a step fails, when a kernel gives up, when options are refused.

No GPU is ever faulted or hung here: a step is made to fail by a kernel-table entry that raises
on the host before anything is launched, and a bounded wait is made to run out by the library's
own self-test kernel (one CTA that waits a few thousand cycles on a barrier nobody arrives at,
then sets the status word and returns).
"""

import types

import pytest
import torch

import fake_kernels
import helpers
import plain_lfm2
from shiso_llm_b200 import LLM, SamplingParams
from shiso_llm_b200.config.errors import InvalidValue
from shiso_llm_b200.engine import EngineOptions, StepEntry
from shiso_llm_b200.engine.core import pool_pages_for_share
from test_engine import BACKENDS, backend_args


def failing_table(base, fail_on_call):
    """The kernel table ``base`` with an ``embed`` (the first launch of every step) that raises
    at its n-th call."""
    table = types.SimpleNamespace(**{k: getattr(base, k) for k in dir(base) if not k.startswith("__")})
    calls = {"n": 0}

    def embed(*args, **kwargs):
        calls["n"] += 1
        if calls["n"] == fail_on_call:
            raise RuntimeError("injected: the launch was refused")
        return base.embed(*args, **kwargs)

    table.embed = embed
    table.calls = calls
    return table


@pytest.mark.parametrize("lookahead", [False, True])
def test_a_step_that_fails_ends_only_its_own_requests(tmp_path, lookahead):
    """Three requests, two of them resident at a time; the second step raises.  The two requests
    of that step end with an error and give back everything; the third, which was waiting, is
    admitted afterwards and produces the tokens it produces when nothing fails
    (crates/shiso-runtime/src/scheduler/mod.rs:1918-1927)."""
    doc, seed = helpers.TINY["A"]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    prompts = [helpers.random_prompt(n, doc["vocab_size"], 70 + n) for n in (9, 14, 6)]
    want = [plain_lfm2.plain_greedy(doc, tensors, p, 6) for p in prompts]
    table = failing_table(fake_kernels, 2)
    llm = LLM(str(tmp_path), dtype="float32", ctx=64, page_size=16, max_num_seqs=2, max_num_batched_tokens=64,
              ops=table, device="cpu", lookahead=lookahead)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=6))
    assert [o.finish_reason for o in outs] == ["error", "error", "length"]
    assert all("injected" in o.error and "could not run" in o.error for o in outs[:2])
    assert all(-1 not in o.token_ids for o in outs)
    assert outs[2].token_ids == want[2]
    llm.engine.cache.check()
    assert llm.engine.cache.slots.free_slots == 2 and llm.engine.cache.free_pages() == [llm.engine.cache.num_pages]
    assert not llm.has_unfinished()
    # the engine goes on: a new request runs to its end
    again = llm.generate([prompts[1]], SamplingParams(temperature=0.0, max_new_tokens=6))
    assert again[0].token_ids == want[1]


@pytest.mark.parametrize("lookahead", [False, True])
def test_a_kernel_that_gave_up_fails_the_steps_it_may_have_touched(tmp_path, lookahead):
    """The status word reaches the host with a step's tokens.  Set during the third step, it ends
    the requests of that step (and of no other step) with an error; later requests run clean."""
    doc, seed = helpers.TINY["B"]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    prompts = [helpers.random_prompt(n, doc["vocab_size"], 80 + n) for n in (5, 11)]
    llm = LLM(str(tmp_path), dtype="float32", ctx=64, page_size=16, max_num_seqs=2, max_num_batched_tokens=32,
              ops=fake_kernels, device="cpu", lookahead=lookahead)
    for p in prompts:
        llm.add_request(p, SamplingParams(temperature=0.0, max_new_tokens=8))
    done = []
    for step in range(40):
        if step == 2:
            fake_kernels.STATUS_WORD[0] = 1
        done += llm.step()
        if not llm.has_unfinished():
            break
    done += llm.drain()
    assert fake_kernels.STATUS_WORD[0] == 0
    assert len(done) == 2 and all(o.finish_reason == "error" and "gave up" in o.error for o in done)
    assert all(-1 not in o.token_ids for o in done)
    llm.engine.cache.check()
    assert llm.engine.cache.slots.free_slots == 2
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
    assert [o.token_ids for o in outs] == [plain_lfm2.plain_greedy(doc, tensors, p, 8) for p in prompts]


@pytest.mark.gpu
def test_a_bounded_wait_that_runs_out_is_seen_and_the_next_step_is_clean(tmp_path):
    """On the GPU: the self-test kernel's wait runs out after 4,000 cycles; the status word is
    set; ``check_kernel_status`` raises once and is clean afterwards; through ``LLM`` the
    requests of the step that carried the word fail, and the same prompts then generate the
    plain implementation's tokens."""
    from shiso_llm_b200.kernels import ops

    ops.require()
    torch.cuda.synchronize()
    ops.check_kernel_status()  # clean to begin with
    ops.selftest_bounded_wait(4000)
    with pytest.raises(ops.KernelError, match="gave up"):
        ops.check_kernel_status()
    ops.check_kernel_status()  # reading cleared it

    doc, seed = helpers.TINY["A"]
    tensors = helpers.make_folder(tmp_path, doc, seed)
    prompts = [helpers.random_prompt(n, doc["vocab_size"], 90 + n) for n in (7, 19)]
    want = [plain_lfm2.plain_greedy(doc, tensors, p, 8) for p in prompts]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(str(tmp_path), dtype=dtype, ctx=64, page_size=16, max_num_seqs=2, max_num_batched_tokens=32)
        for p in prompts:
            llm.add_request(p, SamplingParams(temperature=0.0, max_new_tokens=8))
        done = llm.step() + llm.step()
        ops.selftest_bounded_wait(4000)  # "a kernel of the next step" gives up
        while llm.has_unfinished():
            done += llm.step()
        done += llm.drain()
        assert len(done) == 2 and all(o.finish_reason == "error" and "gave up" in o.error for o in done), done
        llm.engine.cache.check()
        assert llm.engine.cache.slots.free_slots == 2
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
        assert all(o.finish_reason == "length" for o in outs)
        if dtype == "float32":
            assert [o.token_ids for o in outs] == want
        ops.check_kernel_status()


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_refused_step_claims_nothing_for_a_request_it_saw_first(tmp_path, backend):
    """Refusals that are found after room was checked (a wanted place outside the tokens, too
    many tokens, a fed token that is not single) leave a new request unknown to the cache and
    give a known request's pages back, also when the refused tokens would have crossed a page."""
    doc, seed = helpers.TINY["A"]
    helpers.make_folder(tmp_path, doc, seed)
    engine = helpers.make_engine(tmp_path, "float32", page_size=4, kv_cache_tokens=64, ctx=64, max_num_seqs=3,
                                 max_num_batched_tokens=16, **backend_args(backend))
    engine.step([StepEntry("known", [1, 2, 3], [2])])
    before = (engine.cache.free_pages(), engine.cache.slots.free_slots, engine.cache.length("known"))
    bad_steps = [
        [StepEntry("fresh", [1, 2, 3, 4, 5, 6], [6])],  # place outside
        [StepEntry("known", [4, 5, 6, 7, 8], [5])],  # would cross a page edge
        [StepEntry("fresh", [1] * 17, [])],  # more tokens than a step takes
        [StepEntry("fresh", [1, 2], [], feed=0)],  # a fed token is one token
        [StepEntry("known", [9], [0]), StepEntry("fresh", [3, 4], [0]), StepEntry("third", [1], [1])],
    ]
    for entries in bad_steps:
        with pytest.raises(ValueError):
            engine.step(entries)
        assert (engine.cache.free_pages(), engine.cache.slots.free_slots, engine.cache.length("known")) == before
        assert not engine.cache.has("fresh") and not engine.cache.has("third")
        engine.cache.check()
    engine.finish("known")
    assert engine.cache.free_pages() == [16]


def test_pool_sizing_by_share_and_the_refusal_of_a_pool_below_one_context():
    # the arithmetic of crates/shiso-engine/src/options.rs:366-398
    gib = 1 << 30
    pages, left = pool_pages_for_share(0.9, 180 * gib, 170 * gib, page_bytes=196608, state_bytes=64 * 163840, reserve_bytes=gib)
    assert left == int(0.9 * 180 * gib) - 10 * gib - 64 * 163840 - gib and pages == left // 196608
    assert pool_pages_for_share(0.05, 180 * gib, 100 * gib, 196608, 0, 0) == (0, 0)  # the share is spent already
    with pytest.raises(InvalidValue, match="one of the two"):
        EngineOptions(kv_cache_tokens=4096, gpu_memory_utilization=0.5)
    for share in (0.0, -0.1, 1.5):
        with pytest.raises(InvalidValue, match="share"):
            EngineOptions(gpu_memory_utilization=share)
    options = EngineOptions(ctx=4096, page_size=16, kv_cache_tokens=4000)
    with pytest.raises(InvalidValue, match="cannot hold one request of ctx = 4096"):
        options.checked_pages(options.num_pages(), 4000)
    assert EngineOptions(ctx=4096, page_size=16, kv_cache_tokens=4096).checked_pages(256, 4096) == 256
    assert EngineOptions(ctx=4096, page_size=16, kv_cache_tokens=64, allow_small_pool=True).checked_pages(4, 64) == 4


def test_an_engine_refuses_a_pool_smaller_than_one_context_and_sizes_one_by_share(tmp_path, monkeypatch):
    doc, seed = helpers.TINY["A"]
    helpers.make_folder(tmp_path, doc, seed)
    with pytest.raises(InvalidValue, match="cannot hold one request"):
        helpers.make_engine(tmp_path, "float32", ops=fake_kernels, ctx=128, page_size=16, kv_cache_tokens=64)
    engine = helpers.make_engine(tmp_path, "float32", ops=fake_kernels, ctx=128, page_size=16, kv_cache_tokens=64,
                                 allow_small_pool=True)
    assert engine.cache.num_pages == 4 and engine.cache.max_blocks == 4
    # a share of the memory: on the CPU the same arithmetic runs over what the machine reports,
    # here a made-up machine of 1 GiB with 600 MiB free
    import psutil

    mib = 1 << 20
    monkeypatch.setattr(psutil, "virtual_memory", lambda: types.SimpleNamespace(total=1024 * mib, available=600 * mib))
    shared = helpers.make_engine(tmp_path, "float32", ops=fake_kernels, ctx=128, page_size=16, max_num_seqs=2,
                                 max_num_batched_tokens=32, gpu_memory_utilization=0.75)
    page_bytes, state_bytes = shared.cache.costs(shared.model.cache_needs(), 16, torch.float32)
    from shiso_llm_b200.engine.core import step_buffer_bytes

    reserve = step_buffer_bytes(shared.model.plan, shared.options, torch.float32)
    assert shared.cache.num_pages == (768 * mib - 424 * mib - 2 * state_bytes - reserve) // page_bytes >= 8
    with pytest.raises(InvalidValue, match="leaves 0.00 GiB"):
        helpers.make_engine(tmp_path, "float32", ops=fake_kernels, ctx=128, page_size=16, gpu_memory_utilization=0.3)


def test_another_cuda_device_than_the_bound_one_is_refused():
    from shiso_llm_b200.kernels import ops

    assert ops.resolve_binding(None, None, 0) == 0  # a bare "cuda": the current device
    assert ops.resolve_binding(1, None, 0) == 1  # the first engine chooses
    assert ops.resolve_binding(1, 1, 0) == 1
    with pytest.raises(ops.KernelError, match="works on cuda:0"):
        ops.resolve_binding(1, 0, 0)
    with pytest.raises(ops.KernelError, match="works on cuda:2"):
        ops.resolve_binding(None, 2, 0)  # "cuda" means the current device, which is not the bound one
    with pytest.raises(ops.KernelError):
        ops.bind_device(torch.device("cpu"))
