"""The Python entry point: ``LLM(model_dir).generate(prompts, SamplingParams(...))``.

The reference's in-process entry is ``Runtime::generate_blocking(Request) -> Response``
(crates/shiso-runtime/src/runtime.rs:413; README.md:225-272) over token ids prepared by
its tokenizer; this engine takes and returns token ids.  Option names follow the
reference's serve options where it has them (crates/shiso-runtime/src/options.rs:75-320):
``ctx``, ``max_num_seqs``, ``kv_cache_tokens``, ``max_num_batched_tokens``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Union

import torch

from .engine.batch import StepEntry
from .engine.core import Engine, EngineOptions
from .engine.scheduler import Scheduler, SchedulerConfig, StepPlan
from .sampling.device import DeviceSampler
from .sampling.params import SamplingParams


@dataclass
class Output:
    request_id: object
    prompt_token_ids: list
    token_ids: list
    finish_reason: str  # "stop", "length", "abort" or "error"
    error: Optional[str] = None
    preemptions: int = 0


class LLM:
    def __init__(
        self,
        model: Union[str, Engine],
        dtype: str = "bfloat16",
        ctx: int = 4096,
        page_size: int = 16,
        kv_cache_tokens: Optional[int] = None,
        gpu_memory_utilization: Optional[float] = None,
        max_num_seqs: int = 4,
        max_num_batched_tokens: int = 2048,
        prefill_chunk: Optional[int] = None,
        on_exhaustion: str = "preempt",
        cuda_graphs: bool = True,
        device: str = "cuda:0",
        ops=None,
        lookahead: bool = True,
        allow_small_pool: bool = False,
        dump_layers: int = 0,
    ):
        """``model`` is a model folder (config.json + *.safetensors), or an ``Engine`` that is
        already built (then the engine's own options stand for dtype and cache sizes).

        With ``lookahead`` a step is planned and launched while the tokens of the step before
        it are still on their way to the host: a decoding request's next row takes its token
        on the device, and the host reads each step's tokens one step late.  The tokens are the
        same; a request that ends on a stop token has one more row computed, which is dropped."""
        if isinstance(model, Engine):
            self.engine = model
            opts = model.options
            ctx, max_num_seqs = opts.ctx, opts.max_num_seqs
            max_num_batched_tokens = opts.max_num_batched_tokens
        else:
            options = EngineOptions(
                dtype=dtype, ctx=ctx, page_size=page_size, kv_cache_tokens=kv_cache_tokens,
                gpu_memory_utilization=gpu_memory_utilization,
                max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens, device=device,
                cuda_graphs=cuda_graphs, allow_small_pool=allow_small_pool, dump_layers=dump_layers,
            )
            self.engine = Engine.from_folder(model, options, ops)
        self.scheduler = Scheduler(
            self.engine.cache,
            SchedulerConfig(
                max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                prefill_chunk=prefill_chunk, ctx=ctx, on_exhaustion=on_exhaustion,
                portion_multiple=self.engine.model.plan.portion_multiple,
            ),
            self.engine.model.plan.eos_token_ids,
        )
        self.sampler = DeviceSampler(self.engine.env.ops, self.engine.device)
        self._next_id = 0
        self.lookahead = bool(lookahead)
        self._in_flight = None  # (plan, host buffer, count, event) of the step whose tokens are on their way
        self._turn = 0
        pin = self.engine.device.type == "cuda"
        rows = self.engine.fed_tokens.shape[0]  # one entry per sequence and one for the status word
        self._host_picks = [torch.zeros(rows, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        # Kernels whose waits are bounded report a wait that ran out through a status word on the
        # device.  The picking kernel of every step puts it behind the picks, so it reaches the
        # host with the tokens; plans launched since the word was last seen clean wait here.
        self._carries_status = bool(getattr(self.engine.env.ops, "CARRIES_STATUS", False))
        self._unverified: list = []
        # A diagnostic: called as ``logits_tap(plan, logits)`` with every step's logits (one row per
        # sampling entry of the plan, in order) before a token is picked from them.
        self.logits_tap = None

    # ------------------------------------------------------------------ low level

    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, request_id=None, extras=None):
        """``extras``: values of the model's further per-row inputs (``ModelPlan.row_inputs``) for
        the prompt, name -> one int per token; tokens the request produces get their position."""
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        vocab = self.engine.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"a prompt token lies outside the vocabulary of {vocab}")
        unknown = set(extras or ()) - set(self.engine.model.plan.row_inputs)
        if unknown:
            raise ValueError(f"the model reads no per-row input named {sorted(unknown)}")
        return self.scheduler.add(request_id, prompt, params or SamplingParams(), extras)

    def abort(self, request_id) -> bool:
        return self.scheduler.abort(request_id)

    def __del__(self):
        # A step still on its way stores its tokens into this object's pinned buffers: they go
        # back to the allocator only after it has.
        launched = getattr(self, "_in_flight", None)
        if launched is not None and launched[3] is not None:
            try:
                launched[3].synchronize()
            except Exception:
                pass

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or self._in_flight is not None

    def step(self) -> list:
        """One scheduler decision and one engine step; returns the outputs that finished.

        A step that cannot be launched (an exception from the engine) ends its own requests with
        ``finish_reason = "error"`` and leaves the others as they were, as the reference does
        with a failed pass (crates/shiso-runtime/src/scheduler/mod.rs:1918-1927).  So does a
        step of which a kernel gave up on a bounded wait: the host learns of that when the
        step's tokens arrive."""
        plan: StepPlan = self.scheduler.plan()
        launched = None
        if plan.entries:
            entries, params, positions = [], [], []
            for e in plan.entries:
                if e.feed is not None:
                    tokens = [0]  # a placeholder: the device reads the token a sampler left it
                else:
                    tokens = e.request.token_slice(e.start, e.count)
                entries.append(StepEntry(e.request.id, tokens, [e.count - 1] if e.samples else [], e.feed,
                                         e.request.extras_slice(e.start, e.count)))
                if e.samples:
                    params.append(e.request.params)
                    positions.append(e.start + e.count)
            try:
                launched = self._launch(plan, entries, params, positions)
            except Exception as error:  # the step's requests fail; the engine took nothing for them
                self.scheduler.fail_step(plan, f"the step could not run: {type(error).__name__}: {error}")
                plan = StepPlan(preempted=plan.preempted, failed=plan.failed)
        self.scheduler.launched(plan)
        if self.lookahead:
            self._collect(self._in_flight)
            self._in_flight = launched
        else:
            self._collect(launched)
        return [self._output(r) for r in self.scheduler.take_finished()]

    def _launch(self, plan, entries, params, positions):
        logits = self.engine.step(entries)
        if self._carries_status:
            self._unverified.append(plan)
        if logits is None:
            return (plan, None, 0, None)
        count = logits.shape[0]
        if self.logits_tap is not None:
            self.logits_tap(plan, logits)
        picks = self.engine.fed_tokens[:count]
        carried = count + 1 if self._carries_status else count
        if self._carries_status:
            self.sampler.sample_into(logits, params, positions, picks, self.engine.fed_tokens[count:carried])
        else:
            self.sampler.sample_into(logits, params, positions, picks)
        host = self._host_picks[self._turn]
        self._turn ^= 1
        to_host = getattr(self.engine.env.ops, "words_to_host", None) if picks.is_cuda else None
        if to_host is None or not to_host(self.engine.fed_tokens[:carried], host):
            host[:carried].copy_(self.engine.fed_tokens[:carried], non_blocking=True)
        event = None
        if picks.is_cuda:
            event = torch.cuda.Event()
            event.record()
        return (plan, host, count, event)

    def drain(self) -> list:
        """Waits for the step that is still on its way (lookahead), so that every token the
        device has picked is known to the host; returns the outputs that finished with it."""
        self._collect(self._in_flight)
        self._in_flight = None
        return [self._output(r) for r in self.scheduler.take_finished()]

    def _collect(self, launched) -> None:
        """Waits for a launched step's tokens and hands them to the scheduler.  If the status
        word that came with them says a kernel gave up, every step launched since the word was
        last seen clean is failed instead: its requests end with an error."""
        if launched is None:
            return
        plan, host, count, event = launched
        if event is not None:
            event.synchronize()
        sampled = host[:count].tolist() if count else []
        if count and self._carries_status:
            at = next((i for i, p in enumerate(self._unverified) if p is plan), None)
            covered = [plan] if at is None else self._unverified[: at + 1]
            if at is not None:
                del self._unverified[: at + 1]
            if int(host[count]) != 0:
                why = getattr(self.engine.env.ops, "GAVE_UP", "a kernel gave up on a bounded wait")
                for suspect in covered:
                    self.scheduler.fail_step(suspect, why)
        self.scheduler.arrived(plan, sampled)

    @staticmethod
    def _output(req) -> Output:
        return Output(req.id, list(req.prompt), list(req.output), req.finish_reason, req.error, req.preemptions)

    # ------------------------------------------------------------------ the usual call

    def generate(
        self,
        prompts: Sequence[Sequence[int]],
        sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
    ) -> list:
        """Token ids in, token ids out; one ``Output`` per prompt, in the prompts' order."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError(f"{len(sampling_params)} sampling parameter sets for {len(prompts)} prompts")
        ids = [self.add_request(p, sp).id for p, sp in zip(prompts, sampling_params)]
        results = {}
        for out in [self._output(r) for r in self.scheduler.take_finished()]:
            results[out.request_id] = out
        while self.has_unfinished():
            for out in self.step():
                results[out.request_id] = out
        return [results[i] for i in ids]
