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
        max_num_seqs: int = 4,
        max_num_batched_tokens: int = 2048,
        prefill_chunk: Optional[int] = None,
        on_exhaustion: str = "preempt",
        cuda_graphs: bool = True,
        device: str = "cuda:0",
        ops=None,
    ):
        """``model`` is a model folder (config.json + *.safetensors), or an ``Engine`` that is
        already built (then the engine's own options stand for dtype and cache sizes)."""
        if isinstance(model, Engine):
            self.engine = model
            opts = model.options
            ctx, max_num_seqs = opts.ctx, opts.max_num_seqs
            max_num_batched_tokens = opts.max_num_batched_tokens
        else:
            options = EngineOptions(
                dtype=dtype, ctx=ctx, page_size=page_size, kv_cache_tokens=kv_cache_tokens,
                max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens, device=device,
                cuda_graphs=cuda_graphs,
            )
            self.engine = Engine.from_folder(model, options, ops)
        self.scheduler = Scheduler(
            self.engine.cache,
            SchedulerConfig(
                max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                prefill_chunk=prefill_chunk, ctx=ctx, on_exhaustion=on_exhaustion,
            ),
            self.engine.model.plan.eos_token_ids,
        )
        self.sampler = DeviceSampler(self.engine.env.ops, self.engine.device)
        self._next_id = 0

    # ------------------------------------------------------------------ low level

    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, request_id=None):
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        vocab = self.engine.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"a prompt token lies outside the vocabulary of {vocab}")
        return self.scheduler.add(request_id, prompt, params or SamplingParams())

    def abort(self, request_id) -> bool:
        return self.scheduler.abort(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> list:
        """One scheduler decision and one engine step; returns the outputs that finished."""
        plan: StepPlan = self.scheduler.plan()
        sampled = []
        if plan.entries:
            entries, params, positions = [], [], []
            for e in plan.entries:
                tokens = e.request.token_slice(e.start, e.count)
                entries.append(StepEntry(e.request.id, tokens, [e.count - 1] if e.samples else []))
                if e.samples:
                    params.append(e.request.params)
                    positions.append(e.start + e.count)
            logits = self.engine.step(entries)
            if logits is not None:
                sampled = self.sampler.sample(logits, params, positions)
        self.scheduler.step_done(plan, sampled)
        return [self._output(r) for r in self.scheduler.take_finished()]

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
