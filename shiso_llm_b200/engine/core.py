"""The engine: a model, its cache and ONE step function.

``Engine.step(entries)`` takes a batch of (request, its next tokens, wanted places) -
portions of prompts beside single decoded tokens, cut anywhere - claims cache room,
uploads the step's metadata, runs only the tokens it was given as one batch over the
cache earlier steps left, and returns float32 logits at the wanted places, in the
order of the entries and of their ``want`` lists.

The reference has three entry points that are never mixed (``prefill_chunk``,
``prefill_last``, ``decode_batch``: crates/shiso-core/src/model.rs:321-351); its
nearest precedent for one mixed pass is ``PassRows::Segments``
(crates/shiso-engine/src/layers.rs:1735-1766).  The order inside a step follows its
correctness argument (crates/shiso-engine/src/stack.rs:1018-1033): claim pages for
every member, then write inputs and block tables, then launch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..config.registry import Architecture, load_config
from ..parts.base import BuildEnv
from ..parts.model import Model
from ..weights.loader import load_weights
from .batch import StepBuilder, StepEntry

_DTYPES = {
    "bfloat16": torch.bfloat16,
    "bf16": torch.bfloat16,
    "float32": torch.float32,
    "fp32": torch.float32,
}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype {name}: expected bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"compute dtype {name!r}: expected bfloat16 or float32") from None


@dataclass
class EngineOptions:
    """Sizes of the engine's buffers.  Names follow the reference's serve options where it
    has them (crates/shiso-runtime/src/options.rs:75-320): ``ctx``, ``max_num_seqs``,
    ``kv_cache_tokens``, ``max_num_batched_tokens``."""

    dtype: object = "bfloat16"
    ctx: int = 4096
    page_size: int = 16
    kv_cache_tokens: Optional[int] = None  # pool size in tokens; default: max_num_seqs * ctx
    max_num_seqs: int = 4
    max_num_batched_tokens: int = 2048
    device: str = "cuda:0"
    cuda_graphs: bool = True  # replay captured graphs for steps of single decoded tokens

    def num_pages(self) -> int:
        tokens = self.kv_cache_tokens if self.kv_cache_tokens is not None else self.max_num_seqs * self.ctx
        return max(1, -(-tokens // self.page_size))


def default_ops():
    """The CUDA kernel table.  Importing it loads (and if needed builds) the extension and
    fails loudly when that is impossible; there is no fallback."""
    from ..kernels import ops

    ops.require()
    return ops


class Engine:
    def __init__(self, model: Model, cache: CacheManager, options: EngineOptions):
        self.model = model
        self.cache = cache
        self.options = options
        self.env = model.env
        self.device = model.env.device
        self.vocab_size = model.plan.vocab_size
        self.builder = StepBuilder(
            cache, self.device, options.max_num_batched_tokens, options.max_num_seqs
        )
        # Tokens picked on the device from the last step's logits, one per sampling row; an entry
        # with ``feed = j`` takes its token from index j without the host having seen it.
        self.fed_tokens = torch.zeros(max(1, options.max_num_seqs), dtype=torch.int32, device=self.device)
        self.builder.fed_tokens = self.fed_tokens
        self.steps_run = 0
        self.graphs = None
        if options.cuda_graphs and self.device.type == "cuda" and model.graph_safe:
            from .graphs import DecodeGraphs

            decode_builder = StepBuilder(
                cache, self.device, options.max_num_seqs, options.max_num_seqs, fixed_table_width=cache.max_blocks
            )
            decode_builder.fed_tokens = self.fed_tokens
            self.graphs = DecodeGraphs(model, cache, decode_builder)

    def warm_up(self) -> None:
        """Runs a two-token request through a prompt step and a decode step and drops it, so
        that every kernel has been loaded before the first graph capture."""
        probe = ("__warm_up__",)
        graphs, self.graphs = self.graphs, None
        try:
            self.step([StepEntry(probe, [0], [])])
            self.step([StepEntry(probe, [0], [0])])
        finally:
            self.graphs = graphs
            if self.cache.has(probe):
                self.finish(probe)
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_plan(cls, plan, tensors_or_dir, options: EngineOptions, ops=None) -> "Engine":
        dtype = parse_dtype(options.dtype)
        device = torch.device(options.device)
        env = BuildEnv(dtype=dtype, device=device, ops=ops if ops is not None else default_ops())
        model = Model(plan, env)
        specs = model.tensor_specs()
        if isinstance(tensors_or_dir, str):
            tensors = load_weights(tensors_or_dir, specs, dtype, device)
        else:
            tensors = tensors_or_dir
        model.bind(tensors)
        blocks_per_request = -(-options.ctx // options.page_size)
        num_pages = options.num_pages()
        cache = CacheManager(
            model.cache_needs(),
            options.page_size,
            num_pages,
            options.max_num_seqs,
            dtype,
            device,
            max_blocks_per_request=min(blocks_per_request, num_pages),
        )
        engine = cls(model, cache, options)
        if engine.graphs is not None:
            engine.warm_up()
        return engine

    @classmethod
    def from_folder(cls, model_dir: str, options: EngineOptions, ops=None) -> "Engine":
        """A model folder (config.json + *.safetensors); the class comes from config.json."""
        arch, config = load_config(model_dir)
        engine = cls.from_plan(arch.build_plan(config), model_dir, options, ops)
        engine.architecture = arch
        engine.config = config
        return engine

    # ------------------------------------------------------------------ the step

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs one batch; returns float32 logits ``[wanted, vocab]`` on the device, or
        None when nothing was wanted.  Raises ``OutOfPages`` (nothing claimed, nothing
        run) when the cache cannot hold the step."""
        entries = list(entries)
        seen = set()
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request!r}: a step brings at least one token")
            if min(e.tokens) < 0 or max(e.tokens) >= self.vocab_size:
                raise ValueError(f"request {e.request!r}: a token id lies outside the vocabulary of {self.vocab_size}")
            if e.feed is not None and (len(e.tokens) != 1 or not 0 <= e.feed < self.fed_tokens.shape[0]):
                raise ValueError(f"request {e.request!r}: a fed token is one token from index 0..{self.fed_tokens.shape[0] - 1}")
        # Admission check for the whole step before anything is claimed.
        self._check_room(entries)
        starts = []
        claimed = []
        try:
            for e in entries:
                starts.append(self.cache.append(e.request, len(e.tokens)))
                claimed.append(e.request)
            if (
                self.graphs is not None
                and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
            ):
                logits = self.graphs.run(entries, starts)
            else:
                meta = self.builder.build(entries, starts)
                logits = self.model.forward(meta, self.cache)
        except BaseException:
            for request in claimed:
                self.cache.cancel(request)
            raise
        for e in entries:
            self.cache.commit(e.request)
        self.steps_run += 1
        return logits

    def _check_room(self, entries) -> None:
        from ..cache.pages import OutOfPages

        need = [0] * len(self.cache.groups)
        new_requests = 0
        for e in entries:
            if not self.cache.has(e.request):
                new_requests += 1
            for g, n in enumerate(self.cache.pages_needed(e.request, len(e.tokens))):
                need[g] += n
        if new_requests > self.cache.slots.free_slots:
            raise OutOfPages(new_requests, self.cache.slots.free_slots, "state slots")
        for g, group in enumerate(self.cache.groups):
            if need[g] > group.pool.free_pages:
                raise OutOfPages(need[g], group.pool.free_pages)

    def finish(self, request) -> None:
        """The request is over: its pages and its state slot go back to the pools."""
        self.cache.release(request)
