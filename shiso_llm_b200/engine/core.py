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

import os
import sys
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..config.errors import InvalidValue
from ..config.registry import Architecture, load_config
from ..parts.base import BuildEnv
from ..parts.model import Model
from ..weights.loader import load_weights
from .batch import StepBuilder, StepEntry
from .graphs import NOT_RUN

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
    ``kv_cache_tokens``, ``gpu_memory_utilization``, ``max_num_batched_tokens``.

    The cache pool is sized in one of two ways, as there (options.rs:180-203): ``kv_cache_tokens``
    names it outright; ``gpu_memory_utilization`` is the share of the device's memory this
    process may fill, and the pool gets what the weights, the step's buffers and the state
    slots leave of it.  With neither the pool holds ``max_num_seqs * ctx`` tokens.  A pool that
    cannot hold one request of ``ctx`` tokens is refused (crates/shiso-engine/src/options.rs:366-398)
    unless ``allow_small_pool`` is set, which is for tests that want pages to run out."""

    dtype: object = "bfloat16"
    ctx: int = 4096
    page_size: int = 16
    kv_cache_tokens: Optional[int] = None  # pool size in tokens
    gpu_memory_utilization: Optional[float] = None  # or: share of device memory, in (0, 1]
    max_num_seqs: int = 4
    max_num_batched_tokens: int = 2048
    device: str = "cuda:0"
    cuda_graphs: bool = True  # replay captured graphs: decode steps by batch size, mixed steps by padded shape
    graph_mixed_steps: bool = True  # with cuda_graphs: also capture steps that hold prompt portions
    allow_small_pool: bool = False
    dump_layers: int = 0  # 1: a line of residual statistics per run entry; 2: per mixer and feed-forward too

    def __post_init__(self):
        if self.kv_cache_tokens is not None and self.gpu_memory_utilization is not None:
            raise InvalidValue("gpu_memory_utilization", self.gpu_memory_utilization,
                               "kv_cache_tokens is given as well; the pool is sized by one of the two")
        if self.gpu_memory_utilization is not None and not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise InvalidValue("gpu_memory_utilization", self.gpu_memory_utilization, "not a share in (0, 1]")
        if self.kv_cache_tokens is not None and self.kv_cache_tokens <= 0:
            raise InvalidValue("kv_cache_tokens", self.kv_cache_tokens, "the pool needs at least one token")
        for key in ("ctx", "page_size", "max_num_seqs", "max_num_batched_tokens"):
            if getattr(self, key) <= 0:
                raise InvalidValue(key, getattr(self, key), "must be positive")

    def pages_per_context(self) -> int:
        return -(-self.ctx // self.page_size)

    def num_pages(self) -> int:
        """Pages of the pool when it is sized in tokens (explicitly or by default)."""
        tokens = self.kv_cache_tokens if self.kv_cache_tokens is not None else self.max_num_seqs * self.ctx
        return max(1, -(-tokens // self.page_size))

    def checked_pages(self, pages: int, how: str) -> int:
        """``pages`` if the pool may be that small, else the refusal, with the numbers."""
        needed = self.pages_per_context()
        if pages < needed and not self.allow_small_pool:
            raise InvalidValue(
                "gpu_memory_utilization" if self.gpu_memory_utilization is not None else "kv_cache_tokens", how,
                f"a pool of {pages} pages of {self.page_size} tokens cannot hold one request of ctx = {self.ctx} "
                f"tokens, which needs {needed}; enlarge the pool or lower ctx",
            )
        return max(1, pages)


def pool_pages_for_share(fraction: float, total_bytes: int, free_bytes: int, page_bytes: int, state_bytes: int,
                         reserve_bytes: int) -> tuple:
    """Pages a pool gets from a share of the device (crates/shiso-engine/src/options.rs:366-398):
    ``fraction * total`` minus what is in use already (weights included, other processes too),
    minus the state slots and a reserve for the step's buffers.  Returns (pages, bytes left)."""
    share = int(fraction * total_bytes)
    in_use = max(0, total_bytes - free_bytes)
    left = max(0, share - in_use - state_bytes - reserve_bytes)
    return left // max(1, page_bytes), left


def default_ops():
    """The CUDA kernel table.  Importing it loads (and if needed builds) the extension and
    fails loudly when that is impossible; there is no fallback."""
    from ..kernels import ops

    ops.require()
    return ops


def step_buffer_bytes(plan, options: EngineOptions, dtype: torch.dtype) -> int:
    """An upper bound of what one step of ``max_num_batched_tokens`` rows allocates beside
    weights and cache: the residual stream (float32, two copies), a few activations as wide as
    the widest product's output, and the logits of one row per sequence."""
    widest = max([plan.hidden_size] + [int(v) for layer in plan.layers for spec in (layer.mixer, layer.feed_forward)
                                       if spec is not None for k, v in spec.params.items()
                                       if k in ("intermediate_size", "hidden_size") and isinstance(v, int)])
    rows = options.max_num_batched_tokens
    activations = rows * (2 * plan.hidden_size * 4 + 6 * 3 * widest * dtype.itemsize)
    logits = 2 * max(options.max_num_seqs, 1) * plan.vocab_size * 4
    return activations + logits + (256 << 20)


class Engine:
    def __init__(self, model: Model, cache: CacheManager, options: EngineOptions):
        self.model = model
        self.cache = cache
        self.options = options
        self.env = model.env
        self.device = model.env.device
        self.vocab_size = model.plan.vocab_size
        row_inputs = model.plan.row_inputs
        self.builder = StepBuilder(
            cache, self.device, options.max_num_batched_tokens, options.max_num_seqs, row_inputs=row_inputs
        )
        # Tokens picked on the device from the last step's logits, one per sampling row; an entry
        # with ``feed = j`` takes its token from index j without the host having seen it.
        # (One more entry at the end: the picking kernel may leave the kernels' status word there.)
        self.fed_tokens = torch.zeros(max(1, options.max_num_seqs) + 1, dtype=torch.int32, device=self.device)
        self.builder.fed_tokens = self.fed_tokens
        self.builder.ops = model.env.ops
        self.steps_run = 0
        self.graphs = None
        self.step_graphs = None
        level = options.dump_layers or int(os.environ.get("SHISO_LAYER_DUMP", "0") or 0)
        self.layer_hook = self.add_hook = None  # diagnostics; a step with a hook is never captured
        self.profiler = None  # kernels.profile.StepProfiler while launches are being timed
        # SHISO_NVTX=1: every step is an NVTX range named by its shape (for `ncu --nvtx --nvtx-include`)
        self.nvtx = self.device.type == "cuda" and os.environ.get("SHISO_NVTX", "0") not in ("", "0")
        if level:
            self.enable_layer_dump(level)
        if options.cuda_graphs and self.device.type == "cuda" and model.graph_safe:
            from .graphs import DecodeGraphs, decode_bucket

            most = decode_bucket(options.max_num_seqs) if cache.scratch_slot is not None else options.max_num_seqs
            decode_builder = StepBuilder(cache, self.device, most, most, fixed_table_width=cache.max_blocks, row_inputs=row_inputs)
            decode_builder.fed_tokens = self.fed_tokens
            decode_builder.ops = model.env.ops
            self.graphs = DecodeGraphs(model, cache, decode_builder)
            if options.graph_mixed_steps and cache.scratch_slot is not None:
                from .graphs import StepGraphs, sequence_bucket, token_bucket

                most_seqs = 2 * sequence_bucket(options.max_num_seqs)
                padded_builder = StepBuilder(
                    cache, self.device, token_bucket(options.max_num_batched_tokens + most_seqs), most_seqs,
                    fixed_table_width=cache.max_blocks, row_inputs=row_inputs,
                )
                padded_builder.fed_tokens = self.fed_tokens
                padded_builder.ops = model.env.ops
                self.step_graphs = StepGraphs(model, cache, padded_builder)

    def enable_layer_dump(self, level: int = 1, out=None) -> None:
        """Prints a line of statistics of the residual stream (count, rms, largest magnitude,
        zeros, non-finite values, first four values) after the embedding and after every run
        entry of every step; with ``level`` 2 after every mixer and feed-forward too.  The switch
        of the reference's layer loop (``SHISO_LAYER_DUMP=1|2``,
        crates/shiso-engine/src/trace.rs:27-138); the same variable turns it on here.  Lines go
        to standard error; steps run kernel by kernel while it is on."""
        from ..parts.model import residual_stats, stream_value

        out = out if out is not None else sys.stderr
        state = {"entry": -1}

        def after_entry(pos, stream):
            state["entry"] = pos
            kind = "embedding" if pos < 0 else self.model.plan.layers[self.model.plan.order[pos].layer].mixer.kind
            print(residual_stats(f"step {self.steps_run} entry {pos} ({kind})", stream_value(stream)), file=out, flush=True)

        def after_add(stream):
            print(residual_stats(f"step {self.steps_run} entry {state['entry'] + 1} part", stream_value(stream)), file=out, flush=True)

        self.layer_hook = after_entry
        self.add_hook = after_add if level >= 2 else None

    def enable_launch_profile(self, folder=None):
        """Times every launch of every step from now on (kernels/profile.py) and returns the
        ``StepProfiler`` that collects the rows; steps run kernel by kernel meanwhile.
        ``disable_launch_profile`` ends it.  The reference's ``--profile-dir``
        (crates/shiso-runtime/src/options.rs:139-146, crates/shiso-core/src/profile.rs:1-80)."""
        from ..kernels.profile import StepProfiler

        if not hasattr(self.env.ops, "profile_start"):
            raise ValueError("this kernel table has no launch profiler")
        self.profiler = StepProfiler(folder)
        return self.profiler

    def disable_launch_profile(self):
        profiler, self.profiler = self.profiler, None
        return profiler

    def warm_up(self) -> None:
        """Runs a two-token request through a prompt step and a decode step and drops it, so
        that every kernel has been loaded before the first graph capture."""
        probe = ("__warm_up__",)
        graphs, self.graphs = self.graphs, None  # (without decode graphs no step is captured)
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
        ops = ops if ops is not None else default_ops()
        if device.type == "cuda":
            # The kernel library keeps per-process state (kernel attributes it has set, its status
            # word, counters) for ONE device, and launches on the current device's stream: the
            # engine's device must be that one, and it is made the current device here.
            bind = getattr(ops, "bind_device", None)
            if bind is not None:
                device = torch.device("cuda", bind(device))
        env = BuildEnv(dtype=dtype, device=device, ops=ops)
        model = Model(plan, env)
        specs = model.tensor_specs()
        if isinstance(tensors_or_dir, str):
            tensors = load_weights(tensors_or_dir, specs, dtype, device)
        else:
            tensors = tensors_or_dir
            for name, t in tensors.items():
                if t.device != device and not (t.device.type == device.type and device.index is None):
                    raise ValueError(f"tensor {name} lies on {t.device}, the engine runs on {device}")
        model.bind(tensors)
        blocks_per_request = options.pages_per_context()
        needs = model.cache_needs()
        if options.gpu_memory_utilization is not None:
            page_bytes, state_bytes = CacheManager.costs(needs, options.page_size, dtype)
            if device.type == "cuda":
                free_bytes, total_bytes = torch.cuda.mem_get_info(device)
            else:
                import psutil

                memory = psutil.virtual_memory()
                free_bytes, total_bytes = memory.available, memory.total
            reserve = step_buffer_bytes(plan, options, dtype)
            pages, left = pool_pages_for_share(options.gpu_memory_utilization, total_bytes, free_bytes, page_bytes,
                                               options.max_num_seqs * state_bytes, reserve)
            num_pages = options.checked_pages(
                pages, f"{options.gpu_memory_utilization} of {total_bytes / 2**30:.2f} GiB leaves {left / 2**30:.2f} GiB "
                       f"for the cache once {(total_bytes - free_bytes) / 2**30:.2f} GiB in use, "
                       f"{options.max_num_seqs * state_bytes / 2**30:.3f} GiB of state slots and {reserve / 2**30:.2f} GiB "
                       f"for a step's buffers are taken out")
        else:
            num_pages = options.checked_pages(options.num_pages(), options.kv_cache_tokens
                                              if options.kv_cache_tokens is not None else options.max_num_seqs * options.ctx)
        cache = CacheManager(
            needs,
            options.page_size,
            num_pages,
            options.max_num_seqs,
            dtype,
            device,
            max_blocks_per_request=min(blocks_per_request, num_pages),
            # rows that pad a step to a captured shape live on pages and a slot of their own
            scratch_tokens=64 if options.cuda_graphs and options.graph_mixed_steps else 0,
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
        run) when the cache cannot hold the step, and ``ValueError`` (likewise) for a step
        that breaks a limit or names a place outside an entry's tokens."""
        entries = list(entries)
        seen = set()
        total = 0
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            count = len(e.tokens)
            total += count
            if count == 0:
                raise ValueError(f"request {e.request!r}: a step brings at least one token")
            if min(e.tokens) < 0 or max(e.tokens) >= self.vocab_size:
                raise ValueError(f"request {e.request!r}: a token id lies outside the vocabulary of {self.vocab_size}")
            if e.feed is not None and (count != 1 or not 0 <= e.feed < self.fed_tokens.shape[0] - 1):
                raise ValueError(f"request {e.request!r}: a fed token is one token from index 0..{self.fed_tokens.shape[0] - 2}")
            for w in e.want:
                if not 0 <= w < count:
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {count} tokens")
            for name, values in (e.extras or {}).items():
                if name not in self.model.plan.row_inputs:
                    raise ValueError(f"request {e.request!r}: the model reads no per-row input named {name!r}")
                if len(values) != count:
                    raise ValueError(f"request {e.request!r}: {len(values)} values of {name!r} for {count} tokens")
        if not entries:
            raise ValueError("a step needs at least one token")
        if total > self.builder.max_tokens or len(entries) > self.builder.max_seqs:
            raise ValueError(
                f"step of {total} tokens in {len(entries)} sequences exceeds the engine's "
                f"limits ({self.builder.max_tokens} tokens, {self.builder.max_seqs} sequences)"
            )
        # Admission check for the whole step before anything is claimed.
        self._check_room(entries)
        starts = []
        claimed = []
        fresh = [e.request for e in entries if not self.cache.has(e.request)]
        hooked = self.layer_hook is not None or self.add_hook is not None
        try:
            for e in entries:
                starts.append(self.cache.append(e.request, len(e.tokens)))
                claimed.append(e.request)
            ran = False
            if self.nvtx:
                torch.cuda.nvtx.range_push(f"step {self.steps_run}: {total} tokens, {len(entries)} sequences")
            if self.profiler is not None:
                self.env.ops.profile_start()
            if self.graphs is not None and not hooked and self.profiler is None:
                if all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
                    logits, ran = self.graphs.run(entries, starts), True
                elif self.step_graphs is not None:
                    logits = self.step_graphs.run(entries, starts)
                    ran = logits is not NOT_RUN
            if not ran:
                meta = self.builder.build(entries, starts)
                if hooked:
                    logits = self.model.forward(meta, self.cache, self.layer_hook, self.add_hook)
                else:
                    logits = self.model.forward(meta, self.cache)
            if self.profiler is not None:
                samples, wall_us, span_us = self.env.ops.profile_stop()
                decode = all(len(e.tokens) == 1 for e in entries)
                self.profiler.add("decode" if decode else "prompt", samples, wall_us, span_us)
            if self.nvtx:
                torch.cuda.nvtx.range_pop()
        except BaseException:
            if self.nvtx:
                torch.cuda.nvtx.range_pop()
            if self.profiler is not None and getattr(self.env.ops, "_region", None) is not None:
                self.env.ops.profile_stop()
            # Nothing of the step counts: claims are undone, and a request this step saw for the
            # first time holds nothing afterwards.  (Pages a known request grew into stay with it:
            # they hold no position yet and its next step uses them.)
            for request in claimed:
                self.cache.cancel(request)
            for request in fresh:
                if self.cache.has(request):
                    self.cache.release(request)
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
