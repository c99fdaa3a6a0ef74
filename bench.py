#!/usr/bin/env python3
"""Serving benchmark: decode and prefill throughput of an LFM2-1.2B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 (a step = one
decode step over the cache of 2,048-token prompts), timed on the device with CUDA events
around K steps; ``e2e`` is the same through the Python entry point (``LLM.step``: host
token ids in, sampled ids out every step).  ``prefill`` is one 2,048-token prompt step;
``roofline`` relates the decode step's mandatory bytes (every weight once, the live
requests' cache) to the measured HBM bandwidth; ``points`` holds batch 1 and 64.

Protocol after the reference's bench crate (crates/shiso-bench/src/measure.rs:10-33,62-77;
decode.rs:12-22): one warm-up repetition is discarded, then seven repetitions are timed, each
on fresh requests at the same context (prompts read again, W warm-up steps, then exactly K
timed steps); the MEDIAN repetition is reported with the spread (slowest / fastest - 1), and a
spread above 2 % is flagged, not hidden.  Sampling is greedy with end-of-sequence ignored so
every run takes every step; the read-back of the tokens lies inside the end-to-end window.
The model's weights (1.8 GB) are read every step and exceed the 126 MB L2, so consecutive
steps do not reuse cached inputs.  ``points`` also carries two serving workloads after the
reference's own benchmark scenarios (350M shape: 64 concurrent requests; 2.6B shape: a long prompt in portions
beside 32 decoding streams), unless ``--points`` leaves them out.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PROMPT_LEN = 2048
NEW_TOKENS = 256


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for key in out:
                if isinstance(data.get(key), (int, float)):
                    out[key] = float(data[key])
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for parts in self.samples:
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max_clock,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def model_costs(engine, config):
    """Bytes a decode step must read that do not depend on the batch (weights, each once), the
    cache bytes per token and per request, and the FLOPs of a prompt step of T tokens."""
    from shiso_llm_b200.parts.base import FixedState, PagedKV
    from shiso_llm_b200.weights.spec import MATRIX

    specs = {s.name: s for s in engine.model.tensor_specs()}
    embed_name = engine.model.plan.embedding.params["tensor"]
    weight_bytes, gemm_params = 0, 0
    itemsize = 2 if engine.env.dtype.itemsize == 2 else 4
    for name, spec in specs.items():
        n = 1
        for d in spec.shape:
            n *= d
        if spec.role == MATRIX:
            if name == embed_name:
                continue  # only the looked-up rows are read; the head is counted below
            weight_bytes += n * itemsize
            gemm_params += n
        else:
            weight_bytes += n * 4
    head_params = config.vocab_size * config.hidden_size
    weight_bytes += head_params * itemsize  # the output head (the embedding table when tied)
    kv_bytes_per_token, state_bytes = 0, 0
    attn_layers = 0
    for need in engine.model.cache_needs():
        if isinstance(need, PagedKV):
            kv_bytes_per_token += 2 * need.num_kv_heads * need.head_dim * itemsize
            attn_layers += 1
        elif isinstance(need, FixedState):
            state_bytes += need.numel * 4 * 2  # read and written
    return {
        "weight_bytes": weight_bytes,
        "gemm_params": gemm_params,
        "head_params": head_params,
        "kv_bytes_per_token": kv_bytes_per_token,
        "state_bytes_per_request": state_bytes,
        "attn_layers": attn_layers,
    }


def prefill_flops(costs, config, tokens):
    gemm = 2.0 * tokens * costs["gemm_params"] + 2.0 * costs["head_params"]  # head: the last row only
    heads, d = config.num_attention_heads, config.head_dim
    attention = costs["attn_layers"] * 4.0 * heads * d * (tokens * (tokens + 1) / 2)
    return gemm + attention


def load_preset(name, layers=None):
    from shiso_llm_b200.cli import preset_path
    from shiso_llm_b200.config import plan_from_document

    with open(preset_path(name)) as f:
        document = json.load(f)
    full_layers = document["num_hidden_layers"]
    if layers is not None and layers < full_layers:
        document["layer_types"] = document["layer_types"][:layers]
        document["num_hidden_layers"] = layers
    _, config, plan = plan_from_document(document)
    return config, plan, full_layers


def graph_replays(engine) -> dict:
    return {"decode": engine.graphs.replays if engine.graphs else 0,
            "mixed": engine.step_graphs.replays if engine.step_graphs else 0,
            "mixed_shapes_captured": engine.step_graphs.captures if engine.step_graphs else 0,
            "steps": engine.steps_run}


def run_workload(workload, preset, config, plan, full_layers) -> dict:
    """The two serving workloads beside the headline: whole requests through the scheduler and the
    Python entry point, host token ids in and out, wall-clock time.  Returns the record."""
    import torch

    from shiso_llm_b200 import LLM, SamplingParams
    from shiso_llm_b200.engine import Engine, EngineOptions
    from shiso_llm_b200.kernels import ops
    from shiso_llm_b200.parts import BuildEnv, Model
    from shiso_llm_b200.weights import random_device_tensors

    device = torch.device("cuda:0")
    ops.require()
    probe = Model(plan, BuildEnv(dtype=torch.bfloat16, device=device, ops=ops))
    tensors = random_device_tensors(probe.tensor_specs(), 0, torch.bfloat16, device)
    del probe
    gen = torch.Generator().manual_seed(4321)

    def prompt(n):
        return torch.randint(0, config.vocab_size, (n,), generator=gen).tolist()

    def drive(llm, until=None):
        """Steps until nothing is left (or ``until()`` holds); returns (steps, seconds)."""
        torch.cuda.synchronize()
        t0, steps = time.perf_counter(), 0
        while llm.has_unfinished() and not (until and until()):
            llm.step()
            steps += 1
        llm.drain()
        torch.cuda.synchronize()
        return steps, time.perf_counter() - t0

    base = {
        "impl": "ours", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "unit": "tok/s", "higher_is_better": True,
        "config": {"model": f"{preset} (random weights)", "layers_run": config.num_hidden_layers,
                   "layers_full": full_layers, "hidden_size": config.hidden_size,
                   "intermediate_size": config.intermediate_size, "page_size": 16},
    }
    if workload == "serve":
        count, new_tokens, chunk = 64, 128, 512
        lengths = torch.randint(16, 2049, (count,), generator=gen).tolist()
        options = EngineOptions(dtype="bfloat16", ctx=4096, page_size=16, kv_cache_tokens=count * (2048 + new_tokens + 64),
                                max_num_seqs=count, max_num_batched_tokens=chunk + count)
        llm = LLM(Engine.from_plan(plan, tensors, options), prefill_chunk=chunk)
        params = SamplingParams(temperature=0.0, max_new_tokens=new_tokens, ignore_eos=True)
        for rep in range(3):  # two passes warm up (a step's shape is captured when it comes again); the third is timed
            for n in lengths:
                llm.add_request(prompt(n), params)
            steps, seconds = drive(llm)
            llm.scheduler.take_finished()
        produced = count * new_tokens
        return {**base, "metric": "generated tok/s, 64 concurrent requests, prompts 16..2048, 512-token portions, "
                "128 new tokens each (continuous batching through LLM.step)",
                "value": produced / seconds, "seconds": seconds, "steps": steps,
                "prompt_tokens": sum(lengths), "prompt_tok_s": sum(lengths) / seconds,
                "generated_tokens": produced, "preempted": llm.scheduler.stats["preempted"],
                "graph_replays": graph_replays(llm.engine)}
    # mixed: 32 streams decode while one long prompt is read in portions; then 64 streams decode
    streams, long_prompt, chunk, new_tokens = 32, 8192, 1024, 256
    options = EngineOptions(dtype="bfloat16", ctx=8192 + 512, page_size=16,
                            kv_cache_tokens=long_prompt + 512 + 64 * (1024 + new_tokens + 64),
                            max_num_seqs=64, max_num_batched_tokens=chunk + 64)
    llm = LLM(Engine.from_plan(plan, tensors, options), prefill_chunk=chunk)
    params = SamplingParams(temperature=0.0, max_new_tokens=4096, ignore_eos=True)
    results = {}
    for rep in range(3):
        ids = [llm.add_request(prompt(1024), params).id for _ in range(streams)]
        drive(llm, until=lambda: all(r.decoding for r in llm.scheduler.running) and not llm.scheduler.waiting)
        long_request = llm.add_request(prompt(long_prompt), SamplingParams(temperature=0.0, max_new_tokens=1, ignore_eos=True))
        steps, seconds = drive(llm, until=lambda: long_request.state == "finished")
        results["mixed"] = {"steps": steps, "seconds": seconds, "ms_per_step": seconds / max(steps, 1) * 1e3,
                            "prompt_tok_s": long_prompt / seconds, "decode_tok_s_beside": streams * steps / seconds}
        more = [llm.add_request(prompt(1024), params).id for _ in range(64 - streams)]
        drive(llm, until=lambda: all(r.decoding for r in llm.scheduler.running) and not llm.scheduler.waiting)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(new_tokens):
            llm.step()
        llm.drain()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        results["decode_b64"] = {"tok_s": 64 * new_tokens / seconds, "ms_per_step": seconds / new_tokens * 1e3}
        for rid in ids + more:
            llm.abort(rid)
        llm.drain()
        llm.scheduler.take_finished()
    return {**base, "metric": "prompt tok/s of one 8,192-token prompt read in 1,024-token portions beside 32 "
            "decoding streams; then decode tok/s at batch 64 (through LLM.step)",
            "value": results["mixed"]["prompt_tok_s"], **results, "graph_replays": graph_replays(llm.engine)}


def main() -> int:
    global PROMPT_LEN
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--preset", default="lfm2-1.2b")
    parser.add_argument("--layers", type=int, default=None, help="run only the first N layers (recorded in config)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-len", type=int, default=PROMPT_LEN,
                        help="tokens of every prompt, and of the prompt step that is timed (the contract's line: 2,048)")
    parser.add_argument("--points", default="1,64,serve_350m,mixed_2p6b",
                        help="what else to report: decode batch sizes, and the serving workloads serve_350m / mixed_2p6b; 'none' for nothing")
    parser.add_argument("--reps", type=int, default=7, help="timed repetitions of the K-step block (after one that is discarded)")
    parser.add_argument("--no-cuda-graphs", action="store_true")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--workload", choices=["decode", "serve", "mixed"], default="decode",
                        help="decode: the contract's line (default).  serve: 64 concurrent requests with prompts of "
                             "16..2048 tokens, 512-token portions, 128 new tokens each, through LLM.generate (use with "
                             "--preset lfm2-350m).  mixed: one 8,192-token prompt in 1,024-token portions beside 32 "
                             "decoding streams, then batch-64 decode of 256 tokens (use with --preset lfm2-2.6b).")
    parser.add_argument("--profiler-range", choices=["decode", "prefill"], default=None,
                        help="bracket the device-timed decode steps (or the prefill steps) with cudaProfilerStart/Stop, "
                             "for `ncu --profile-from-start off`")
    args = parser.parse_args()
    PROMPT_LEN = args.prompt_len

    if args.impl == "reference":
        print(json.dumps({
            "impl": "reference",
            "unavailable": "the reference is a Rust workspace and this image has no cargo/rustc; its LFM2 path is "
                           "GGUF-quantized only and its short-conv kernel exists only for Metal, so it cannot run here",
        }))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from shiso_llm_b200 import LLM, SamplingParams
    from shiso_llm_b200.engine import Engine, EngineOptions, StepEntry
    from shiso_llm_b200.engine.batch import MetaLayout
    from shiso_llm_b200.kernels import ops
    from shiso_llm_b200.parts import BuildEnv, Model
    from shiso_llm_b200.weights import random_device_tensors

    config, plan, full_layers = load_preset(args.preset, args.layers)
    device = torch.device("cuda:0")
    if args.workload != "decode":
        print(json.dumps(run_workload(args.workload, args.preset, config, plan, full_layers)))
        return 0
    names = [b.strip().lower() for b in args.points.split(",") if b.strip() and b.strip().lower() != "none"]
    batches = [args.batch] + [int(b) for b in names if b.isdigit()]
    max_batch = max(batches)
    reps = max(3, args.reps)
    # a repetition's requests: prompt, warm-up steps, the end-to-end block and the device-timed block
    # (the first request also decodes while the others' prompts are read, one prompt a step)
    budget = PROMPT_LEN + 2 * (args.steps + args.warmup) + 2 * max_batch + 64
    ctx = max(4096, -(-budget // 16) * 16)
    options = EngineOptions(
        dtype="bfloat16", ctx=ctx, page_size=16, kv_cache_tokens=max(max_batch * budget, ctx),
        max_num_seqs=max_batch, max_num_batched_tokens=PROMPT_LEN, cuda_graphs=not args.no_cuda_graphs,
    )
    ops.require()
    probe = Model(plan, BuildEnv(dtype=torch.bfloat16, device=device, ops=ops))
    tensors = random_device_tensors(probe.tensor_specs(), 0, torch.bfloat16, device)
    del probe
    engine = Engine.from_plan(plan, tensors, options)
    costs = model_costs(engine, config)
    peak, peak_source = peaks()
    gen = torch.Generator().manual_seed(1234)

    def prompts(n):
        return [torch.randint(0, config.vocab_size, (PROMPT_LEN,), generator=gen).tolist() for _ in range(n)]

    def one_repetition(batch: int, steps: int, warmup: int, profile: bool) -> dict:
        """Fresh requests: prompts of 2,048 tokens, ``warmup`` decode steps, then ``steps`` steps end
        to end through LLM.step and ``steps`` steps device-timed through Engine.step."""
        llm = LLM(engine)
        params = SamplingParams(temperature=0.0, max_new_tokens=2 * batch + steps + warmup + 16, ignore_eos=True)
        for p in prompts(batch):
            llm.add_request(p, params)
        # prompts are admitted one per step; run until every request is decoding
        while any(not r.decoding for r in llm.scheduler.running) or llm.scheduler.waiting:
            llm.step()
        for _ in range(warmup):
            llm.step()
        llm.drain()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        llm.drain()  # the last step's tokens reach the host inside the timed region too
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        assert len(llm.scheduler.running) == batch, "a request ended inside the timed region"

        # device-timed: the same requests, next tokens fed without waiting for the host
        requests = list(llm.scheduler.running)
        entries = [StepEntry(r.id, [r.tokens[-1]], [0]) for r in requests]
        for _ in range(3):
            ops.argmax(engine.step(entries))
        torch.cuda.synchronize()
        launches_before = ops.launch_count
        replays_before = engine.graphs.replays if engine.graphs else 0
        first_context = sum(engine.cache.length(r.id) for r in requests) / batch
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if profile:
            torch.cuda.cudart().cudaProfilerStart()
        start.record()
        for _ in range(steps):
            ops.argmax(engine.step(entries))
        end.record()
        torch.cuda.synchronize()
        if profile:
            torch.cuda.cudart().cudaProfilerStop()
        ops.check_kernel_status()
        device_ms = start.elapsed_time(end)
        launches = ops.launch_count - launches_before
        if engine.graphs:
            launches += (engine.graphs.replays - replays_before) * engine.graphs.launches(batch)
        context = first_context + (steps - 1) / 2.0  # the mean over the timed steps
        for r in requests:
            llm.abort(r.id)
        llm.drain()
        return {"device_ms": device_ms / steps, "e2e_ms": e2e_s / steps * 1e3, "launches": launches, "context": context}

    def measure_decode(batch: int, steps: int, warmup: int, sampler=None) -> dict:
        """The median of ``reps`` repetitions after one that is discarded."""
        one_repetition(batch, steps, warmup, False)
        if sampler is not None:
            sampler.start()
        runs = [one_repetition(batch, steps, warmup, args.profiler_range == "decode" and batch == args.batch and i == 0)
                for i in range(reps)]
        clock_info = sampler.stop() if sampler is not None else None
        device = sorted(r["device_ms"] for r in runs)
        e2e = sorted(r["e2e_ms"] for r in runs)
        ms, e2e_ms = statistics.median(device), statistics.median(e2e)
        context = runs[0]["context"]
        step_bytes = costs["weight_bytes"] + batch * (context * costs["kv_bytes_per_token"] + costs["state_bytes_per_request"])
        spread = device[-1] / device[0] - 1.0
        return {
            "batch": batch, "tok_s": batch / (ms / 1e3), "ms_per_step": ms, "spread": spread,
            "spread_over_2_percent": spread > 0.02, "repetitions": reps,
            "e2e_tok_s": batch / (e2e_ms / 1e3), "e2e_ms_per_step": e2e_ms, "e2e_spread": e2e[-1] / e2e[0] - 1.0,
            "launches": runs[0]["launches"], "context": context, "clocks": clock_info,
            "bytes_per_step": step_bytes, "gbs": step_bytes / (ms / 1e3) / 1e9,
            "frac": step_bytes / (ms / 1e3) / 1e9 / peak["hbm_gbs"],
            "h2d": 4 * MetaLayout(batch, batch, batch, len(engine.cache.groups), engine.cache.max_blocks).total,
            "d2h": 4 * (batch + 1),
        }

    def measure_prefill(reps: int = 11, warmup: int = 3) -> dict:
        times = []
        for i in range(warmup + reps):
            tokens = prompts(1)[0]
            request = ("prefill", i)
            torch.cuda.synchronize()
            profiled = args.profiler_range == "prefill" and i == warmup
            if profiled:
                torch.cuda.cudart().cudaProfilerStart()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([StepEntry(request, tokens, [PROMPT_LEN - 1])])
            end.record()
            torch.cuda.synchronize()
            if profiled:
                torch.cuda.cudart().cudaProfilerStop()
            engine.finish(request)
            if i >= warmup:
                times.append(start.elapsed_time(end))
        ops.check_kernel_status()
        ms = statistics.median(times)
        flops = prefill_flops(costs, config, PROMPT_LEN)
        return {
            "value": PROMPT_LEN / (ms / 1e3), "tokens": PROMPT_LEN, "ms": ms,
            "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12),
            "tflops": flops / (ms / 1e3) / 1e12, "spread": max(times) / min(times) - 1.0, "repetitions": reps,
        }

    main_point = measure_decode(args.batch, args.steps, args.warmup, ClockSampler())
    points, details = {}, {}

    def detail(m):
        return {k: m[k] for k in ("tok_s", "ms_per_step", "spread", "bytes_per_step", "gbs", "frac", "e2e_tok_s", "context")}

    details[f"decode_b{args.batch}"] = detail(main_point)
    for b in batches[1:]:
        try:
            m = measure_decode(b, args.steps, args.warmup)
            points[f"decode_b{b}"] = m["tok_s"]
            points[f"decode_b{b}_frac"] = m["frac"]
            details[f"decode_b{b}"] = detail(m)
        except Exception as e:  # a point that cannot run is reported, not hidden
            points[f"decode_b{b}"] = None
            points[f"decode_b{b}_error"] = f"{type(e).__name__}: {e}"[:200]
    prefill = None if args.skip_prefill else measure_prefill()

    # the serving workloads of the other two shapes, each with a model of its own
    del engine, tensors
    torch.cuda.empty_cache()
    for name, workload, preset in (("serve_350m", "serve", "lfm2-350m"), ("mixed_2p6b", "mixed", "lfm2-2.6b")):
        if name not in names:
            continue
        try:
            other_config, other_plan, other_layers = load_preset(preset)
            record = run_workload(workload, preset, other_config, other_plan, other_layers)
            points[name] = record["value"]
            details[name] = {k: v for k, v in record.items() if k not in ("config", "impl", "n_gpus", "dtype", "data", "higher_is_better")}
        except Exception as e:
            points[name] = None
            points[f"{name}_error"] = f"{type(e).__name__}: {e}"[:200]
        torch.cuda.empty_cache()

    line = {
        "metric": f"decode tok/s at batch {args.batch} ({args.preset.upper()}-shaped, bf16, {PROMPT_LEN}-token prompts)",
        "value": main_point["tok_s"],
        "unit": "tok/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": main_point["ms_per_step"],
        "spread": main_point["spread"],
        "repetitions": reps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": f"{args.preset} (random weights)",
            "global_batch": args.batch,
            "seq_len": ctx,
            "parallelism": "single-gpu",
            "layers_run": config.num_hidden_layers,
            "layers_full": full_layers,
            "hidden_size": config.hidden_size,
            "intermediate_size": config.intermediate_size,
            "heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim,
            "vocab_size": config.vocab_size,
            "conv_L_cache": config.conv_L_cache,
            "attention_layers": costs["attn_layers"],
            "prompt_len": PROMPT_LEN,
            "mean_context": main_point["context"],
            "page_size": 16,
            "step_launch": ("cuda graph" if not args.no_cuda_graphs else "kernel by kernel") + ", lookahead 1 in e2e; the step's inputs and tokens cross from and to pinned host memory by kernel",
            "l2": "inputs larger than L2 (1.8 GB of weights read per step)",
            "peaks": peak_source,
        },
        "clocks": main_point["clocks"],
        "e2e": {
            "value": main_point["e2e_tok_s"], "unit": "tok/s", "ms_per_step": main_point["e2e_ms_per_step"],
            "spread": main_point["e2e_spread"],
            "h2d_bytes_per_step": main_point["h2d"], "d2h_bytes_per_step": main_point["d2h"],
        },
        "gpu_launches": main_point["launches"],
        "prefill": prefill,
        "roofline": {
            "bound": "hbm", "achieved": main_point["gbs"], "peak": peak["hbm_gbs"], "unit": "GB/s",
            "frac": main_point["frac"], "bytes_per_step": main_point["bytes_per_step"],
        },
        "points": points,
        "point_details": details,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
