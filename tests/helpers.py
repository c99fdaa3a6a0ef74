"""Shared by the tests: the two tiny configurations, model folders, engines, replays."""

from __future__ import annotations

import json
import os

import torch

from shiso_llm_b200.config import plan_from_document
from shiso_llm_b200.engine import Engine, EngineOptions, StepEntry
from shiso_llm_b200.parts import BuildEnv, Model
from shiso_llm_b200.weights import random_tensors, write_model_folder

# Two tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Lfm2ForCausalLM"],
    "model_type": "lfm2",
    "vocab_size": 512,
    "hidden_size": 64,
    "num_hidden_layers": 4,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "conv_L_cache": 3,
    "conv_bias": False,
    "block_ff_dim": 192,
    "block_auto_adjust_ff_dim": False,
    "block_multiple_of": 256,
    "block_ffn_dim_multiplier": 1.0,
    "norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "tie_embedding": True,
}

TINY_B = {
    "architectures": ["Lfm2ForCausalLM"],
    "model_type": "lfm2",
    "vocab_size": 1000,
    "hidden_size": 96,
    "num_hidden_layers": 6,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "layer_types": ["conv", "conv", "full_attention", "conv", "full_attention", "full_attention"],
    "conv_L_cache": 4,
    "conv_bias": True,
    "block_ff_dim": 384,
    "block_auto_adjust_ff_dim": True,
    "block_multiple_of": 64,
    "block_ffn_dim_multiplier": 1.0,
    "norm_eps": 1e-6,
    "rope_theta": 1000000.0,
    "tie_embedding": False,
}

TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1)}


def tensor_specs_of(document):
    """The tensors a configuration's model asks for (no device, no kernels needed)."""
    _, _, plan = plan_from_document(document)
    env = BuildEnv(dtype=torch.float32, device=torch.device("cpu"), ops=None)
    return Model(plan, env).tensor_specs()


def make_tensors(document, seed, std=0.02, norm_jitter=0.1, storage_dtype="bfloat16"):
    """Random weights whose values are exactly representable in bfloat16, so that the
    float32 and bfloat16 engines and the plain implementation all see the same weights.
    Norm weights are jittered around 1 so that a norm applied with the wrong weight shows."""
    return random_tensors(tensor_specs_of(document), seed, std, storage_dtype, norm_jitter)


def make_folder(path, document, seed, **kw):
    tensors = make_tensors(document, seed, **kw)
    write_model_folder(str(path), document, tensors)
    return tensors


def random_prompt(length, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def make_engine(model_dir, dtype, ops=None, device=None, **options):
    opts = EngineOptions(dtype=dtype, device=device or ("cpu" if ops is not None else "cuda:0"), **options)
    return Engine.from_folder(str(model_dir), opts, ops)


def run_steps(engine, steps):
    """Runs ``steps`` = list of (entries, end) where entries = [(request, tokens, want)];
    returns {request: {position: logits row (CPU float32)}}."""
    rows = {}
    consumed = {}
    for entries, end in steps:
        batch = [StepEntry(r, t, w) for r, t, w in entries]
        logits = engine.step(batch)
        if logits is not None:
            logits = logits.float().cpu()
        at = 0
        for r, t, w in entries:
            base = consumed.get(r, 0)
            for place in w:
                rows.setdefault(r, {})[base + place] = logits[at].clone()
                at += 1
            consumed[r] = base + len(t)
        for r in end:
            engine.finish(r)
            consumed.pop(r, None)
        engine.cache.check()
    return rows


def whole(request, tokens):
    """One step: the whole sequence, every position wanted."""
    return [([(request, tokens, list(range(len(tokens))))], [request])]


def tail_one_by_one(request, tokens, tail=32):
    tail = min(tail, len(tokens) - 1)
    head = len(tokens) - tail
    steps = [([(request, tokens[:head], list(range(head)))], [])]
    for i in range(head, len(tokens)):
        steps.append(([(request, [tokens[i]], [0])], [request] if i == len(tokens) - 1 else []))
    return steps


def portions(request, tokens, sizes):
    """Portions of changing size (cycled), every position wanted."""
    steps, at, i = [], 0, 0
    while at < len(tokens):
        n = min(sizes[i % len(sizes)], len(tokens) - at)
        last = at + n == len(tokens)
        steps.append(([(request, tokens[at : at + n], list(range(n)))], [request] if last else []))
        at += n
        i += 1
    return steps
