"""Traces for the replay tests and a driver for ``bin/trace_run``."""

from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def round64(n):
    return -(-n // 64) * 64


def mixed_trace(requests, seed, max_tokens, max_live=4, tail=8, portion_sizes=(2, 3, 5, 7, 13)):
    """Up to ``max_live`` requests at a time; prompt portions of some beside single
    decoded tokens of others; a request is sometimes left out of a step; a new request
    starts as soon as the token budget (lengths rounded up to 64) allows, so pages that a
    finished request gave back are used again.  Every position is wanted."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}  # id -> [tokens, consumed]
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting[0]
            held = sum(round64(len(t)) for t, _ in live.values())
            if held + round64(len(toks)) > max_tokens:
                break
            waiting.pop(0)
            live[rid] = [toks, 0]
        if not live:
            raise ValueError("max_tokens is too small for the first waiting request")
        entries, end = [], []
        ids = list(live)
        rng.shuffle(ids)
        for rid in ids:
            toks, done = live[rid]
            if len(ids) > 1 and rng.random() < 0.25 and entries:
                continue  # left out of this step
            left = len(toks) - done
            if left <= tail:
                n = 1
            else:
                n = min(rng.choice(portion_sizes), left - tail) if left - tail >= 2 else left - tail
            entries.append((rid, toks[done : done + n], list(range(n))))
            live[rid][1] = done + n
            if done + n == len(toks):
                end.append(rid)
        for rid in end:
            del live[rid]
        steps.append((entries, end))
    return steps


def run_trace_run(model_dir, dtype, steps, max_tokens, out_dir, vocab, page_size=16, env=None, timeout=900):
    """Drives bin/trace_run over ``steps`` (as run_steps takes them), one line at a time,
    waiting for each ``done``; returns {request: {position: logits row}}."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, TRACE_RUN, "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    rows, consumed = {}, {}
    try:
        for number, (entries, end) in enumerate(steps):
            record = {
                "step": number,
                "entries": [{"id": r, "tokens": list(t), "want": list(w)} for r, t, w in entries],
                "end": list(end),
            }
            proc.stdin.write(json.dumps(record) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            if line.strip() != f"done {number}":
                raise RuntimeError(f"trace_run answered {line!r} to step {number} (exit code {proc.poll()})")
            wanted = sum(len(w) for _, _, w in entries)
            if wanted:
                data = np.fromfile(os.path.join(out_dir, f"{number}.f32"), dtype="<f4")
                assert data.size == wanted * vocab, (data.size, wanted, vocab)
                data = torch.from_numpy(data.reshape(wanted, vocab).copy())
            at = 0
            for r, t, w in entries:
                base = consumed.get(r, 0)
                for place in w:
                    rows.setdefault(r, {})[base + place] = data[at]
                    at += 1
                consumed[r] = base + len(t)
            for r in end:
                consumed.pop(r, None)
        proc.stdin.close()
        code = proc.wait(timeout=timeout)
        if code != 0:
            raise RuntimeError(f"trace_run exited with {code}")
    finally:
        if proc.poll() is None:
            proc.kill()
    return rows


def stack_rows(rows, request, length):
    return torch.stack([rows[request][i] for i in range(length)]).double()
