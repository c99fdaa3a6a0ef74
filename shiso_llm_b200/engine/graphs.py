"""Captured steps: decode steps by batch size, mixed steps by padded shape.

A step in which every sequence brings exactly one token launches a hundred or more small
kernels; captured once per batch size as a CUDA graph it is replayed with one call.  The
step's metadata lives in the step builder's fixed device block (laid out by batch size
alone, with block tables at their full width), and is written outside the capture, before
each replay; every kernel reads positions, lengths and tables from that block, so the same
graph serves any mix of requests of that count.  The reference keys its decode graphs by
(rows, ordered session ids) and likewise writes inputs outside the capture at fixed
addresses (crates/shiso-engine/src/stack.rs:228-245,1199-1239).

Kernels inside a captured step must not size their launches by host facts that change from
step to step (context lengths); they size by the capacity (the table width) instead.
"""

from __future__ import annotations

from collections import OrderedDict

import torch


def decode_bucket(seqs: int) -> int:
    """The captured batch size a decode step of ``seqs`` rows runs as: itself up to 8 rows (the
    products for a handful of rows are kernels of their own), then the next multiple of 8, from
    64 on of 16.  A workload that drains walks through a dozen graphs instead of one per size."""
    if seqs <= 8:
        return seqs
    if seqs <= 64:
        return -(-seqs // 8) * 8
    return -(-seqs // 16) * 16


class DecodeGraphs:
    def __init__(self, model, cache, builder, max_graphs: int = 24):
        self.model = model
        self.cache = cache
        self.builder = builder  # a StepBuilder with a fixed table width
        self.max_graphs = max_graphs
        self._graphs: OrderedDict = OrderedDict()  # captured batch size -> (graph, logits)
        self.replays = 0
        self.launches_per_graph: dict = {}

    def run(self, entries, starts):
        """Uploads the step's metadata and replays (capturing first if needed) the graph for
        this many sequences, or for the next captured size with made-up rows on the cache's
        scratch page behind the step's own.  Every entry wants its one row.  Returns logits
        [S, vocab]."""
        seqs = len(entries)
        key = decode_bucket(seqs)
        if key == seqs or key > self.builder.max_seqs or self.cache.scratch_slot is None:
            key = seqs
            meta = self.builder.build(entries, starts)
        else:
            meta = self.builder.build(entries, starts, pad=(key, key, key))
        held = self._graphs.get(key)
        if held is None:
            held = self._capture(meta)
            self._graphs[key] = held
            while len(self._graphs) > self.max_graphs:
                self._graphs.popitem(last=False)
        else:
            self._graphs.move_to_end(key)
        graph, logits = held
        graph.replay()
        self.replays += 1
        return logits if key == seqs else logits[:seqs]

    def _capture(self, meta):
        ops = self.model.env.ops
        before = getattr(ops, "launch_count", 0)
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            logits = self.model.forward(meta, self.cache)
        self.launches_per_graph[meta.num_seqs] = getattr(ops, "launch_count", 0) - before
        return graph, logits

    def launches(self, num_seqs: int) -> int:
        return self.launches_per_graph.get(decode_bucket(num_seqs), self.launches_per_graph.get(num_seqs, 0))


NOT_RUN = object()  # StepGraphs.run: the caller runs the step kernel by kernel
LONG_PORTION = 128  # a step with a portion of at least this many rows takes the attention kernel for long portions


def token_bucket(tokens: int) -> int:
    """The captured row count a step of ``tokens`` rows is padded to: 16, 32, then multiples of 64."""
    if tokens <= 16:
        return 16
    if tokens <= 32:
        return 32
    return -(-tokens // 64) * 64


def sequence_bucket(seqs: int) -> int:
    """The captured sequence count: the next power of two."""
    n = 1
    while n < seqs:
        n *= 2
    return n


def padded_shape(tokens: int, seqs: int) -> tuple:
    """``(rows, sequences)`` a step of ``tokens`` rows in ``seqs`` sequences runs as.  Rows that
    are added need a made-up sequence to belong to, and every made-up sequence a row; a step
    that lies on the grid already (2,048 rows of one prompt) is taken as it is, so that padding
    never costs a product another tile of tokens where it can be helped."""
    many = sequence_bucket(seqs)
    while True:
        made_up = many - seqs
        rows = token_bucket(tokens + made_up)
        if made_up > 0 or rows == tokens:
            return rows, many
        many *= 2


class StepGraphs:
    """Captured mixed steps - portions of prompts beside decoded tokens.

    Such a step launches a hundred or more kernels from Python, which takes as long as the
    device needs for them; its shape (rows, sequences, wanted rows) seldom comes twice, so the
    step is padded to a shape out of a small set: rows to 16, 32 or a multiple of 64, sequences
    to a power of two, wanted rows to the sequence count.  The padding is made-up sequences on
    the cache manager's scratch pages and scratch slot (``StepBuilder.build(.., pad=..)``), so no
    kernel knows of it.  A shape is captured when it comes the second time (the first time it
    runs kernel by kernel, which also loads every kernel of its route before a capture needs
    it), and replayed from then on; metadata is written outside the capture at fixed
    addresses, and kernels size their launches by the shape, never by the step's own lengths.
    All graphs share one memory pool, which therefore holds what the widest step needs: the
    engine's workspace.  The reference allocates its scratch once for the widest pass
    (crates/shiso-engine/src/layers.rs:861-1027) and captures decode passes only
    (crates/shiso-engine/src/stack.rs:1199-1239)."""

    def __init__(self, model, cache, builder, max_graphs: int = 32):
        self.model = model
        self.cache = cache
        self.builder = builder  # fixed table width, sized for the largest padded shape
        self.max_graphs = max_graphs
        self._graphs: OrderedDict = OrderedDict()  # key -> (graph, logits)
        self._seen: dict = {}
        self.pool = None
        self.replays = 0
        self.captures = 0
        self.launches_per_graph: dict = {}

    def shape_of(self, entries):
        """``(rows, sequences, wanted, long)`` the step is padded to, or None when it does not fit."""
        tokens = sum(len(e.tokens) for e in entries)
        wanted = sum(len(e.want) for e in entries)
        rows, seqs = padded_shape(tokens, len(entries))
        made_up = seqs - len(entries)
        spare_last = rows - tokens - (made_up - 1) if made_up else 0
        if (rows > self.builder.max_tokens or seqs > self.builder.max_seqs or wanted > seqs
                or spare_last > len(self.cache.scratch_pages) * self.cache.page_size):
            return None
        long = max(len(e.tokens) for e in entries) >= LONG_PORTION
        return rows, seqs, seqs, long

    def run(self, entries, starts):
        """Logits ``[wanted, vocab]`` of the step (None when nothing is wanted) from a replayed
        graph, or ``NOT_RUN`` when the caller should run the step kernel by kernel (a shape
        that does not fit, or that came for the first time)."""
        key = self.shape_of(entries)
        if key is None:
            return NOT_RUN
        held = self._graphs.get(key)
        if held is None:
            self._seen[key] = self._seen.get(key, 0) + 1
            if self._seen[key] < 2:
                return NOT_RUN
        rows, seqs, wanted, long = key
        meta = self.builder.build(entries, starts, pad=(rows, seqs, wanted))
        # what kernels choose their route by is the shape's, not this step's
        meta.max_q_len = rows if long else min(rows, LONG_PORTION - 1)
        if held is None:
            held = self._capture(key, meta)
            self._graphs[key] = held
            while len(self._graphs) > self.max_graphs:
                self._graphs.popitem(last=False)
        else:
            self._graphs.move_to_end(key)
        graph, logits = held
        graph.replay()
        self.replays += 1
        real_wanted = sum(len(e.want) for e in entries)
        if real_wanted == 0:
            return None
        return logits[:real_wanted]

    def _capture(self, key, meta):
        ops = self.model.env.ops
        before = getattr(ops, "launch_count", 0)
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(graph, pool=self.pool):
            logits = self.model.forward(meta, self.cache)
        self.launches_per_graph[key] = getattr(ops, "launch_count", 0) - before
        self.captures += 1
        return graph, logits
