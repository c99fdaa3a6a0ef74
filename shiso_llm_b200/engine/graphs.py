"""Captured decode steps.

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


class DecodeGraphs:
    def __init__(self, model, cache, builder, max_graphs: int = 24):
        self.model = model
        self.cache = cache
        self.builder = builder  # a StepBuilder with a fixed table width
        self.max_graphs = max_graphs
        self._graphs: OrderedDict = OrderedDict()  # num_seqs -> (graph, logits)
        self.replays = 0
        self.launches_per_graph: dict = {}

    def run(self, entries, starts):
        """Uploads the step's metadata and replays (capturing first if needed) the graph for
        this many sequences.  Every entry wants its one row.  Returns logits [S, vocab]."""
        meta = self.builder.build(entries, starts)
        key = meta.num_seqs
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
        return logits

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
        return self.launches_per_graph.get(num_seqs, 0)
