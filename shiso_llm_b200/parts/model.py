"""The model: parts assembled from a plan, run in the plan's order.

Nothing here names an architecture.  ``Model`` builds one block per layer of the
plan, collects the tensors they ask for, binds them after loading, reports the cache
need of every run entry, and runs a step: embedding, the run order, and the final
norm + head for the rows whose logits are wanted.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..weights.spec import TensorSpec
from .base import BLOCKS, EMBEDDINGS, HEADS, NORMS, BuildEnv, DeferredLinear, Stream
from .plan import ModelPlan


def stream_value(stream: Stream) -> torch.Tensor:
    """The residual stream as float32 rows, with the block output that is still waiting to be
    added, without touching the stream: a product that has not run is run on the side."""
    x = stream.residual
    waiting = stream.pending
    if waiting is None:
        return x.clone()
    if isinstance(waiting, DeferredLinear):
        waiting = waiting.materialize()
    return x + waiting.to(x.dtype)


def residual_stats(label: str, x: torch.Tensor) -> str:
    """One line about a block of float32 rows: element count, root mean square and largest
    magnitude of the finite values, zeros, non-finite values and the first four values - the
    line of the reference's layer dump (crates/shiso-engine/src/trace.rs:49-138)."""
    flat = x.detach().to(torch.float64).flatten().cpu()
    finite = torch.isfinite(flat)
    good = flat[finite]
    rms = float(good.pow(2).mean().sqrt()) if good.numel() else 0.0
    absmax = float(good.abs().max()) if good.numel() else 0.0
    first = [float(v) for v in flat[:4]]
    return (f"{label}: n={flat.numel()} rms={rms:.6e} absmax={absmax:.6e} zeros={int((good == 0).sum())} "
            f"non_finite={int((~finite).sum())} first={first}")


class Model:
    def __init__(self, plan: ModelPlan, env: BuildEnv):
        self.plan = plan
        self.env = env
        self.embedding = EMBEDDINGS.build(plan.embedding, env)
        self.blocks = [BLOCKS.build(layer.block, env, layer) for layer in plan.layers]
        self.final_norm = NORMS.build(plan.final_norm, env)
        self.head = HEADS.build(plan.head, env)
        self.bound = False

    # ------------------------------------------------------------------ weights

    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def tensor_specs(self) -> list[TensorSpec]:
        specs = []
        for part in self.parts():
            specs += part.tensor_specs()
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.bind(tensors)
        self.bound = True

    @property
    def graph_safe(self) -> bool:
        def walk(part):
            yield part
            for sub in part.sub_parts():
                yield from walk(sub)

        return all(p.graph_safe for top in self.parts() for p in walk(top))

    # ------------------------------------------------------------------ cache needs

    def cache_needs(self) -> list:
        """Per run entry: the cache its mixer needs, or None (also for a borrowing entry)."""
        needs = []
        for entry in self.plan.order:
            if entry.cache_of is not None:
                needs.append(None)
            else:
                needs.append(self.blocks[entry.layer].mixer_part().cache_spec())
        return needs

    # ------------------------------------------------------------------ one step

    def forward(self, step, cache, layer_hook=None, add_hook=None) -> Optional[torch.Tensor]:
        """Runs the rows of ``step`` through every run entry; returns float32 logits
        ``[len(step.want_rows), vocab]`` or None when no row is wanted.

        ``layer_hook(position, stream)`` is called after the embedding (position -1) and after
        every run entry; ``stream_value(stream)`` gives the residual rows at that point.
        ``add_hook(stream)`` is called whenever a part leaves its output on the stream (after the
        mixer and after the feed-forward of a block).  Both are diagnostics: they synchronise,
        so a step with a hook is never captured."""
        if not self.bound:
            raise RuntimeError("the model has no weights yet: load or bind them first")
        stream = Stream(self.embedding.forward(step), add_hook)
        if layer_hook is not None:
            layer_hook(-1, stream)
        for pos, entry in enumerate(self.plan.order):
            if entry.cache_of is None:
                view = cache.view(pos)
            else:
                view = cache.view(entry.cache_of, owner=False)
            self.blocks[entry.layer].forward(stream, step, view)
            if layer_hook is not None:
                layer_hook(pos, stream)
        if step.num_wanted == 0:
            return None
        if getattr(step, "wants_every_row", False):
            # every row in order (a decode step): the norm that closes the last block is the final norm
            # (handed over unevaluated to a head that says it takes that: its product may apply the row scale itself)
            return self.head.forward(stream.normed(self.final_norm, deferred=getattr(self.head, "takes_deferred_norm", False)))
        rows = step.want_rows
        delta = stream.take_pending()
        if delta is not None:
            normed = self.final_norm.add_apply(stream.residual, delta, rows)
        else:
            normed = self.final_norm.apply(self.env.ops.gather_rows(stream.residual, rows))
        return self.head.forward(normed)
