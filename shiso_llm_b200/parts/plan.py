"""The description of a model as data: which parts, with which sizes, in which order.

An architecture's builder turns its typed configuration into a ``ModelPlan``.
Nothing below the plan knows the architecture's name: every part is chosen by
a ``PartSpec`` (a registry key plus parameters), layer by layer, so one model
may hold different mixers and feed-forwards in different layers.  The run
order is data as well (``ModelPlan.order``): an entry names the layer whose
weights run and the run-order position whose cache it reads, so a layer may run
twice (shared weights, each run with a cache of its own) or read the cache an
earlier entry wrote.

The reference keeps the same facts in ``HybridShape`` with one ``LayerKind``
per slot and one ``AttnLayer`` geometry per attention slot
(crates/shiso-engine/src/shape.rs:36-53,99-194,426-493).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: the registry key that builds it and the parameters it gets."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer's parts.  ``name`` prefixes the layer's tensor names.

    ``block`` chooses the arrangement (how norms, mixer, feed-forward and the
    residual stream are wired); the other specs are handed to that block.
    """

    name: str
    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None


@dataclass(frozen=True)
class RunEntry:
    """One position of the run order.

    ``layer`` indexes ``ModelPlan.layers`` (whose weights run here).
    ``cache_of`` is the run-order position whose cache this entry reads and
    writes; ``None`` means its own.  An entry that names another position reads
    that position's cache and stores nothing.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    """Everything the generic model needs to assemble itself."""

    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple[int, ...] = ()
    max_position: Optional[int] = None
    # A portion of a prompt that is not the request's last must be a multiple of this many tokens,
    # so that every portion starts on that grid: what a mixer needs whose recurrence is evaluated
    # in chunks of fixed length (the reference cuts on such a grid for its chunked delta-net,
    # crates/shiso-runtime/src/scheduler/config.rs:35-44).  1: a portion may end anywhere.
    portion_multiple: int = 1
    # Names of further int32 arrays, one value per row, that parts of this model read from the
    # step (``step.extras[name]``) beside token ids and positions: more position streams, segment
    # ids and the like (the reference keeps such arrays in its batch metadata,
    # crates/shiso-engine/src/attn.rs:244-284).  A caller gives them per entry
    # (``StepEntry.extras``); a row for which none is given gets its position.
    row_inputs: tuple[str, ...] = ()

    def __post_init__(self):
        if self.portion_multiple < 1:
            raise ValueError(f"portion_multiple = {self.portion_multiple} must be at least 1")
        if not self.order:
            raise ValueError("a model plan needs at least one run entry")
        for pos, entry in enumerate(self.order):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"run entry {pos} names layer {entry.layer}, which does not exist")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < pos:
                    raise ValueError(
                        f"run entry {pos} reads the cache of entry {entry.cache_of}: "
                        "only an earlier entry can have written it"
                    )
                if self.order[entry.cache_of].cache_of is not None:
                    raise ValueError(
                        f"run entry {pos} reads the cache of entry {entry.cache_of}, "
                        "which itself borrows a cache; name the owner"
                    )


def sequential_order(n_layers: int) -> tuple[RunEntry, ...]:
    """Every layer once, in index order, each with a cache of its own."""
    return tuple(RunEntry(layer=i) for i in range(n_layers))
