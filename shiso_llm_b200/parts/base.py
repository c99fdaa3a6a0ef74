"""Interfaces of the parts a model is put together from, and their registries.

A part is built from a ``PartSpec`` (its sizes and constants) and a ``BuildEnv``
(compute dtype, device, the kernel table).  It lists the tensors it needs, is
handed them by name after loading, says what cache it needs, and runs on the
rows of one step.  No part knows which model it is in.

Kinds of part and what each must provide:

``Norm``             ``apply(x)``, ``add_apply(residual, delta, rows=None)``, optional ``add_apply_linear``
``PositionEncoding`` ``rotary()`` - the per-pair frequencies the fused kernel rotates by
``Mixer``            ``cache_spec()``, ``forward(x, step, cache)`` -> tensor or ``DeferredLinear``
``FeedForward``      ``forward(x, step)`` -> tensor or ``DeferredLinear``
                     (both: ``takes_deferred_norm = True`` to get ``x`` as a ``DeferredNorm``)
``Block``            ``forward(stream, step, cache)`` - the arrangement of the above
``Embedding``        ``forward(step)`` -> float32 residual rows
``Head``             ``forward(x)`` -> float32 logits
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from ..weights.spec import TensorSpec
from .plan import PartSpec


@dataclass
class BuildEnv:
    """What every part needs to know about where it runs."""

    dtype: torch.dtype  # compute dtype: activations between kernels, 16-bit weights
    device: torch.device
    ops: Any  # the kernel table (shiso_llm_b200.kernels.ops, or a stand-in in CPU tests)

    def empty(self, shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


# --------------------------------------------------------------------------- cache needs


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every position, in pages.  ``window`` = how many of the most
    recent positions are ever read again (None: all of them).  Values may have another width
    than keys (``v_head_dim``; None: the same), and the entry may ask for an element type of
    its own (``dtype``; None: the engine's compute type)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    dtype: Optional[torch.dtype] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class FixedState:
    """Per-request state of fixed size, zero for a new request; float32 unless the entry asks
    for another element type."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        return self.numel * self.dtype.itemsize


# --------------------------------------------------------------------------- part classes


class Part:
    """Common protocol: tensors wanted, tensors bound.

    ``graph_safe``: the part's launches depend on the step only through device arrays
    (positions, tables, slots), never through host values that change from step to step,
    so a captured decode step can be replayed.  A part that loops on the host over the
    step's sequences sets it to False and its model runs decode steps without graphs."""

    graph_safe = True

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receives every loaded tensor by name; keep what ``tensor_specs`` named."""

    def sub_parts(self) -> list["Part"]:
        return []


class Norm(Part):
    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """Normalises float32 rows ``x[T, size]``; returns compute-dtype rows."""
        raise NotImplementedError

    def add_apply(self, residual: torch.Tensor, delta: torch.Tensor, rows: Optional[torch.Tensor] = None):
        """``residual += delta`` (float32, in place) and returns norm(residual).

        With ``rows`` (int32 row numbers) only those rows are summed and normalised,
        into a ``[len(rows), size]`` result, and ``residual`` is left untouched."""
        raise NotImplementedError


class PositionEncoding(Part):
    # Which two elements of a head form rotation pair i: False - (i, i + rotary_dim/2), the
    # half-split pairing; True - the neighbours (2i, 2i + 1).
    interleaved = False

    def rotary(self):
        """``(inv_freq, rotary_dim)``: the encoding rotates pair i of every query and key head
        (see ``interleaved``) by the angle ``position * inv_freq[i]`` (float32
        ``[rotary_dim / 2]`` on the device); ``(None, 0)`` leaves heads as they are.
        The fused norm + rotate + store kernel applies it."""
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self):
        """``PagedKV``, ``FixedState`` or ``None``."""
        return None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        """``x[T, hidden]`` (compute dtype, already normalised) -> mixer output ``[T, hidden]``.

        ``cache`` is this run entry's view of the cache (``PagedKVView`` or
        ``FixedStateView``), or ``None``; ``cache.owner`` is False when the entry
        borrows another entry's cache and must not write it."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, step) -> torch.Tensor:
        """Float32 residual rows ``[T, hidden]`` for ``step.token_ids``."""
        raise NotImplementedError

    def table(self) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``x[R, hidden]`` (compute dtype) -> float32 logits ``[R, vocab]``.  A head that sets
        ``takes_deferred_norm = True`` may be handed a ``DeferredNorm`` and starts with ``project``."""
        raise NotImplementedError


class DeferredLinear:
    """A block's output projection that has not run yet: ``x @ w^T``.

    A mixer or feed-forward may return this instead of a tensor; the stream then runs the
    product together with the residual add and the next norm when the norm can
    (``Norm.add_apply_linear``), which for decode-sized steps is one launch instead of two.
    ``materialize()`` runs it on its own."""

    def __init__(self, ops, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype):
        self.ops, self.x, self.w, self.out_dtype = ops, x, w, out_dtype

    def materialize(self) -> torch.Tensor:
        return self.ops.linear(self.x, self.w, self.out_dtype)


class DeferredNorm:
    """The normed rows a mixer or feed-forward is about to read, not computed yet:
    ``norm(residual + pending)`` of a stream.

    A part that sets ``takes_deferred_norm = True`` is handed this instead of a tensor and
    starts with ``project(ops, x, w, ...)``.  Where the block output waiting to be added is a
    product (``DeferredLinear``), the norm is an RMS norm and the kernel table has the pair
    ``linear_into_stream`` / ``linear_scaled`` (a handful of rows), the two products run with
    nothing between them: the first adds into the stream and leaves unscaled rows, the second
    applies the row scale.  Else the norm runs first, as it always did.  ``materialize()``
    gives the rows themselves."""

    def __init__(self, stream: "Stream", norm: Norm):
        self.stream, self.norm = stream, norm

    def materialize(self) -> torch.Tensor:
        return self.stream.normed(self.norm)

    def _scaled_rows(self):
        """The rows without their scale (``ScaledRows`` of the kernel table) when the block output
        waiting to be added is a product that the table can send straight into the stream;
        else None, and nothing has happened."""
        stream, norm = self.stream, self.norm
        ops = norm.env.ops
        waiting = stream.pending
        into_stream = getattr(ops, "linear_into_stream", None)
        params = norm.rms_params() if hasattr(norm, "rms_params") else None
        if isinstance(waiting, DeferredLinear) and into_stream is not None and params is not None:
            result = into_stream(waiting.x, waiting.w, stream.residual, params[0], params[1])
            if result is not None:
                stream.residual, rows = result
                stream.pending = None
                return rows
        return None

    def linear(self, w: torch.Tensor, out_dtype: torch.dtype, glu: bool = False) -> torch.Tensor:
        ops = self.norm.env.ops
        rows = self._scaled_rows()
        if rows is not None:
            return ops.linear_scaled(rows, w, out_dtype, glu)  # this product scales the rows by itself
        x = self.stream.normed(self.norm)
        return ops.linear_swiglu(x, w, out_dtype) if glu else ops.linear(x, w, out_dtype)

    def linear_short_conv(self, in_proj: torch.Tensor, taps, bias, state, step) -> torch.Tensor:
        """``ops.linear_short_conv`` of these rows (the input projection of a gated short
        convolution and the convolution behind it)."""
        ops = self.norm.env.ops
        rows = self._scaled_rows()
        return ops.linear_short_conv(rows if rows is not None else self.stream.normed(self.norm), in_proj, taps, bias, state, step)


def project(ops, x, w: torch.Tensor, out_dtype: torch.dtype, glu: bool = False) -> torch.Tensor:
    """``x @ w^T`` (or SwiGLU over the gate/up pair ``w``) for rows ``x`` that are a tensor or a
    ``DeferredNorm``."""
    if isinstance(x, DeferredNorm):
        return x.linear(w, out_dtype, glu)
    return ops.linear_swiglu(x, w, out_dtype) if glu else ops.linear(x, w, out_dtype)


class Stream:
    """The residual stream between blocks.

    ``residual`` is float32 ``[T, hidden]``.  ``pending`` is a block output not yet
    added: the next norm adds it while it normalises (one fused kernel), which is how
    the reference closes every block (crates/shiso-engine/src/layers.rs:2476-2498)."""

    def __init__(self, residual: torch.Tensor, observer: Optional[Callable] = None):
        self.residual = residual
        self.pending: Optional[torch.Tensor] = None
        self.observer = observer  # a diagnostic: called with the stream after every ``add``

    def normed(self, norm: Norm, deferred: bool = False):
        """The normed rows; with ``deferred`` a ``DeferredNorm`` that computes them when (and how)
        its reader wants."""
        if deferred:
            return DeferredNorm(self, norm)
        if self.pending is None:
            return norm.apply(self.residual)
        delta, self.pending = self.pending, None
        if isinstance(delta, DeferredLinear):
            fused = getattr(norm, "add_apply_linear", None)
            if fused is not None:
                return fused(self.residual, delta)
            delta = delta.materialize()
        return norm.add_apply(self.residual, delta)

    def take_pending(self) -> Optional[torch.Tensor]:
        """The block output still waiting to be added, as a tensor (or None)."""
        delta, self.pending = self.pending, None
        if isinstance(delta, DeferredLinear):
            delta = delta.materialize()
        return delta

    def add(self, delta) -> None:
        if self.pending is not None:
            raise RuntimeError("a block output is already waiting to be added to the residual")
        self.pending = delta
        if self.observer is not None:
            self.observer(self)


class Block(Part):
    def mixer_part(self) -> Mixer:
        raise NotImplementedError

    def forward(self, stream: Stream, step, cache) -> None:
        raise NotImplementedError


# --------------------------------------------------------------------------- registries


class Registry:
    """Name -> factory(spec, env, ...) for one kind of part."""

    def __init__(self, what: str):
        self.what = what
        self._factories: dict[str, Callable] = {}

    def register(self, kind: str, factory: Callable = None):
        def add(f):
            if kind in self._factories:
                raise ValueError(f"{self.what} {kind!r} is registered already")
            self._factories[kind] = f
            return f

        return add if factory is None else add(factory)

    def unregister(self, kind: str) -> None:
        self._factories.pop(kind, None)

    def build(self, spec: PartSpec, env: BuildEnv, *args, **kwargs):
        factory = self._factories.get(spec.kind)
        if factory is None:
            raise KeyError(
                f"no {self.what} named {spec.kind!r}; registered: {', '.join(sorted(self._factories))}"
            )
        return factory(spec, env, *args, **kwargs)

    def kinds(self) -> list[str]:
        return sorted(self._factories)


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
