"""The kernel table: one Python function per CUDA kernel, launched on the current stream.

Every function checks shapes, types, contiguity and device, then calls the C launcher
with raw pointers.  Nothing here computes on the CPU and nothing calls a library
routine for the model's arithmetic; if the extension cannot be loaded the first call
raises.  Inputs must be CUDA tensors.
"""

from __future__ import annotations

from typing import Optional

import torch

from .library import KernelLibraryError, library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

# How many kernels were launched through this table (bench.py reports it).
launch_count = 0


class KernelError(RuntimeError):
    pass


_ERRORS = {
    1001: "unsupported element type",
    1002: "unsupported shape",
    1003: "misaligned pointer or stride",
    1004: "unsupported combination",
}


def require() -> None:
    """Loads the extension now, or raises with the reason."""
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device: this engine has no CPU path")
    library()


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_DEVICE_INDEX = None  # the one device this process's kernel library works on, once bound


def resolve_binding(wanted_index, bound_index, current_index) -> int:
    """Which device an engine asked for ends up on, or the refusal.  ``wanted_index`` is the
    index the caller named (None for a bare "cuda"), ``bound_index`` the device the library is
    bound to already (None: not yet), ``current_index`` the process's current device."""
    index = current_index if wanted_index is None else wanted_index
    if bound_index is not None and index != bound_index:
        raise KernelError(
            f"this process's kernel library works on cuda:{bound_index} (attributes of its kernels and its status word "
            f"live there); an engine on cuda:{index} needs a process of its own"
        )
    return index


def bind_device(device) -> int:
    """Binds the kernel library to ``device`` (a torch.device of type cuda) and makes it the
    current device; returns its index.  The library keeps per-process state for one device -
    which kernels were given their shared-memory attribute, the status word of the bounded
    waits - and every launch goes to the current device's
    stream, so all engines of a process share one device; another one is refused here, before
    a pointer of one device could reach a kernel on another."""
    global _DEVICE_INDEX
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"the CUDA kernels cannot run on {device}")
    index = resolve_binding(device.index, _DEVICE_INDEX, torch.cuda.current_device())
    if index >= torch.cuda.device_count():
        raise KernelError(f"cuda:{index} does not exist: this process sees {torch.cuda.device_count()} device(s)")
    torch.cuda.set_device(index)
    _DEVICE_INDEX = index
    return index


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch (a graph capture changes it), so
    through torch's raw binding where it exists: the public call costs 13 us of Python per launch,
    a third of a kernel-by-kernel step's host time."""
    global _DEVICE_INDEX
    if _RAW_STREAM is None:
        return torch.cuda.current_stream().cuda_stream
    if _DEVICE_INDEX is None:
        _DEVICE_INDEX = torch.cuda.current_device()
    return _RAW_STREAM(_DEVICE_INDEX)


def _check(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor, got one on {t.device}")
    if not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name}: expected {ndim} dimensions, got shape {tuple(t.shape)}")


_region = None  # the open profile region, if any (kernels/profile.py)
_plain_library = library


class _TimedLibrary:
    """The kernel library while a region is open: an event is recorded before every call."""

    def __init__(self, lib):
        self._lib = lib

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not name.startswith("shiso_"):
            return fn

        def call(*args):
            if _region is not None:
                _region.before()
            return fn(*args)

        return call


def profile_start() -> None:
    """Opens a region: until ``profile_stop`` every launch stands between two events."""
    global _region, library
    from .profile import Region

    if _region is not None:
        raise KernelError("a profile region is already open")
    require()
    timed = _TimedLibrary(_plain_library())
    library = lambda: timed  # noqa: E731
    _region = Region(torch)


def profile_stop():
    """Closes the region: ((kernel, shape, launches, microseconds) in launch order, host
    microseconds, microseconds from the first launch's start to the last one's end)."""
    global _region, library
    if _region is None:
        raise KernelError("no profile region is open")
    region, _region = _region, None
    library = _plain_library
    return region.close()


def _done(status: int, what: str, launches: int = 1, shape=()) -> None:
    global launch_count
    if status != 0:
        why = _ERRORS.get(status)
        if why is None:
            why = f"CUDA error {status} at launch"
        raise KernelError(f"{what}: {why} (status {status})")
    launch_count += launches
    if _region is not None:
        _region.mark(what, "x".join(str(int(d)) for d in shape), launches)


# --------------------------------------------------------------------------- rows


def embed(ids: torch.Tensor, table: torch.Tensor, feed_index=None, fed_tokens=None) -> torch.Tensor:
    """Rows of ``table`` for ``ids``.  Where ``feed_index[t] >= 0`` the id is read on the device
    from ``fed_tokens[feed_index[t]]`` instead (a token picked a step earlier that the host has
    not seen)."""
    _check(ids, "ids", torch.int32, 1)
    _check(table, "embedding table", None, 2)
    tokens, (vocab, hidden) = ids.shape[0], table.shape
    if (feed_index is None) != (fed_tokens is None):
        raise KernelError("embed: feed_index and fed_tokens come together")
    if feed_index is not None:
        _check(feed_index, "feed_index", torch.int32, 1)
        _check(fed_tokens, "fed_tokens", torch.int32, 1)
        if feed_index.shape[0] != tokens:
            raise KernelError(f"feed_index has {feed_index.shape[0]} entries for {tokens} rows")
    out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    status = library().shiso_embed(
        _ptr(ids), _ptr(feed_index), _ptr(fed_tokens), _ptr(table), _code(table), _ptr(out), tokens, hidden, vocab, _stream()
    )
    _done(status, "embed", shape=(tokens, hidden))
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _check(x, "x", torch.float32, 2)
    _check(rows, "rows", torch.int32, 1)
    out = torch.empty((rows.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
    _done(library().shiso_gather_rows(_ptr(x), _ptr(rows), _ptr(out), rows.shape[0], x.shape[1], _stream()), "gather_rows")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    return add_rmsnorm(x, None, w, eps, out_dtype, None)


def add_rmsnorm(residual, delta, w, eps, out_dtype, rows=None):
    """``residual`` float32 [T, H]; ``delta`` [T, H] in the output type or None; returns
    norm(residual + delta).  Without ``rows`` the sum is stored back into ``residual``."""
    _check(residual, "residual", torch.float32, 2)
    _check(w, "norm weight", torch.float32, 1)
    tokens, hidden = residual.shape
    if w.shape[0] != hidden:
        raise KernelError(f"norm weight has {w.shape[0]} entries for rows of {hidden}")
    if delta is not None:
        _check(delta, "delta", out_dtype, 2)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match the residual {tuple(residual.shape)}")
    out_rows = tokens
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        out_rows = rows.shape[0]
    out = torch.empty((out_rows, hidden), dtype=out_dtype, device=residual.device)
    status = library().shiso_rmsnorm(
        _ptr(residual), _ptr(delta), _ptr(rows), _ptr(w), _ptr(out), _code(out), out_rows, hidden, float(eps), _stream()
    )
    _done(status, "rmsnorm" if delta is None else "add + rmsnorm", shape=(out_rows, hidden))
    return out


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    _check(gate_up, "gate_up", None, 2)
    tokens, two_inter = gate_up.shape
    if two_inter % 2:
        raise KernelError(f"gate_up rows of {two_inter} cannot be split in two halves")
    out = torch.empty((tokens, two_inter // 2), dtype=gate_up.dtype, device=gate_up.device)
    _done(library().shiso_swiglu(_ptr(gate_up), _ptr(out), _code(gate_up), tokens, two_inter // 2, _stream()), "swiglu")
    return out


# --------------------------------------------------------------------------- matrix products


_SM_COUNT = None
PROMPT_MIN_TOKENS = 193  # from here the persistent tensor-memory kernels (tokens as the MMA's M operand): plain products on pairs of SMs; below, 64-token tiles with K split over a cluster are faster
# Portions of a few hundred rows times a matrix of few rows: the kernel for long portions would have a
# handful of 256 x 256 tiles for 74 pairs of SMs and walk a long K alone.  Up to FEW_PAIR_TILES such
# tiles, and while tiles of 128 features x 64 tokens stay within the CTAs that are resident at once, the
# product runs as those tiles on single SMs with K split over a cluster (576 rows: 2048 x 5632 31.2 ->
# 22.2 us, 2048 x 2048 14.9 -> 12.3 us, 3072 x 2048 17.2 -> 14.6 us; 1024 x 4608 at 512 rows 26.2 -> 12.5 us;
# 6144 x 2048 at 512 rows would lose, 18.0 -> 28.2 us, and is left where it was).
FEW_PAIR_TILES = 36
FEW_TILES_MAX_TOKENS = 1024
PAIR_MIN_TOKENS_GLU = 512  # gate/up pairs below this stay on single SMs: the pairs' 256-token tiles would leave a second, nearly empty wave


def _sm_count() -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _SM_COUNT


STREAM_KERNEL_MAX_TOKENS = 8  # up to here the persistent weight-streaming kernel runs the product (9..16 rows measured slower there than in the tensor-memory kernel)


def _few_pair_tiles(tokens: int, n: int) -> bool:
    """Whether a plain bfloat16 product of this shape runs as token tiles of 64 in the kernel for
    few rows rather than as 256 x 256 tiles on SM pairs (the rule stands at FEW_PAIR_TILES)."""
    return (
        PROMPT_MIN_TOKENS <= tokens <= FEW_TILES_MAX_TOKENS
        and -(-tokens // 256) * -(-n // 256) <= FEW_PAIR_TILES and -(-tokens // 64) * -(-n // 128) <= 2 * _sm_count()
    )


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[T, K] @ w[N, K]^T`` with float accumulation.

    bfloat16 x bfloat16 runs on the tensor cores (tcgen05, accumulators in TMEM); the true
    32-bit path and mixed types run the CUDA-core kernel, whose rows do not depend on the
    batch."""
    _check(x, "x", None, 2)
    _check(w, "w", None, 2)
    tokens, k = x.shape
    n, k2 = w.shape
    if k != k2:
        raise KernelError(f"x has rows of {k}, the matrix has rows of {k2}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    out = torch.empty((tokens, n), dtype=out_dtype, device=x.device)
    lib = library()
    both_bf16 = x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if both_bf16 and k % 8 == 0 and tokens <= STREAM_KERNEL_MAX_TOKENS:
        status = lib.shiso_gemm_stream(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, 0, _sm_count(), _stream()
        )
        _done(status, "linear (streaming)", shape=(tokens, n, k))
        return out
    if both_bf16 and _few_pair_tiles(tokens, n) and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        status = lib.shiso_gemm_tcgen05_tokens64(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, _sm_count(), _stream()
        )
        _done(status, "linear (tcgen05, token tiles of 64)", shape=(tokens, n, k))
        return out
    if both_bf16 and tokens >= PROMPT_MIN_TOKENS and n % 8 == 0 and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        status = lib.shiso_gemm_tcgen05_pair(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, 0, _sm_count(), _stream()
        )
        _done(status, "linear (tcgen05, persistent)", shape=(tokens, n, k))
        return out
    if both_bf16 and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        status = lib.shiso_gemm_tcgen05(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, _sm_count(), _stream()
        )
        _done(status, "linear (tcgen05)", shape=(tokens, n, k))
        return out
    status = lib.shiso_gemm_simple(
        _ptr(x), _code(x), _ptr(w), _code(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, _stream()
    )
    _done(status, "linear", shape=(tokens, n, k))
    return out


def linear_swiglu(x: torch.Tensor, gate_up: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``silu(x @ gate^T) * (x @ up^T)`` for ``gate_up = [gate; up]`` of shape ``[2I, K]``.
    In bfloat16 the activation is applied in the product's epilogue (the streaming kernel for a
    handful of rows, the tensor-memory kernel with two accumulators otherwise); other types
    run the product and then the activation kernel."""
    _check(x, "x", None, 2)
    _check(gate_up, "gate_up", None, 2)
    tokens, k = x.shape
    two_inter = gate_up.shape[0]
    if two_inter % 2 or gate_up.shape[1] != k:
        raise KernelError(f"gate/up matrix of shape {tuple(gate_up.shape)} does not fit rows of {k}")
    if (
        x.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and out_dtype == torch.bfloat16
        and tokens <= STREAM_KERNEL_MAX_TOKENS and k % 8 == 0
    ):
        out = torch.empty((tokens, two_inter // 2), dtype=out_dtype, device=x.device)
        status = library().shiso_gemm_stream(
            _ptr(x), _ptr(gate_up), 0, _ptr(out), _code(out), tokens, two_inter, k, two_inter // 2,
            _sm_count(), _stream(),
        )
        _done(status, "linear_swiglu (streaming)", shape=(tokens, two_inter, k))
        return out
    lib = library()
    if (
        x.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16
        and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(gate_up))
    ):
        out = torch.empty((tokens, two_inter // 2), dtype=out_dtype, device=x.device)
        if tokens >= PROMPT_MIN_TOKENS and (two_inter // 2) % 8 == 0:
            product = lib.shiso_gemm_tcgen05_pair if tokens >= PAIR_MIN_TOKENS_GLU else lib.shiso_gemm_tcgen05_prompt
            status = product(
                _ptr(x), _ptr(gate_up), 0, _ptr(out), _code(out), tokens, two_inter // 2, k, two_inter // 2,
                _sm_count(), _stream(),
            )
            _done(status, "linear_swiglu (tcgen05, persistent)", shape=(tokens, two_inter, k))
            return out
        status = lib.shiso_gemm_tcgen05_swiglu(
            _ptr(x), _ptr(gate_up), _ptr(out), _code(out), tokens, two_inter // 2, k, _stream()
        )
        _done(status, "linear_swiglu (tcgen05)", shape=(tokens, two_inter, k))
        return out
    return swiglu(linear(x, gate_up, out_dtype))


STREAM_MAX_TOKENS = 8  # rows for which the weight-streaming kernel runs the product-into-stream / scaled-product pair
GLU_ONE_TILE_MAX_TOKENS = 64  # above one token tile the scaled gate/up pair runs as a plain product and the activation kernel: a gate/up CTA has an SM to itself, so two token tiles are 88 CTAs that each walk the whole K (20.9 us at 128 rows of the 1.2B shape against 17.8 us; decode at batch 96 / 128 +3.2 / +2.0 %)
FUSED_NORM_MAX_TOKENS = 192  # up to here (all the rows it takes) the tensor-memory kernel (tokens as the MMA's N operand) runs the pair: decode at batch 9 / 16 / 32 / 64 gained 11 / 10 / 4 / 1 % over product + norm kernel when the pair was built, batch 80 / 96 / 128 gain 4.2 / 4.2 / 3.6 % since a warp finishes whole tokens of the split products


class ScaledRows:
    """Rows that still lack their RMS scale: ``x`` is bfloat16 ``(residual * norm weight)`` and
    ``partials[c, t]`` are sums of squares of token ``t`` whose total over ``c`` gives the mean
    square.  ``linear_scaled`` applies the scale after its product."""

    def __init__(self, x, partials, eps):
        self.x, self.partials, self.eps = x, partials, float(eps)


def linear_into_stream(x, w, residual, next_norm_w, eps, bias=None):
    """A block's output projection, the residual add and the first half of the next RMS norm in
    one launch, for up to 192 bfloat16 rows and for the products of a few hundred rows that run
    as token tiles of 64 (``_few_pair_tiles``): returns ``(residual + x @ w^T, ScaledRows)`` -
    ``residual`` (float32 ``[T, N]``) itself is not changed - or None when sizes or types are
    not the ones the kernels take.  A handful of rows run in the weight-streaming kernel, more
    in the tensor-memory kernel whose threads own a feature each, so that a warp reads and
    writes neighbouring values of a token's row.  (The product into the stream in the
    tensor-memory kernels for long prompts was measured slower than product + row kernel:
    there a thread owns a row, and its strided reads and writes of the stream cost more than
    the row kernel they replace.  Applying the row scale is one factor a thread there, so those
    kernels do take the rows this one leaves: ``linear_scaled``.)"""
    tokens, k = x.shape
    n = w.shape[0]
    if (
        x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or residual.dtype != torch.float32
        or k % 8 or w.shape[1] != k or n % 8
        or (tokens > FUSED_NORM_MAX_TOKENS and not _few_pair_tiles(tokens, n))
    ):
        return None
    lib = library()
    streaming = tokens <= min(STREAM_MAX_TOKENS, STREAM_KERNEL_MAX_TOKENS)
    if not streaming and not lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        return None
    _check(x, "x", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    _check(residual, "residual", torch.float32, 2)
    _check(next_norm_w, "norm weight", torch.float32, 1)
    if residual.shape != (tokens, n) or next_norm_w.shape[0] != n:
        raise KernelError(f"a residual of shape {tuple(residual.shape)} beside a product of {tokens} x {n}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    summed = torch.empty_like(residual)
    rows = torch.empty((tokens, n), dtype=torch.bfloat16, device=x.device)
    if streaming:
        partials = torch.empty((-(-n // 16), 16), dtype=torch.float32, device=x.device)
        status = lib.shiso_gemm_stream_into(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(summed), _ptr(next_norm_w), _ptr(rows), _ptr(partials),
            tokens, n, k, _sm_count(), _stream(),
        )
    else:
        partials = torch.empty((lib.shiso_gemm_tcgen05_into_partial_rows(n), tokens), dtype=torch.float32, device=x.device)
        status = lib.shiso_gemm_tcgen05_into(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(summed), _ptr(next_norm_w), _ptr(rows), _ptr(partials),
            tokens, n, k, _sm_count(), _stream(),
        )
    _done(status, "linear_into_stream" + (" (streaming)" if streaming else " (tcgen05)"), shape=(tokens, n, k))
    return summed, ScaledRows(rows, partials, eps)


def linear_scaled(rows: ScaledRows, w, out_dtype, glu=False):
    """``rmsnorm(..) @ w^T`` (SwiGLU over the gate/up pair ``w`` when ``glu``) for rows that
    ``linear_into_stream`` left: the row scale is applied to the accumulators."""
    x = rows.x
    _check(x, "x", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    tokens, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or (glu and n % 2):
        raise KernelError(f"a matrix of shape {tuple(w.shape)} for rows of {k}")
    if tokens > FUSED_NORM_MAX_TOKENS:
        return _linear_scaled_long(rows, w, out_dtype, glu)
    if glu and tokens > GLU_ONE_TILE_MAX_TOKENS and out_dtype == torch.bfloat16 and (n // 2) % 8 == 0:
        return swiglu(linear_scaled(rows, w, out_dtype, False))
    inter = n // 2 if glu else 0
    out = torch.empty((tokens, inter if glu else n), dtype=out_dtype, device=x.device)
    lib = library()
    if tokens <= min(STREAM_MAX_TOKENS, STREAM_KERNEL_MAX_TOKENS):
        status = lib.shiso_gemm_stream_scaled(
            _ptr(x), _ptr(rows.partials), rows.partials.shape[0], rows.eps, _ptr(w), _ptr(out), _code(out),
            tokens, n, k, inter, _sm_count(), _stream(),
        )
    else:
        status = lib.shiso_gemm_tcgen05_scaled(
            _ptr(x), _ptr(rows.partials), rows.partials.shape[0], rows.partials.shape[1], rows.eps, _ptr(w), _ptr(out),
            _code(out), tokens, n, k, inter, _sm_count(), _stream(),
        )
    _done(status, "linear_scaled", shape=(tokens, n, k))
    return out


def _linear_scaled_long(rows: ScaledRows, w, out_dtype, glu):
    """``linear_scaled`` for more than 192 rows: the kernel ``linear`` / ``linear_swiglu`` would
    take for the shape, with the row scale in its epilogue."""
    x = rows.x
    tokens, k = x.shape
    n = w.shape[0]
    lib = library()
    partials = rows.partials
    if n % 8 or k % 8 or (glu and (n // 2) % 8):
        # widths the prompt kernels do not take: the kernel for up to 192 rows takes any, a
        # slice of the rows at a time (the partial sums' columns are the tokens)
        out = torch.empty((tokens, n // 2 if glu else n), dtype=out_dtype, device=x.device)
        stride = partials.shape[1]
        for first in range(0, tokens, FUSED_NORM_MAX_TOKENS):
            count = min(FUSED_NORM_MAX_TOKENS, tokens - first)
            status = lib.shiso_gemm_tcgen05_scaled(
                _ptr(x[first : first + count]), partials.data_ptr() + 4 * first, partials.shape[0], stride, rows.eps, _ptr(w),
                _ptr(out[first : first + count]), _code(out), count, n, k, n // 2 if glu else 0, _sm_count(), _stream(),
            )
            _done(status, "linear_scaled (a slice of the rows)", shape=(count, n, k))
        return out
    if glu:
        inter = n // 2
        out = torch.empty((tokens, inter), dtype=out_dtype, device=x.device)
        product = lib.shiso_gemm_tcgen05_pair_scaled if tokens >= PAIR_MIN_TOKENS_GLU else lib.shiso_gemm_tcgen05_prompt_scaled
        status = product(_ptr(x), _ptr(partials), partials.shape[0], partials.shape[1], rows.eps, _ptr(w), _ptr(out), _code(out),
                         tokens, inter, k, inter, _sm_count(), _stream())
        _done(status, "linear_scaled + swiglu (tcgen05, persistent)", shape=(tokens, n, k))
        return out
    out = torch.empty((tokens, n), dtype=out_dtype, device=x.device)
    if _few_pair_tiles(tokens, n) and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        status = lib.shiso_gemm_tcgen05_scaled(
            _ptr(x), _ptr(partials), partials.shape[0], partials.shape[1], rows.eps, _ptr(w), _ptr(out), _code(out),
            tokens, n, k, 0, _sm_count(), _stream(),
        )
        _done(status, "linear_scaled (tcgen05, token tiles of 64)", shape=(tokens, n, k))
        return out
    status = lib.shiso_gemm_tcgen05_pair_scaled(
        _ptr(x), _ptr(partials), partials.shape[0], partials.shape[1], rows.eps, _ptr(w), _ptr(out), _code(out),
        tokens, n, k, 0, _sm_count(), _stream(),
    )
    _done(status, "linear_scaled (tcgen05, persistent)", shape=(tokens, n, k))
    return out


def linear_add_rmsnorm(x, w, residual, norm_w, eps, out_dtype):
    """A block's output projection, the residual add and the next RMS norm:
    ``residual += x @ w^T`` (float32, in place) and returns ``rmsnorm(residual) * norm_w``.
    Two launches: the product, then the fused add + norm row kernel.  (One launch, with the
    CTA that finishes last normalising, was measured at 10.5 us against 6.1 us for the pair
    in a dependent-launch chain and was dropped.)"""
    return add_rmsnorm(residual, linear(x, w, out_dtype), norm_w, eps, out_dtype)


CONV_FUSED_MAX_TAPS = 4  # taps the weight-streaming kernel's convolution epilogue takes


def linear_short_conv(x, in_proj, taps, bias, state, step):
    """The short conv's input projection followed by the gated convolution; ``x`` is a tensor or
    ``ScaledRows``.  For a handful of bfloat16 rows, one per sequence, the convolution runs in
    the product's epilogue (a tile of the weight-streaming kernel is then the B, C and x rows of
    five channels); else the product and the convolution kernel run one after the other."""
    rows = x if isinstance(x, ScaledRows) else None
    xt = rows.x if rows is not None else x
    tokens, k = xt.shape
    hidden, n_taps = taps.shape
    if (
        xt.dtype == torch.bfloat16 and in_proj.dtype == torch.bfloat16 and tokens <= STREAM_KERNEL_MAX_TOKENS
        and getattr(step, "all_decode", False) and 2 <= n_taps <= CONV_FUSED_MAX_TAPS and k % 8 == 0
    ):
        _check(xt, "x", torch.bfloat16, 2)
        _check(in_proj, "in_proj", torch.bfloat16, 2)
        _check(taps, "conv taps", torch.float32, 2)
        if in_proj.shape != (3 * hidden, k):
            raise KernelError(f"an input projection of shape {tuple(in_proj.shape)} for {hidden} channels of rows of {k}")
        if state.dtype != torch.float32 or not state.is_cuda or state.dim() != 3:
            raise KernelError("conv state: expected a float32 CUDA tensor [slots, taps-1, hidden]")
        if state.shape[1:] != (n_taps - 1, hidden) or state.stride(2) != 1 or state.stride(1) != hidden:
            raise KernelError(f"conv state of shape {tuple(state.shape)} / strides {state.stride()} does not fit {n_taps} taps x {hidden}")
        if bias is not None:
            _check(bias, "conv bias", torch.float32, 1)
        y = torch.empty((tokens, hidden), dtype=xt.dtype, device=xt.device)
        status = library().shiso_gemm_stream_conv(
            _ptr(xt), _ptr(rows.partials) if rows is not None else 0, rows.partials.shape[0] if rows is not None else 0,
            rows.eps if rows is not None else 0.0, _ptr(in_proj), _ptr(taps), _ptr(bias), state.data_ptr(), state.stride(0),
            _ptr(step.seq_of_token), _ptr(step.state_slots), _ptr(y), _code(y), tokens, hidden, k, n_taps,
            _sm_count(), _stream(),
        )
        _done(status, "linear_short_conv (streaming)", shape=(tokens, 3 * hidden, k))
        return y
    proj = linear_scaled(rows, in_proj, xt.dtype) if rows is not None else linear(xt, in_proj, xt.dtype)
    return short_conv(proj, taps, bias, state, step)


def linear_simple(x, w, out_dtype, bias=None):
    """The CUDA-core product for any element types (used by tests to compare kernels)."""
    _check(x, "x", None, 2)
    _check(w, "w", None, 2)
    out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    status = library().shiso_gemm_simple(
        _ptr(x), _code(x), _ptr(w), _code(w), _ptr(bias), _ptr(out), _code(out), x.shape[0], w.shape[0], x.shape[1], _stream()
    )
    _done(status, "linear")
    return out


CARRIES_STATUS = True  # argmax and sample take ``status_out``
GAVE_UP = "a kernel gave up waiting on a barrier; what it wrote is not valid"


def check_kernel_status() -> None:
    """Raises when a bounded wait inside a kernel ran out since the status word was last read
    (here, or by a token-picking kernel that was given a place for it).  Synchronises the
    device; not for use while a stream is being captured."""
    status = library().shiso_gemm_tcgen05_status()
    if status != 0:
        raise KernelError(f"{GAVE_UP} (status {status})")


def selftest_bounded_wait(limit_cycles: int = 4000) -> None:
    """Launches one CTA that waits ``limit_cycles`` clock cycles on a barrier nobody arrives at
    and then gives up, as any kernel here does when a wait runs out: the status word is set and
    the kernel returns.  For tests of what the host does then."""
    _done(library().shiso_selftest_bounded_wait(int(limit_cycles), _stream()), "selftest_bounded_wait")


# --------------------------------------------------------------------------- short convolution


def short_conv(proj, taps, bias, state, step):
    """``proj[T, 3H]`` -> ``y[T, H]``; ``state`` is the float32 view ``[slots, taps-1, H]`` of
    the slot buffer (rows of one slot contiguous) and is updated for the step's sequences."""
    _check(proj, "proj", None, 2)
    _check(taps, "conv taps", torch.float32, 2)
    tokens, h3 = proj.shape
    hidden, n_taps = taps.shape
    if h3 != 3 * hidden:
        raise KernelError(f"proj rows of {h3} are not 3 x {hidden}")
    if state.dtype != torch.float32 or not state.is_cuda or state.dim() != 3:
        raise KernelError("conv state: expected a float32 CUDA tensor [slots, taps-1, hidden]")
    if state.shape[1:] != (n_taps - 1, hidden) or state.stride(2) != 1 or state.stride(1) != hidden:
        raise KernelError(f"conv state of shape {tuple(state.shape)} / strides {state.stride()} does not fit {n_taps} taps x {hidden}")
    if bias is not None:
        _check(bias, "conv bias", torch.float32, 1)
    y = torch.empty((tokens, hidden), dtype=proj.dtype, device=proj.device)
    status = library().shiso_short_conv(
        _ptr(proj), _code(proj), _ptr(taps), _ptr(bias), state.data_ptr(), state.stride(0),
        _ptr(step.seq_of_token), _ptr(step.q_start), _ptr(step.state_slots), _ptr(y),
        tokens, step.num_seqs, hidden, n_taps, 1, int(getattr(step, "max_q_len", 0)), _stream(),
    )
    _done(status, "short_conv", 2, shape=(tokens, hidden))
    return y


# --------------------------------------------------------------------------- attention


def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_w, k_w, eps, inv_freq, rotary_dim, step,
                       k_cache, v_cache, block_table, page_size, store, interleaved=False):
    """Per-head norm, rotation and cache store.  The rotation pairs are ``(i, i + rotary_dim/2)``,
    or neighbours ``(2i, 2i + 1)`` with ``interleaved``."""
    _check(qkv, "qkv", None, 2)
    tokens, width = qkv.shape
    if width != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qkv rows of {width} are not ({heads} + 2 x {kv_heads}) x {head_dim}")
    for name, t in (("q norm weight", q_w), ("k norm weight", k_w)):
        if t is not None:
            _check(t, name, torch.float32, 1)
            if t.shape[0] != head_dim:
                raise KernelError(f"{name} has {t.shape[0]} entries for heads of {head_dim}")
    if rotary_dim:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError(f"inv_freq has {inv_freq.shape[0]} entries for a rotation over {rotary_dim}")
    _check(block_table, "block table", torch.int32, 2)
    do_store = bool(store) and kv_heads > 0
    if do_store:
        for name, t in (("k cache", k_cache), ("v cache", v_cache)):
            _check(t, name, qkv.dtype, 4)
            if t.shape[1:] != (page_size, kv_heads, head_dim):
                raise KernelError(f"{name} of shape {tuple(t.shape)} does not fit pages of {page_size} x {kv_heads} x {head_dim}")
    q = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    status = library().shiso_qk_norm_rope_store(
        _ptr(qkv), _code(qkv), _ptr(q_w), _ptr(k_w), _ptr(inv_freq) if rotary_dim else 0,
        _ptr(step.positions), _ptr(step.seq_of_token), _ptr(block_table), block_table.shape[1],
        _ptr(k_cache) if do_store else 0, _ptr(v_cache) if do_store else 0, _ptr(q),
        tokens, heads, kv_heads, head_dim, int(rotary_dim), page_size, float(eps), int(do_store), int(bool(interleaved)),
        _stream(),
    )
    _done(status, "qk_norm_rope_store", shape=(tokens, heads + 2 * kv_heads, head_dim))
    return q


MAX_DECODE_GROUP = 16  # query heads per KV head the decode kernel serves from one read (rows of one MMA tile)
DECODE_HEAD_DIMS = tuple(range(16, 129, 16))  # larger head sizes take the general kernel
PREFILL_MAX_HEAD_DIM = 128  # the tiled prompt kernel keeps a row's output in registers
TC_ATTENTION_MIN_TOKENS = 256  # steps from here on, with a portion of at least ...
TC_ATTENTION_MIN_PORTION = 128  # ... this many rows, take the tensor-memory attention kernel (head size 64)


_WIDE_CLUSTERS = None


def _wide_clusters() -> bool:
    """Whether the fused decode kernel may be launched as clusters of 16 CTAs on this device."""
    global _WIDE_CLUSTERS
    if _WIDE_CLUSTERS is None:
        _WIDE_CLUSTERS = int(library().shiso_decode_attention_fused_max_parts()) >= 16
    return _WIDE_CLUSTERS


def decode_splits(tokens: int, kv_heads: int, capacity: int, fused: bool = False) -> int:
    """Into how many parts a decode kernel cuts a sequence's keys.  It depends on the launch
    shape only, never on current lengths, so a captured step stays valid.  The two-launch
    kernel wants enough CTAs (tokens x KV heads x parts) to fill the SMs a few times over, no
    part shorter than 128 keys of the table's capacity.  The fused kernel streams a long part
    at full rate through its ring, and every CTA costs it a start and a hand-over at the end:
    it wants one wave of the two CTAs an SM holds (measured when three fitted: batch 8 x 8 KV
    heads x 2,190 keys took 14.8 us in 4 parts, 16.5 in 6, 21 in 10; batch 32 30 us whole, 43 in 2)."""
    if fused:
        # the parts of a (sequence, KV head) are a thread-block cluster: at most 8, or 16 where the
        # device places such clusters and one or two sequences leave room for them (a part of two
        # tiles instead of four: batch 1 x 2,158 keys)
        room = 2 * _sm_count() // (tokens * kv_heads)
        most = 16 if room >= 16 and _wide_clusters() else 8
        return max(1, min(most, room, -(-capacity // 128)))
    return max(1, min(16, -(-4 * _sm_count() // (tokens * kv_heads)), -(-capacity // 128)))


DECODE_FROM_QKV_MAX_TOKENS = 64  # rows up to which attention takes the qkv rows itself: one launch fewer per layer, and the keys and values move before the predecessor ends (batch 8 / 16 / 32 / 64 decode 1 / 1.8 / 2.0 / 1.0 % faster; no change at 96 and 128 rows)


def decode_attention_from_qkv(qkv, heads, kv_heads, head_dim, q_w, k_w, eps, inv_freq, rotary_dim, step,
                              k_cache, v_cache, block_table, page_size, store, scale, window, interleaved=False):
    """``qk_norm_rope_store`` and ``paged_attention`` in one launch for steps of single tokens:
    the attention kernel takes the rows of the qkv product, norms and rotates the queries and
    each token's new key itself, and (with ``store``) writes the new key and value into the
    caches, with the bits ``qk_norm_rope_store`` would write.  bfloat16, heads of 64 rotated
    whole, both norms present, a handful of rows; None when the step or the sizes are others (the
    caller then runs the two kernels)."""
    lib = library()
    if (
        qkv.shape[0] > DECODE_FROM_QKV_MAX_TOKENS or qkv.dtype != torch.bfloat16 or not getattr(step, "all_decode", False) or q_w is None or k_w is None
        or interleaved
        or inv_freq is None or head_dim != 64 or rotary_dim != 64 or kv_heads <= 0
        or not lib.shiso_decode_attention_fused_supported(heads, kv_heads, head_dim, page_size)
    ):
        return None
    _check(qkv, "qkv", torch.bfloat16, 2)
    tokens, width = qkv.shape
    if width != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qkv rows of {width} are not ({heads} + 2 x {kv_heads}) x {head_dim}")
    for name, t in (("k cache", k_cache), ("v cache", v_cache)):
        _check(t, name, torch.bfloat16, 4)
        if t.shape[1:] != (page_size, kv_heads, head_dim):
            raise KernelError(f"{name} of shape {tuple(t.shape)} does not fit pages of {page_size} x {kv_heads} x {head_dim}")
    _check(block_table, "block table", torch.int32, 2)
    _check(q_w, "q norm weight", torch.float32, 1)
    _check(k_w, "k norm weight", torch.float32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    if q_w.shape[0] != head_dim or k_w.shape[0] != head_dim or inv_freq.shape[0] != rotary_dim // 2:
        raise KernelError("norm weights of the head size and one frequency per rotated pair are expected")
    out = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    splits = decode_splits(tokens, kv_heads, block_table.shape[1] * page_size, True)
    status = lib.shiso_decode_attention_from_qkv(
        _ptr(qkv), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), float(eps), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
        block_table.shape[1], _ptr(step.positions), _ptr(step.seq_of_token), _ptr(out),
        tokens, heads, kv_heads, head_dim, page_size, k_cache.shape[0], float(scale), int(window), splits, int(bool(store)),
        _stream(),
    )
    _done(status, "decode_attention_from_qkv", shape=(tokens, heads, head_dim))
    return out


def paged_attention(q, heads, kv_heads, head_dim, k_cache, v_cache, block_table, page_size, scale, window, step,
                    general=False):
    """Attention of every row over its sequence's cache.  Steps of single tokens in bfloat16
    take the split-key decode kernel (keys and values read once per KV head); other bfloat16
    steps take the tiled tensor-core kernel; float32 and head sizes above 128 take the general
    kernel.  ``general=True`` forces the general kernel (tests compare the routes)."""
    _check(q, "q", None, 2)
    tokens = q.shape[0]
    if q.shape[1] != heads * head_dim:
        raise KernelError(f"q rows of {q.shape[1]} are not {heads} x {head_dim}")
    for name, t in (("k cache", k_cache), ("v cache", v_cache)):
        _check(t, name, q.dtype, 4)
        if t.shape[1:] != (page_size, kv_heads, head_dim):
            raise KernelError(f"{name} of shape {tuple(t.shape)} does not fit pages of {page_size} x {kv_heads} x {head_dim}")
    _check(block_table, "block table", torch.int32, 2)
    out = torch.empty_like(q)
    lib = library()
    if general:
        pass
    elif (
        q.dtype == torch.bfloat16 and getattr(step, "all_decode", False)
        and heads // kv_heads <= MAX_DECODE_GROUP and head_dim in DECODE_HEAD_DIMS
    ):
        fused = bool(lib.shiso_decode_attention_fused_supported(heads, kv_heads, head_dim, page_size))
        splits = decode_splits(tokens, kv_heads, block_table.shape[1] * page_size, fused)
        if fused:
            # keys and values by TMA, the parts merged through their cluster's shared memory: one launch
            status = lib.shiso_decode_attention_fused(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.positions),
                _ptr(step.seq_of_token), _ptr(out), tokens, heads, kv_heads, head_dim,
                page_size, k_cache.shape[0], float(scale), int(window), splits, _stream(),
            )
            _done(status, "decode_attention (fused)", shape=(tokens, heads, head_dim))
            return out
        scratch = torch.empty((tokens * heads * splits * (head_dim + 2),), dtype=torch.float32, device=q.device)
        status = lib.shiso_decode_attention(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.positions),
            _ptr(step.seq_of_token), _ptr(scratch), _ptr(out), tokens, heads, kv_heads, head_dim, page_size,
            float(scale), int(window), splits, _stream(),
        )
        _done(status, "decode_attention", 2, shape=(tokens, heads, head_dim))
        return out
    elif (
        q.dtype == torch.bfloat16 and tokens >= TC_ATTENTION_MIN_TOKENS
        and getattr(step, "max_q_len", tokens) >= TC_ATTENTION_MIN_PORTION
        and lib.shiso_prefill_attention_tc_supported(head_dim, page_size)
    ):
        # long portions: products in tensor memory, 128 query rows per CTA
        starts = getattr(step, "h_q_start", None)
        if starts:
            tiles = sum(-(-(b - a) // 128) for a, b in zip(starts[:-1], starts[1:]))
        else:
            tiles = tokens // 128 + step.num_seqs
        status = lib.shiso_prefill_attention_tc(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.q_start),
            _ptr(step.start_pos), _ptr(out), tokens, step.num_seqs, tiles, heads, kv_heads, page_size,
            k_cache.shape[0], float(scale), int(window), _stream(),
        )
        _done(status, "prefill_attention (tcgen05)", shape=(tokens, heads, head_dim))
        return out
    elif q.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= PREFILL_MAX_HEAD_DIM:
        starts = getattr(step, "h_q_start", None)
        if starts:
            tiles = sum(-(-(b - a) // 64) for a, b in zip(starts[:-1], starts[1:]))
        else:
            tiles = tokens // 64 + step.num_seqs
        status = lib.shiso_prefill_attention(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.q_start),
            _ptr(step.start_pos), _ptr(out), step.num_seqs, tiles, heads, kv_heads, head_dim, page_size,
            float(scale), int(window), _stream(),
        )
        _done(status, "prefill_attention", shape=(tokens, heads, head_dim))
        return out
    status = lib.shiso_paged_attention(
        _ptr(q), _code(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(step.positions), _ptr(step.seq_of_token), _ptr(out), tokens, heads, kv_heads, head_dim,
        page_size, float(scale), int(window), _stream(),
    )
    _done(status, "paged_attention", shape=(tokens, heads, head_dim))
    return out


# --------------------------------------------------------------------------- sampling


def _picks(out, rows, device):
    if out is None:
        return torch.empty((rows,), dtype=torch.int32, device=device)
    _check(out, "out", torch.int32, 1)
    if out.shape[0] != rows:
        raise KernelError(f"out has {out.shape[0]} entries for {rows} rows")
    return out


def _status_place(status_out) -> int:
    if status_out is None:
        return 0
    _check(status_out, "status_out", torch.int32, 1)
    if status_out.shape[0] != 1:
        raise KernelError("status_out is one int32")
    return status_out.data_ptr()


def suppress(logits: torch.Tensor, rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Sets ``logits[rows[i], ids[i]]`` to -inf, in place, before a pick
    (crates/shiso-engine/src/sampling.rs:156-174; kernels/cuda/sample/sample.cu:18-26)."""
    _check(logits, "logits", torch.float32, 2)
    _check(rows, "rows", torch.int32, 1)
    _check(ids, "ids", torch.int32, 1)
    if rows.shape != ids.shape:
        raise KernelError(f"{rows.shape[0]} rows for {ids.shape[0]} ids")
    _done(library().shiso_suppress(_ptr(logits), _ptr(rows), _ptr(ids), rows.shape[0], logits.shape[0], logits.shape[1],
                                   _stream()), "suppress")
    return logits


def words_to_host(src: torch.Tensor, host: torch.Tensor) -> bool:
    """``host[:n] = src`` for int32 ``src`` on the device and pinned ``host``, as a kernel in the
    stream that stores into the host's memory in place: a step's tokens reach the host without a
    turn of the copy engine between two kernels (decode at batch 8 loses 2 to 3 % to that turn).
    The host reads them after an event, as after a copy.  False when the device cannot address
    the memory; the caller then copies."""
    _check(src, "src", torch.int32, 1)
    if host.is_cuda or host.dtype != torch.int32 or not host.is_contiguous() or not host.is_pinned() or host.numel() < src.numel():
        return False
    status = library().shiso_copy_words(_ptr(src), host.data_ptr(), src.numel(), 2, _stream())
    if status == 1004:  # memory the device cannot address
        return False
    _done(status, "words_to_host", shape=(src.numel(),))
    return True


def words_from_host(host: torch.Tensor, dst: torch.Tensor) -> bool:
    """``dst = host[:n]`` for pinned int32 ``host`` and ``dst`` on the device, as a kernel in the
    stream that loads from the host's memory in place (a step's few KB of positions and block
    tables).  The host may write the buffer again after an event that follows, as after a copy.
    False when the device cannot address the memory; the caller then copies."""
    _check(dst, "dst", torch.int32, 1)
    if host.is_cuda or host.dtype != torch.int32 or not host.is_contiguous() or not host.is_pinned() or host.numel() < dst.numel():
        return False
    status = library().shiso_copy_words(host.data_ptr(), _ptr(dst), dst.numel(), 1, _stream())
    if status == 1004:  # memory the device cannot address
        return False
    _done(status, "words_from_host", shape=(dst.numel(),))
    return True


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, status_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The index of each row's largest value (the smallest index among equals), int32, written
    to ``out`` when one is given.  ``status_out`` (one int32) receives the status word of the
    bounded waits, which is cleared: see ``check_kernel_status``."""
    _check(logits, "logits", torch.float32, 2)
    rows, vocab = logits.shape
    out = _picks(out, rows, logits.device)
    status = _status_place(status_out)
    if vocab >= 8192:
        # chunks of at least 1,024 values; no more blocks (rows x chunks)
        # than a few waves: 64 rows x 64 chunks of four values a thread took 13.6 us for 17 MB
        chunks = max(1, min(128, -(-vocab // 1024), -(-4 * _sm_count() // rows)))
        scratch = torch.empty((2 * rows * chunks,), dtype=torch.float32, device=logits.device)
        code = library().shiso_argmax_chunked(_ptr(logits), _ptr(out), _ptr(scratch), rows, vocab, chunks, status, _stream())
        _done(code, "argmax", 2)
        return out
    _done(library().shiso_argmax(_ptr(logits), _ptr(out), rows, vocab, status, _stream()), "argmax")
    return out


def sample(logits, temperature, top_k, top_p, min_p, keys, positions, out=None, status_out=None) -> torch.Tensor:
    """Keyed sampling, one row per request: float32 ``temperature``/``top_p``/``min_p``,
    int32 ``top_k`` (0 = off) and ``positions``, int64 ``keys``, all of length rows.
    ``status_out`` as in ``argmax``."""
    _check(logits, "logits", torch.float32, 2)
    rows = logits.shape[0]
    for name, t, dt in (
        ("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
        ("keys", keys, torch.int64), ("positions", positions, torch.int32),
    ):
        _check(t, name, dt, 1)
        if t.shape[0] != rows:
            raise KernelError(f"{name} has {t.shape[0]} entries for {rows} rows")
    out = _picks(out, rows, logits.device)
    status = library().shiso_sample(
        _ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(keys), _ptr(positions),
        _ptr(out), rows, logits.shape[1], _status_place(status_out), _stream(),
    )
    _done(status, "sample")
    return out
