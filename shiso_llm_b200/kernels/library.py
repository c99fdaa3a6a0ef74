"""Loads the kernel library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded, or no CUDA device is
present, ``library()`` raises and every op with it.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

from .build import BuildError, library_path

_LIB = None

P = c_void_p
I = c_int
F = c_float
LL = c_longlong

_SIGNATURES = {
    "shiso_embed": [P, P, P, P, I, P, I, I, I, P],
    "shiso_gather_rows": [P, P, P, I, I, P],
    "shiso_rmsnorm": [P, P, P, P, P, I, I, I, F, P],
    "shiso_swiglu": [P, P, I, I, I, P],
    "shiso_gemm_simple": [P, I, P, I, P, P, I, I, I, I, P],
    "shiso_gemm_tcgen05": [P, P, P, P, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_tokens64": [P, P, P, P, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_swiglu": [P, P, P, I, I, I, I, P],
    "shiso_gemm_tcgen05_prompt": [P, P, P, P, I, I, I, I, I, I, P],
    "shiso_prefill_attention_tc_supported": [I, I],
    "shiso_prefill_attention_tc": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, LL, F, I, P],
    "shiso_gemm_tcgen05_pair": [P, P, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_supported": [I, P, P],
    "shiso_gemm_tcgen05_fused_max_tokens": [],
    "shiso_gemm_tcgen05_into_partial_rows": [I],
    "shiso_gemm_tcgen05_into": [P, P, P, P, P, P, P, P, I, I, I, I, P],
    "shiso_gemm_tcgen05_scaled": [P, P, I, I, F, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_pair_scaled": [P, P, I, I, F, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_prompt_scaled": [P, P, I, I, F, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_status": [],
    "shiso_gemm_stream": [P, P, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_stream_into": [P, P, P, P, P, P, P, P, I, I, I, I, P],
    "shiso_gemm_stream_scaled": [P, P, I, F, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_stream_conv": [P, P, I, F, P, P, P, P, LL, P, P, P, I, I, I, I, I, I, P],
    "shiso_short_conv": [P, I, P, P, P, LL, P, P, P, P, I, I, I, I, I, I, P],
    "shiso_qk_norm_rope_store": [P, I, P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "shiso_paged_attention": [P, I, P, P, P, I, P, P, P, I, I, I, I, I, F, I, P],
    "shiso_decode_attention": [P, P, P, P, I, P, P, P, P, I, I, I, I, I, F, I, I, P],
    "shiso_decode_attention_fused_supported": [I, I, I, I],
    "shiso_decode_attention_fused_max_parts": [],
    "shiso_decode_attention_fused": [P, P, P, P, I, P, P, P, I, I, I, I, I, LL, F, I, I, P],
    "shiso_decode_attention_from_qkv": [P, P, P, P, F, P, P, P, I, P, P, P, I, I, I, I, I, LL, F, I, I, I, P],
    "shiso_prefill_attention": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, P],
    "shiso_argmax": [P, P, I, I, P, P],
    "shiso_argmax_chunked": [P, P, P, I, I, I, P, P],
    "shiso_sample": [P, P, P, P, P, P, P, P, I, I, P, P],
    "shiso_suppress": [P, P, P, I, I, I, P],
    "shiso_copy_words": [P, P, I, I, P],
    "shiso_selftest_bounded_wait": [LL, P],
}


class KernelLibraryError(RuntimeError):
    pass


def library():
    global _LIB
    if _LIB is not None:
        return _LIB
    try:
        path = library_path()
    except BuildError as e:
        raise KernelLibraryError(f"the CUDA kernels are required and could not be built: {e}") from e
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise KernelLibraryError(f"the CUDA kernel library {path} could not be loaded: {e}") from e
    for name, argtypes in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise KernelLibraryError(f"{path} does not export {name}; rebuild it") from e
        fn.argtypes = argtypes
        fn.restype = c_int
    _LIB = lib
    return lib


def declare(name: str, argtypes) -> None:
    """Declares one more entry point (used by kernels added in their own files)."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None:
        fn = getattr(_LIB, name)
        fn.argtypes = argtypes
        fn.restype = c_int
