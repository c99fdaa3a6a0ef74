"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called the way
an embedder would call it: through its exported C symbol, with raw device pointers.

Some hosts of this library cannot give a kernel scratch memory: they have handed all device
memory to a pool of their own, or they sit on a path where the device-wide synchronisation of
cudaMalloc is not acceptable.  For them the partial results live in a fixed array inside the
library.  The test runs the entry point twice in a row (the second call with other sizes, so
it meets the first call's leftovers in the shared array) and compares each result with the
ordinary entry point, which takes its scratch from the caller, and with the plain attention
of ``fake_kernels`` (the reference the ordinary entry point is itself tested against, so
that the two entry points cannot be wrong together); and it checks that a call too large
for the array is refused with a clear message and launches nothing.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It passes alone in a fresh process and after the other tests.
"""

import ctypes
import math
from types import SimpleNamespace

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = 1005
ARRAY_FLOATS = 1 << 20


def load():
    from shiso_llm_b200.kernels.build import library_path

    lib = ctypes.CDLL(library_path())
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.shiso_decode_attention_no_alloc.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, P]
    lib.shiso_decode_attention_no_alloc.restype = I
    lib.shiso_decode_attention.argtypes = [P, P, P, P, I, P, P, P, P, I, I, I, I, I, F, I, I, P]
    lib.shiso_decode_attention.restype = I
    lib.shiso_no_alloc_last_error.argtypes = []
    lib.shiso_no_alloc_last_error.restype = ctypes.c_char_p
    return lib


def problem(seed, lengths, heads, kv_heads, d, page):
    g = torch.Generator().manual_seed(seed)
    n = len(lengths)
    blocks = [-(-length // page) for length in lengths]
    num_pages = sum(blocks) + 2
    order = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((n, max(blocks)), -1, dtype=torch.int32)
    for i, b in enumerate(blocks):
        for j in range(b):
            table[i, j] = order.pop()
    k = torch.randn(num_pages, page, kv_heads, d, generator=g).to(torch.bfloat16)
    v = torch.randn(num_pages, page, kv_heads, d, generator=g).to(torch.bfloat16)
    q = torch.randn(n, heads * d, generator=g).to(torch.bfloat16)
    return SimpleNamespace(
        q=q.cuda(), k=k.cuda(), v=v.cuda(), table=table.cuda(),
        positions=torch.tensor([length - 1 for length in lengths], dtype=torch.int32).cuda(),
        seq=torch.arange(n, dtype=torch.int32).cuda(), n=n, heads=heads, kv_heads=kv_heads, d=d, page=page,
    )


def run(lib, p, splits, window, static):
    out = torch.full_like(p.q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    common_head = (p.q.data_ptr(), p.k.data_ptr(), p.v.data_ptr(), p.table.data_ptr(), p.table.shape[1],
                   p.positions.data_ptr(), p.seq.data_ptr())
    common_tail = (out.data_ptr(), p.n, p.heads, p.kv_heads, p.d, p.page, 1.0 / math.sqrt(p.d), window, splits, stream)
    if static:
        status = lib.shiso_decode_attention_no_alloc(*common_head, *common_tail)
    else:
        scratch = torch.empty(p.n * p.heads * splits * (p.d + 2), dtype=torch.float32, device="cuda")
        status = lib.shiso_decode_attention(*common_head, scratch.data_ptr(), *common_tail)
    torch.cuda.synchronize()
    return status, out


def agree(got, want):
    # the tolerance of the kernel tests: one bfloat16 unit in the last place at the largest value
    assert torch.isfinite(got).all()
    scale = want.float().abs().max().item()
    assert (got.float() - want.float()).abs().max().item() <= 2 ** -7 * scale


def plain(p, window):
    """The same attention by ``fake_kernels.paged_attention`` (float64 on the CPU)."""
    import fake_kernels

    step = SimpleNamespace(seq_of_token=p.seq.cpu(), positions=p.positions.cpu())
    return fake_kernels.paged_attention(p.q.cpu(), p.heads, p.kv_heads, p.d, p.k.cpu(), p.v.cpu(), p.table.cpu(), p.page,
                                        1.0 / math.sqrt(p.d), window, step)


def test_two_calls_in_a_row_match_the_entry_point_with_caller_scratch():
    lib = load()
    first = problem(1, [700, 1, 16, 2100, 33], heads=8, kv_heads=2, d=64, page=16)
    second = problem(2, [5, 300], heads=3, kv_heads=1, d=32, page=4)
    for p, splits, window in ((first, 9, 0), (second, 4, 50), (first, 3, 0)):
        status, got = run(lib, p, splits, window, static=True)
        assert status == 0, lib.shiso_no_alloc_last_error()
        status, want = run(lib, p, splits, window, static=False)
        assert status == 0
        agree(got, want)
        agree(got.cpu(), plain(p, window))


def test_a_call_beyond_the_array_is_refused_and_launches_nothing():
    lib = load()
    p = problem(3, [40] * 64, heads=32, kv_heads=8, d=64, page=16)
    splits = 32
    assert p.n * p.heads * splits * (p.d + 2) > ARRAY_FLOATS
    status, out = run(lib, p, splits, 0, static=True)
    assert status == TOO_LARGE
    message = lib.shiso_no_alloc_last_error().decode()
    assert str(p.n * p.heads * splits * (p.d + 2)) in message and str(ARRAY_FLOATS) in message
    assert torch.isnan(out.float()).all(), "a refused call must not write its output"
    status, got = run(lib, p, 2, 0, static=True)  # the same problem with fewer parts fits
    assert status == 0 and lib.shiso_no_alloc_last_error() == b""
    agree(got, run(lib, p, 2, 0, static=False)[1])
