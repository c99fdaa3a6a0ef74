"""Every CUDA kernel alone against its plain PyTorch reference (tests/fake_kernels.py),
at sizes other than the engine tests use: widths that are no power of two, head sizes in
steps of 16, odd numbers of heads and groups, several sequences per launch, pages out of
order, non-zero starting states.
"""

import math
from types import SimpleNamespace

import pytest
import torch

import fake_kernels as ref

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from shiso_llm_b200.kernels import ops as table

    table.require()
    return table


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(got, want, dtype, what, rel32=2e-6, scale=None, slack=0.0):
    """``slack`` is added to the relative bound (times the scale): the share of an error source
    that grows with something else than the values, such as a rotation angle's rounding."""
    got, want = got.double().cpu(), want.double().cpu()
    s = scale if scale is not None else max(want.abs().max().item(), 1e-6)
    err = (got - want).abs().max().item()
    rel32 = rel32 + slack
    # bfloat16: both sides round their result to bfloat16, so where the unrounded values
    # straddle a rounding boundary they differ by one unit in the last place, which is between
    # 2^-8 and 2^-7 of the value; one such unit at the largest value is the bound.
    bound = rel32 * s if dtype == torch.float32 else 2 ** -7 * s
    assert err <= bound, f"{what}: error {err:.3e} > {bound:.3e} (scale {s:.3e})"


def make_step(q_lens, starts, page_size, num_pages, seed, num_slots=None, device="cuda"):
    """Step metadata with shuffled, non-contiguous pages for each sequence."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    S = len(q_lens)
    width = max(-(-(s + n) // page_size) for s, n in zip(starts, q_lens))
    table = torch.full((S, width), -1, dtype=torch.int32)
    for i, (s, n) in enumerate(zip(starts, q_lens)):
        need = -(-(s + n) // page_size)
        for b in range(need):
            table[i, b] = perm.pop()
    q_start = [0]
    for n in q_lens:
        q_start.append(q_start[-1] + n)
    pos, seq = [], []
    for i, (s, n) in enumerate(zip(starts, q_lens)):
        pos += list(range(s, s + n))
        seq += [i] * n
    slots = torch.randperm(num_slots or S, generator=g)[:S].to(torch.int32)

    def dev(x):
        return torch.as_tensor(x, dtype=torch.int32).to(device)

    cpu = SimpleNamespace(
        num_tokens=q_start[-1], num_seqs=S, positions=dev(pos).cpu(), seq_of_token=dev(seq).cpu(),
        q_start=dev(q_start).cpu(), state_slots=slots, start_pos=dev(starts).cpu(),
    )
    gpu = SimpleNamespace(
        num_tokens=q_start[-1], num_seqs=S, positions=dev(pos), seq_of_token=dev(seq),
        q_start=dev(q_start), state_slots=slots.to(device), start_pos=dev(starts),
    )
    return cpu, gpu, table


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    table = rnd((777, 200), dtype, 1)
    ids = torch.tensor([0, 776, 5, 5, 300], dtype=torch.int32)
    got = ops().embed(ids.cuda(), table.cuda())
    assert torch.equal(got.cpu(), ref.embed(ids, table))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [96, 200, 2048, 5000])
def test_rmsnorm_and_fused_add(dtype, hidden):
    x = rnd((7, hidden), torch.float32, 2, 3.0)
    delta = rnd((7, hidden), dtype, 3)
    w = 1.0 + 0.2 * rnd((hidden,), torch.float32, 4)
    eps = 1e-6
    close(ops().rmsnorm(x.cuda(), w.cuda(), eps, dtype), ref.rmsnorm(x, w, eps, dtype), dtype, "rmsnorm")
    res_gpu, res_cpu = x.clone().cuda(), x.clone()
    got = ops().add_rmsnorm(res_gpu, delta.cuda(), w.cuda(), eps, dtype)
    want = ref.add_rmsnorm(res_cpu, delta, w, eps, dtype)
    close(got, want, dtype, "add_rmsnorm")
    assert torch.equal(res_gpu.cpu(), res_cpu), "the stored sum must be the float32 sum"
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    res_gpu2 = x.clone().cuda()
    got = ops().add_rmsnorm(res_gpu2, delta.cuda(), w.cuda(), eps, dtype, rows.cuda())
    want = ref.add_rmsnorm(x.clone(), delta, w, eps, dtype, rows)
    close(got, want, dtype, "add_rmsnorm rows")
    assert torch.equal(res_gpu2.cpu(), x), "with rows the residual is left alone"
    close(ops().gather_rows(x.cuda(), rows.cuda()), ref.gather_rows(x, rows), torch.float32, "gather_rows", rel32=0.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    gu = rnd((9, 2 * 300), dtype, 5, 2.0)
    close(ops().swiglu(gu.cuda()), ref.swiglu(gu), dtype, "swiglu")


@pytest.mark.parametrize("shape", [(1, 96, 64), (5, 1000, 96), (67, 130, 257), (130, 65, 48)])
@pytest.mark.parametrize("xw", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_linear(shape, xw):
    T, N, K = shape
    xd, wd = xw
    x, w = rnd((T, K), xd, 6), rnd((N, K), wd, 7, 0.05)
    for out_dtype in (xd, torch.float32):
        got = ops().linear(x.cuda(), w.cuda(), out_dtype)
        close(got, ref.linear(x, w, out_dtype), out_dtype, f"linear {shape} {xw} -> {out_dtype}", rel32=1e-5)


@pytest.mark.parametrize("shape", [(512, 256, 64), (700, 1000, 264), (1030, 2048, 2048), (2048, 6144, 512), (515, 520, 5632),
                                   (193, 2048, 2048), (300, 776, 520), (600, 2048, 8192), (257, 16384, 2048)])
def test_linear_on_sm_pairs(shape, monkeypatch):
    """From 193 bfloat16 rows a plain product runs on pairs of SMs (one 256-row tile per pair, each CTA
    loading half of both operands): row counts that leave the second CTA of the last pair with
    few or no rows, feature counts that leave its weight half partly or wholly outside the
    matrix, one and many k steps, more tiles than pairs; bfloat16 and float32 results, a bias."""
    from shiso_llm_b200.kernels import ops as ops_module

    monkeypatch.setattr(ops_module, "FEW_PAIR_TILES", 0)  # this kernel, also where the table would choose token tiles of 64
    T, N, K = shape
    x, w = rnd((T, K), torch.bfloat16, 140), rnd((N, K), torch.bfloat16, 141, 0.05)
    bias = rnd((N,), torch.float32, 142)
    # The tensor core rounds its float32 accumulator once per 16-wide k block, so the error of a
    # float32 result grows with K: 1e-5 of the largest value was fixed for K up to 5,632 and is
    # scaled from there for longer sums.
    rel32 = 1e-5 * max(1.0, K / 5632)
    for out_dtype in (torch.bfloat16, torch.float32):
        got = ops().linear(x.cuda(), w.cuda(), out_dtype)
        ops().check_kernel_status()
        close(got, ref.linear(x, w, out_dtype), out_dtype, f"pair linear {shape} -> {out_dtype}", rel32=rel32)
    got = ops().linear(x.cuda(), w.cuda(), torch.float32, bias.cuda())
    close(got, ref.linear(x, w, torch.float32, bias), torch.float32, f"pair linear {shape} with bias", rel32=rel32)
    # the rows of a long step are those of a short one (other kernel, same sums up to rounding)
    short = ops().linear(x[:100].contiguous().cuda(), w.cuda(), torch.float32, bias.cuda())
    close(got[:100], short, torch.float32, "pair against single-SM kernel", rel32=rel32)


@pytest.mark.parametrize("shape", [(576, 2048, 5632), (512, 1024, 4608), (300, 776, 520), (1000, 1000, 264), (193, 40, 72), (768, 3072, 1024),
                                   (1024, 2048, 2048), (250, 6144, 2048), (640, 136, 8192)])
def test_linear_of_a_few_hundred_rows_on_token_tiles_of_64(shape, monkeypatch):
    """A portion of a few hundred rows times a matrix of few rows: the product runs as tiles of 128
    features x 64 tokens on single SMs, K split over clusters of 1 to 8 CTAs, instead of a handful
    of 256 x 256 tiles on pairs of SMs.  Row and feature counts that fill no tile, K of one block
    and of many, both result types, a bias; and the same rows through the kernel for long portions."""
    from shiso_llm_b200.kernels import ops as ops_module

    T, N, K = shape
    assert -(-T // 256) * -(-N // 256) <= ops_module.FEW_PAIR_TILES and T <= ops_module.FEW_TILES_MAX_TOKENS
    x, w = rnd((T, K), torch.bfloat16, 143), rnd((N, K), torch.bfloat16, 144, 0.05)
    bias = rnd((N,), torch.float32, 145)
    rel32 = 1e-5 * max(1.0, K / 5632)
    before = ops_module.launch_count
    for out_dtype in (torch.bfloat16, torch.float32):
        got = ops().linear(x.cuda(), w.cuda(), out_dtype)
        ops().check_kernel_status()
        close(got, ref.linear(x, w, out_dtype), out_dtype, f"token tiles of 64 {shape} -> {out_dtype}", rel32=rel32)
    got = ops().linear(x.cuda(), w.cuda(), torch.float32, bias.cuda())
    close(got, ref.linear(x, w, torch.float32, bias), torch.float32, f"token tiles of 64 {shape} with bias", rel32=rel32)
    assert ops_module.launch_count - before == 3
    monkeypatch.setattr(ops_module, "FEW_PAIR_TILES", 0)
    pairs = ops().linear(x.cuda(), w.cuda(), torch.float32, bias.cuda())
    close(got, pairs, torch.float32, "token tiles of 64 against SM pairs", rel32=rel32)


def test_linear_rows_do_not_depend_on_the_batch():
    x, w = rnd((70, 200), torch.float32, 8), rnd((150, 200), torch.float32, 9)
    full = ops().linear(x.cuda(), w.cuda(), torch.float32)
    one = ops().linear(x[33:34].contiguous().cuda(), w.cuda(), torch.float32)
    assert torch.equal(full[33:34], one)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,hidden,bias", [(3, 300, False), (4, 96, True), (2, 130, True), (8, 64, False)])
def test_short_conv(dtype, taps, hidden, bias):
    q_lens, starts = [4, 1, 3, 9, 2], [0, 5, 2, 0, 7]
    cpu, gpu, _ = make_step(q_lens, starts, 4, 32, 10, num_slots=7)
    T = cpu.num_tokens
    proj = rnd((T, 3 * hidden), dtype, 11)
    w = rnd((hidden, taps), torch.float32, 12)
    b = rnd((hidden,), torch.float32, 13) if bias else None
    # a slot buffer wider than this layer's state, as the cache manager lays it out
    buf = rnd((7, 50 + (taps - 1) * hidden + 9), torch.float32, 14)
    state_cpu = buf.clone()[:, 50 : 50 + (taps - 1) * hidden].unflatten(1, (taps - 1, hidden))
    buf_gpu = buf.clone().cuda()
    state_gpu = buf_gpu[:, 50 : 50 + (taps - 1) * hidden].unflatten(1, (taps - 1, hidden))
    want = ref.short_conv(proj, w, b, state_cpu, cpu)
    got = ops().short_conv(proj.cuda(), w.cuda(), b.cuda() if bias else None, state_gpu, gpu)
    close(got, want, dtype, "short_conv y", rel32=4e-6)
    # the new state is a copy of products of two stored values: exact in float32
    assert torch.allclose(state_gpu.cpu(), state_cpu, rtol=0, atol=0 if dtype == torch.float32 else 1e-7)
    untouched = torch.ones(7, dtype=torch.bool)
    untouched[cpu.state_slots.long()] = False
    assert torch.equal(buf_gpu.cpu()[untouched], buf[untouched]), "slots of other requests must not change"
    assert torch.equal(buf_gpu.cpu()[:, :50], buf[:, :50]) and torch.equal(buf_gpu.cpu()[:, -9:], buf[:, -9:])


@pytest.mark.parametrize("taps,hidden,bias", [(3, 304, False), (4, 96, True), (2, 136, True), (5, 64, True)])
def test_short_conv_long_portions(taps, hidden, bias):
    """Steps of 512 rows and more in bfloat16 walk runs of rows with the window in registers:
    sequences that start and end inside a run, one with history in its state, single rows, and
    a tap count the run kernel leaves to the per-row kernel.  Both give the same bits."""
    q_lens, starts = [7, 300, 1, 40, 250, 1, 21], [0, 5, 9, 0, 64, 3, 0]
    cpu, gpu, _ = make_step(q_lens, starts, 16, 64, 130, num_slots=9)
    T = cpu.num_tokens
    assert T >= 512
    proj = rnd((T, 3 * hidden), torch.bfloat16, 131)
    w = rnd((hidden, taps), torch.float32, 132)
    b = rnd((hidden,), torch.float32, 133) if bias else None
    start = rnd((9, taps - 1, hidden), torch.float32, 134)
    s_ref, s_gpu = start.clone(), start.clone().cuda()
    want = ref.short_conv(proj, w, b, s_ref, cpu)
    got = ops().short_conv(proj.cuda(), w.cuda(), b.cuda() if bias else None, s_gpu, gpu)
    close(got, want, torch.bfloat16, "short conv over runs")
    assert torch.allclose(s_gpu.cpu(), s_ref, rtol=0, atol=1e-7)
    # the same rows through the per-row kernel (a step of fewer than 512 rows): identical bits
    cut = q_lens[0] + q_lens[1]
    cpu2, gpu2, _ = make_step(q_lens[:2], starts[:2], 16, 64, 130, num_slots=9)
    gpu2.state_slots = gpu.state_slots[:2]
    s_two = start.clone().cuda()
    two = ops().short_conv(proj[:cut].contiguous().cuda(), w.cuda(), b.cuda() if bias else None, s_two, gpu2)
    assert torch.equal(two, got[:cut])


def test_short_conv_portions_match_whole():
    """Chunks [4, 1, 3] against one run of 8 from the same starting state."""
    hidden, taps = 300, 3
    proj = rnd((8, 3 * hidden), torch.float32, 15)
    w = rnd((hidden, taps), torch.float32, 16)
    start = rnd((1, taps - 1, hidden), torch.float32, 17)
    cpu, gpu, _ = make_step([8], [0], 4, 8, 18, num_slots=1)
    s_whole = start.clone().cuda()
    y_whole = ops().short_conv(proj.cuda(), w.cuda(), None, s_whole, gpu)
    s_cut = start.clone().cuda()
    ys, at = [], 0
    for n in (4, 1, 3):
        _, g, _ = make_step([n], [at], 4, 8, 19, num_slots=1)
        ys.append(ops().short_conv(proj[at : at + n].contiguous().cuda(), w.cuda(), None, s_cut, g))
        at += n
    assert torch.equal(torch.cat(ys), y_whole)
    assert torch.equal(s_cut, s_whole)


CASES = [  # heads, kv_heads, head_dim, page_size, rotary_dim
    (4, 2, 16, 4, 16),
    (3, 1, 32, 16, 32),
    (6, 3, 48, 8, 32),
    (5, 5, 80, 16, 80),
    (8, 2, 64, 16, 64),
    (2, 1, 256, 4, 128),
    (6, 3, 64, 8, 64),  # heads of 64 rotated whole (in bfloat16 the kernel of eight lanes per head): groups of four heads that mix kinds
    (5, 1, 64, 16, 64),
    (32, 8, 64, 16, 64),
    (4, 4, 64, 4, 32),  # heads of 64 rotated in part: the general kernel
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_norm_rope_store_then_attention(dtype, case):
    heads, kv_heads, d, page, rot = case
    q_lens, starts = [5, 1, 40, 2], [0, 37, 3, 130]
    num_pages = 64
    cpu, gpu, table = make_step(q_lens, starts, page, num_pages, 20)
    T = cpu.num_tokens
    qkv = rnd((T, (heads + 2 * kv_heads) * d), dtype, 21)
    qw = 1.0 + 0.2 * rnd((d,), torch.float32, 22)
    kw = 1.0 + 0.2 * rnd((d,), torch.float32, 23)
    theta = 10000.0
    inv_freq = (theta ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    eps = 1e-5
    # caches start filled with earlier positions' keys and values
    k0, v0 = rnd((num_pages, page, kv_heads, d), dtype, 24), rnd((num_pages, page, kv_heads, d), dtype, 25)
    kc, vc = k0.clone(), v0.clone()
    kg, vg = k0.clone().cuda(), v0.clone().cuda()
    want_q = ref.qk_norm_rope_store(qkv, heads, kv_heads, d, qw, kw, eps, inv_freq, rot, cpu, kc, vc, table, page, True)
    got_q = ops().qk_norm_rope_store(
        qkv.cuda(), heads, kv_heads, d, qw.cuda(), kw.cuda(), eps, inv_freq.cuda(), rot, gpu, kg, vg, table.cuda(), page, True
    )
    # the kernel multiplies position and frequency in float32: the angle is off by up to
    # position * 2^-24 radians (the plain reference forms it in float64), and so is the rotated value
    angle_slack = max(s + n for s, n in zip(starts, q_lens)) * 2.0 ** -24
    close(got_q, want_q, dtype, "q after norm and rotation", rel32=4e-6, slack=angle_slack)
    close(kg, kc, dtype, "k cache", rel32=4e-6, slack=angle_slack)
    assert torch.equal(vg.cpu(), vc), "values are stored raw"
    written = (kc != k0).flatten(1).any(1)
    assert torch.equal(kg.cpu()[~written], k0[~written]), "rows of other positions must not change"

    scale = 1.0 / math.sqrt(d)
    for window in (0, 7):
        want = ref.paged_attention(want_q, heads, kv_heads, d, kc, vc, table, page, scale, window, cpu)
        got = ops().paged_attention(want_q.cuda(), heads, kv_heads, d, kc.cuda(), vc.cuda(), table.cuda(), page, scale, window, gpu)
        close(got, want, dtype, f"attention window {window}", rel32=4e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [(4, 2, 16, 4, 16), (6, 3, 48, 8, 32), (8, 2, 64, 16, 64), (5, 5, 80, 16, 40), (2, 1, 24, 4, 24)])
def test_rotation_over_pairs_of_neighbours(dtype, case):
    """A position encoding may pair neighbours (2i, 2i + 1) instead of (i, i + rotary_dim / 2):
    the same kernel with the other pairing, also for bfloat16 heads of 64 (which otherwise take
    the kernel that knows the half-split pairing only) and for a head size that is no multiple
    of 16; and the two pairings differ."""
    heads, kv_heads, d, page, rot = case
    q_lens, starts = [3, 1, 9], [0, 20, 5]
    cpu, gpu, table = make_step(q_lens, starts, page, 32, 190)
    qkv = rnd((cpu.num_tokens, (heads + 2 * kv_heads) * d), dtype, 191)
    qw, kw = 1.0 + 0.2 * rnd((d,), torch.float32, 192), 1.0 + 0.2 * rnd((d,), torch.float32, 193)
    inv_freq = (10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    k0, v0 = rnd((32, page, kv_heads, d), dtype, 194), rnd((32, page, kv_heads, d), dtype, 195)
    results = {}
    for interleaved in (True, False):
        kc, vc, kg, vg = k0.clone(), v0.clone(), k0.clone().cuda(), v0.clone().cuda()
        want = ref.qk_norm_rope_store(qkv, heads, kv_heads, d, qw, kw, 1e-5, inv_freq, rot, cpu, kc, vc, table, page, True, interleaved)
        got = ops().qk_norm_rope_store(qkv.cuda(), heads, kv_heads, d, qw.cuda(), kw.cuda(), 1e-5, inv_freq.cuda(), rot, gpu, kg, vg,
                                       table.cuda(), page, True, interleaved=interleaved)
        slack = 30 * 2.0 ** -24
        close(got, want, dtype, f"q, interleaved={interleaved}", rel32=4e-6, slack=slack)
        close(kg, kc, dtype, f"k cache, interleaved={interleaved}", rel32=4e-6, slack=slack)
        assert torch.equal(vg.cpu(), vc)
        results[interleaved] = got.float().cpu()
    assert (results[True] - results[False]).abs().max() > 0.05


@pytest.mark.parametrize("case", [(32, 8, 16), (12, 3, 8), (5, 1, 64), (7, 7, 32), (16, 1, 16)])
@pytest.mark.parametrize("store", [True, False])
@pytest.mark.parametrize("many", [False, True])
def test_decode_attention_from_the_qkv_rows(case, store, many):
    """Steps of single tokens, bfloat16, heads of 64: norm + rotation + cache store + attention
    as one launch.  Against the two kernels it replaces: the caches must hold the same bits
    afterwards (and nothing else may have changed), the outputs agree up to the rounding of
    the queries; against the plain implementation too.  Sequences of one key, at a page's and
    a tile's edge and thousands long, with and without a window, and with another layer's
    cache (nothing is stored then)."""
    heads, kv_heads, page = case
    d = 64
    starts = [0, page - 1, page, 63, 64, 700, 2100]  # seven rows; the engine sends up to 64 this way
    if many:
        starts = starts[:6] + [(i * 53) % 600 for i in range(34)]  # forty rows: parts of other lengths, clusters of other sizes
    num_pages = sum(-(-(s + 1) // page) for s in starts) + 3
    cpu, gpu, table = make_step([1] * len(starts), starts, page, num_pages, 170)
    cpu.all_decode = gpu.all_decode = True
    dtype = torch.bfloat16
    T = len(starts)
    qkv = rnd((T, (heads + 2 * kv_heads) * d), dtype, 171)
    qw = 1.0 + 0.2 * rnd((d,), torch.float32, 172)
    kw = 1.0 + 0.2 * rnd((d,), torch.float32, 173)
    inv_freq = (10000.0 ** (-torch.arange(d // 2, dtype=torch.float64) * 2 / d)).float()
    eps = 1e-5
    k0 = rnd((num_pages, page, kv_heads, d), dtype, 174)
    v0 = rnd((num_pages, page, kv_heads, d), dtype, 175)
    scale = 1.0 / math.sqrt(d)
    for window in (0, 50):
        k_two, v_two, k_one, v_one = k0.clone().cuda(), v0.clone().cuda(), k0.clone().cuda(), v0.clone().cuda()
        q = ops().qk_norm_rope_store(qkv.cuda(), heads, kv_heads, d, qw.cuda(), kw.cuda(), eps, inv_freq.cuda(), d, gpu,
                                     k_two, v_two, table.cuda(), page, store)
        two = ops().paged_attention(q, heads, kv_heads, d, k_two, v_two, table.cuda(), page, scale, window, gpu)
        one = ops().decode_attention_from_qkv(qkv.cuda(), heads, kv_heads, d, qw.cuda(), kw.cuda(), eps, inv_freq.cuda(), d, gpu,
                                              k_one, v_one, table.cuda(), page, store, scale, window)
        ops().check_kernel_status()
        assert one is not None
        assert torch.equal(k_one, k_two) and torch.equal(v_one, v_two), "the caches differ from the two-kernel route's"
        if not store:
            assert torch.equal(k_one.cpu(), k0) and torch.equal(v_one.cpu(), v0)
        close(one, two, dtype, f"from qkv against two kernels {case} window {window}")
        kc, vc = k0.clone(), v0.clone()
        want_q = ref.qk_norm_rope_store(qkv, heads, kv_heads, d, qw, kw, eps, inv_freq, d, cpu, kc, vc, table, page, store)
        want = ref.paged_attention(want_q, heads, kv_heads, d, kc, vc, table, page, scale, window, cpu)
        close(one, want, dtype, f"from qkv against the plain implementation {case} window {window}")
    # other steps and sizes are declined
    cpu2, gpu2, table2 = make_step([2], [5], page, num_pages, 176)
    assert ops().decode_attention_from_qkv(qkv[:2].cuda(), heads, kv_heads, d, qw.cuda(), kw.cuda(), eps, inv_freq.cuda(), d, gpu2,
                                           k0.cuda(), v0.cuda(), table2.cuda(), page, True, scale, 0) is None


def test_attention_finds_a_far_key():
    """One key among hundreds is made to stand out; the output must be (almost) its value."""
    heads, kv_heads, d, page = 2, 1, 32, 16
    n = 700
    cpu, gpu, table = make_step([1], [n - 1], page, 64, 30)
    k = rnd((64, page, kv_heads, d), torch.float32, 31, 0.1)
    v = rnd((64, page, kv_heads, d), torch.float32, 32)
    q = rnd((1, heads * d), torch.float32, 33, 0.1)
    far = 3  # position 3, hundreds of keys back
    row = table[0, far // page].item() * page + far % page
    k.view(-1, kv_heads, d)[row, 0] = 40.0 * q[0, :d] / q[0, :d].norm()
    q[0, :d] = 40.0 * q[0, :d] / q[0, :d].norm()
    got = ops().paged_attention(q.cuda(), heads, kv_heads, d, k.cuda(), v.cuda(), table.cuda(), page, 1.0, 0, gpu).cpu()
    want = ref.paged_attention(q, heads, kv_heads, d, k, v, table, page, 1.0, 0, cpu)
    close(got, want, torch.float32, "far key", rel32=1e-5)
    assert (got[0, :d] - v.view(-1, kv_heads, d)[row, 0]).abs().max() < 1e-3


def test_argmax_ties_and_non_finite():
    logits = rnd((5, 1000), torch.float32, 40)
    logits[0, 17] = logits[0, 900] = 50.0  # tie: the lower id wins
    logits[1, :] = float("-inf")  # nothing finite: id 0
    logits[2, 3] = float("nan")
    logits[3, 999] = 60.0
    logits[4, 0] = float("inf")  # not finite, never chosen
    got = ops().argmax(logits.cuda()).cpu().tolist()
    want = []
    for r in range(5):
        row = logits[r].clone()
        row[~torch.isfinite(row)] = float("-inf")
        want.append(int(row.argmax()) if torch.isfinite(row).any() else 0)
    assert got == want and got[0] == 17 and got[1] == 0 and got[3] == 999


def test_sample_kernel_follows_the_host_rule():
    """The device sampler against the host statement of the same rule.  expf/logf differ from
    NumPy in the last place, so the device's pick must be an allowed candidate whose score is
    within rounding of the best score; with these seeds it is the same token."""
    import numpy as np

    from shiso_llm_b200.sampling import SamplingParams, candidate_mask, keyed_sample
    from shiso_llm_b200.sampling.host import argmax as host_argmax, keyed_uniform

    vocab = 3000
    cases = [
        SamplingParams(temperature=0.8, seed=1), SamplingParams(temperature=1.3, top_k=40, seed=2),
        SamplingParams(temperature=0.7, top_p=0.8, seed=3), SamplingParams(temperature=1.0, min_p=0.05, seed=4),
        SamplingParams(temperature=0.9, top_k=100, top_p=0.6, min_p=0.01, seed=2**63 + 5),
        SamplingParams(temperature=0.0, seed=6), SamplingParams(temperature=2.0, top_k=1, seed=7),
        SamplingParams(temperature=0.5, top_k=5000, top_p=1.5, min_p=-1.0, seed=8),
    ]
    logits = rnd((len(cases), vocab), torch.float32, 50, 2.5)
    logits[1, 5] = logits[1, 9] = logits[1].max() + 1.0  # a tie at the top
    logits[3, 100:200] = float("-inf")
    logits[4, 7] = float("nan")
    from shiso_llm_b200.sampling import DeviceSampler

    sampler = DeviceSampler(ops(), "cuda")
    same = 0
    for position in (0, 1, 17, 4095):
        picks = sampler.sample(logits.cuda(), cases, [position] * len(cases))
        for r, (p, pick) in enumerate(zip(cases, picks)):
            row = logits[r].numpy()
            want = keyed_sample(row, p, p.seed, position)
            if p.greedy:
                assert pick == want == host_argmax(row)
                continue
            mask = candidate_mask(row, p)
            assert mask[pick], f"row {r}: token {pick} is not an allowed candidate"
            ids = np.nonzero(mask)[0]
            score = (row[ids] - row[host_argmax(row)]) / np.float32(p.temperature) - np.log(-np.log(keyed_uniform(p.seed, position, ids)))
            assert score[list(ids).index(pick)] >= score.max() - 1e-4
            same += pick == want
    assert same >= 4 * 6 - 1


def test_suppressed_ids_on_the_device_follow_the_host_rule():
    """``bad_token_ids``: -inf before the pick, in the greedy kernels (one and two stages) and in
    the keyed kernel; rows without such ids are not touched; the pick equals the host's."""
    import numpy as np

    from shiso_llm_b200.sampling import DeviceSampler, SamplingParams, candidate_mask, keyed_sample

    sampler = DeviceSampler(ops(), "cuda")
    for vocab in (3000, 20000):
        logits = rnd((4, vocab), torch.float32, 60 + vocab, 2.0)
        order = [torch.argsort(logits[r], descending=True).tolist() for r in range(4)]
        cases = [
            SamplingParams(temperature=0.0, bad_token_ids=order[0][:3]),
            SamplingParams(temperature=0.0),
            SamplingParams(temperature=0.0, bad_token_ids=[order[2][0], vocab + 5]),  # an id past the row is ignored
            SamplingParams(temperature=0.0, bad_token_ids=order[3][1:4]),
        ]
        dev = logits.cuda()
        assert sampler.sample(dev, cases, [0] * 4) == [order[0][3], order[1][0], order[2][1], order[3][0]]
        assert torch.isneginf(dev.cpu()[0, order[0][:3]]).all() and torch.equal(dev.cpu()[1], logits[1])
        mixed = [
            SamplingParams(temperature=1.1, top_k=50, seed=4, bad_token_ids=order[0][:25]),
            SamplingParams(temperature=0.0, bad_token_ids=order[1][:1]),
            SamplingParams(temperature=0.9, top_p=0.7, seed=5),
            SamplingParams(temperature=1.0, seed=6, bad_token_ids=order[3][:2]),
        ]
        for position in (0, 9, 300):
            picks = sampler.sample(logits.cuda(), mixed, [position] * 4)
            for r, (p, pick) in enumerate(zip(mixed, picks)):
                assert pick not in p.bad_token_ids
                row = logits[r].numpy()
                if p.greedy:
                    assert pick == keyed_sample(row, p, p.seed, position)
                else:
                    cut = row.copy()
                    cut[[t for t in p.bad_token_ids if t < vocab]] = -np.inf
                    assert candidate_mask(cut, p)[pick]
            assert picks[1] == order[1][1]


def test_the_status_word_travels_with_the_picks():
    """A picking kernel that is given a place for it moves the status word there and clears it."""
    logits = rnd((3, 20000), torch.float32, 70).cuda()
    small = rnd((3, 500), torch.float32, 71).cuda()
    out = torch.full((4,), -7, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ops().check_kernel_status()
    for rows in (logits, small):
        ops().argmax(rows, out[:3], out[3:4])
        assert out[3].item() == 0
        ops().selftest_bounded_wait(3000)
        ops().argmax(rows, out[:3], out[3:4])
        assert out[3].item() == 1 and out[:3].tolist() == rows.argmax(-1).tolist()
        ops().argmax(rows, out[:3], out[3:4])
        assert out[3].item() == 0
        ops().check_kernel_status()  # the kernel cleared it
    from shiso_llm_b200.sampling import DeviceSampler, SamplingParams

    ops().selftest_bounded_wait(3000)
    DeviceSampler(ops(), "cuda").sample_into(small, [SamplingParams(temperature=0.9, seed=r) for r in range(3)], [5, 6, 7],
                                             out[:3], out[3:4])
    assert out[3].item() == 1
    ops().check_kernel_status()


@pytest.mark.parametrize("case", [(4, 2, 16, 4), (3, 1, 32, 16), (32, 8, 64, 16), (6, 6, 48, 8), (8, 1, 128, 16), (2, 1, 256, 4), (5, 5, 80, 16), (32, 2, 64, 16), (36, 2, 32, 8),
                                  (6, 2, 64, 8), (5, 1, 64, 32), (12, 4, 64, 64), (7, 7, 64, 16), (4, 2, 64, 4)])
def test_decode_attention_split_keys(case):
    """Steps of single tokens in bfloat16 take the split-key kernel: sequences of very
    different lengths in one launch (one key, a page's edge, thousands of keys), windows."""
    heads, kv_heads, d, page = case
    starts = [0, page - 1, page, 700, 2100, 33]
    num_pages = sum(-(-(s + 1) // page) for s in starts) + 3
    cpu, gpu, table = make_step([1] * len(starts), starts, page, num_pages, 60)
    cpu.all_decode = gpu.all_decode = True
    dtype = torch.bfloat16
    k = rnd((num_pages, page, kv_heads, d), dtype, 61)
    v = rnd((num_pages, page, kv_heads, d), dtype, 62)
    q = rnd((len(starts), heads * d), dtype, 63)
    scale = 1.0 / math.sqrt(d)
    for window in (0, 50):
        want = ref.paged_attention(q, heads, kv_heads, d, k, v, table, page, scale, window, cpu)
        got = ops().paged_attention(q.cuda(), heads, kv_heads, d, k.cuda(), v.cuda(), table.cuda(), page, scale, window, gpu)
        close(got, want, dtype, f"decode attention {case} window {window}")
        # the general kernel on the same inputs, for the difference between the two routes
        general = ops().paged_attention(q.cuda(), heads, kv_heads, d, k.cuda(), v.cuda(), table.cuda(), page, scale, window, gpu,
                                        general=True)
        close(got, general, dtype, "decode kernel against the general kernel")


@pytest.mark.parametrize("page", [16, 64, 8])
@pytest.mark.parametrize("parts", [1, 2, 3, 5, 7, 8, 16])
def test_decode_attention_long_parts(page, parts, monkeypatch):
    """Head size 64 takes the kernel that brings pages in by TMA and merges the parts itself:
    parts of many tiles (the ring is refilled dozens of times), one part alone (no merge), more
    parts than a short sequence has tiles (the cluster's idle CTAs still meet the others), a
    window whose edge lies inside a page, and the same launch repeated."""
    from shiso_llm_b200.kernels import ops as ops_module
    if parts > 8 and not ops_module._wide_clusters():
        pytest.skip("this device places no clusters of 16 CTAs")
    heads, kv_heads, d = 12, 3, 64
    starts = [9000, 5003, 63, 64, 65, 0]
    num_pages = sum(-(-(s + 1) // page) for s in starts) + 2
    cpu, gpu, table = make_step([1] * len(starts), starts, page, num_pages, 64)
    cpu.all_decode = gpu.all_decode = True
    dtype = torch.bfloat16
    k = rnd((num_pages, page, kv_heads, d), dtype, 65)
    v = rnd((num_pages, page, kv_heads, d), dtype, 66)
    q = rnd((len(starts), heads * d), dtype, 67)
    monkeypatch.setattr(ops_module, "decode_splits", lambda tokens, kv, capacity, fused=False: parts)
    for window in (0, 3001, 0):
        want = ref.paged_attention(q, heads, kv_heads, d, k, v, table, page, 0.125, window, cpu)
        got = ops().paged_attention(q.cuda(), heads, kv_heads, d, k.cuda(), v.cuda(), table.cuda(), page, 0.125, window, gpu)
        ops().check_kernel_status()
        close(got, want, dtype, f"decode attention by TMA, pages of {page}, {parts} parts, window {window}")


@pytest.mark.parametrize("case", [(4, 2, 16, 4), (3, 1, 32, 16), (8, 2, 64, 16), (6, 3, 48, 8), (5, 5, 80, 16), (4, 1, 128, 16), (2, 2, 112, 4),
                                  (10, 2, 64, 16), (12, 2, 96, 8)])
def test_prefill_attention_tiles(case):
    """Prompt portions in bfloat16 take the tiled tensor-core kernel: portions that span several
    query tiles and many key tiles, portions that start deep in a sequence, single rows beside
    them, windows that cut inside and between tiles."""
    heads, kv_heads, d, page = case
    q_lens, starts = [5, 1, 130, 64, 2, 65], [0, 37, 3, 70, 333, 0]
    num_pages = sum(-(-(s + n) // page) for s, n in zip(starts, q_lens)) + 3
    cpu, gpu, table = make_step(q_lens, starts, page, num_pages, 70)
    cpu.h_q_start = gpu.h_q_start = cpu.q_start.tolist()
    dtype = torch.bfloat16
    k = rnd((num_pages, page, kv_heads, d), dtype, 71)
    v = rnd((num_pages, page, kv_heads, d), dtype, 72)
    q = rnd((sum(q_lens), heads * d), dtype, 73)
    scale = 1.0 / math.sqrt(d)
    for window in (0, 100, 9):
        want = ref.paged_attention(q, heads, kv_heads, d, k, v, table, page, scale, window, cpu)
        got = ops().paged_attention(q.cuda(), heads, kv_heads, d, k.cuda(), v.cuda(), table.cuda(), page, scale, window, gpu)
        close(got, want, dtype, f"tiled attention {case} window {window}")


@pytest.mark.parametrize("case", [(4, 2, 16), (8, 2, 8), (3, 1, 64), (6, 6, 128), (32, 8, 16)])
def test_prefill_attention_in_tensor_memory(case):
    """Long portions of head size 64 in bfloat16 take the tcgen05 kernel (128 query rows per CTA,
    key tiles of 128 through one TMA box per page): portions of several tiles beside short ones
    and single rows, portions that start deep in a sequence, windows that cut inside and between
    tiles and leave holes in the table; cache rows outside every range hold NaN."""
    heads, kv_heads, page = case
    d = 64
    q_lens, starts = [300, 1, 130, 128, 5, 257], [0, 37, 300, 70, 333, 1000]
    if heads >= 32:
        q_lens, starts = [300, 130, 1], [200, 0, 5]
    need = [-(-(s + n) // page) for s, n in zip(starts, q_lens)]
    num_pages = sum(need) + 3
    cpu, gpu, table = make_step(q_lens, starts, page, num_pages, 170)
    cpu.h_q_start = gpu.h_q_start = cpu.q_start.tolist()
    cpu.max_q_len = gpu.max_q_len = max(q_lens)
    dtype = torch.bfloat16
    k = rnd((num_pages, page, kv_heads, d), dtype, 171)
    v = rnd((num_pages, page, kv_heads, d), dtype, 172)
    q = rnd((sum(q_lens), heads * d), dtype, 173)
    scale = 1.0 / math.sqrt(d)
    for window in (0, 200, 9):
        want = ref.paged_attention(q, heads, kv_heads, d, k, v, table, page, scale, window, cpu)
        kn, vn, holes = k.clone(), v.clone(), table.clone()
        used = set()
        for s, (start, n) in enumerate(zip(starts, q_lens)):
            lo = max(0, start + 1 - window) if window > 0 else 0
            for p in range(lo, start + n):
                used.add((table[s, p // page].item(), p % page))
            for b in range(lo // page):
                holes[s, b] = -1  # pages before every row's window
        for pg in range(num_pages):
            for r in range(page):
                if (pg, r) not in used:
                    kn[pg, r] = float("nan")
                    vn[pg, r] = float("nan")
        got = ops().paged_attention(q.cuda(), heads, kv_heads, d, kn.cuda(), vn.cuda(), holes.cuda(), page, scale, window, gpu)
        ops().check_kernel_status()
        assert torch.isfinite(got).all(), f"window {window}: something outside the range reached the result"
        close(got, want, dtype, f"tensor-memory attention {case} window {window}")


def test_prefill_attention_never_reads_outside_its_range():
    """Cache rows the portion must not see hold NaN: pages of other requests, positions after
    the portion, pages a window has passed (holes in the table)."""
    heads, kv_heads, d, page = 4, 2, 64, 16
    q_lens, starts = [70, 3], [60, 0]
    num_pages = 16
    cpu, gpu, table = make_step(q_lens, starts, page, num_pages, 80)
    cpu.h_q_start = gpu.h_q_start = cpu.q_start.tolist()
    k = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 81)
    v = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 82)
    q = rnd((73, heads * d), torch.bfloat16, 83)
    window = 40
    want = ref.paged_attention(q, heads, kv_heads, d, k, v, table, page, 0.125, window, cpu)
    kn, vn = k.clone(), v.clone()
    used = set()
    for s, (start, n) in enumerate(zip(starts, q_lens)):
        for p in range(max(0, start + 1 - window), start + n):
            used.add((table[s, p // page].item(), p % page))
    for pg in range(num_pages):
        for r in range(page):
            if (pg, r) not in used:
                kn[pg, r] = float("nan")
                vn[pg, r] = float("nan")
    holes = table.clone()
    holes[0, 0] = -1  # positions 0..15 of sequence 0 lie before every row's window
    got = ops().paged_attention(q.cuda(), heads, kv_heads, d, kn.cuda(), vn.cuda(), holes.cuda(), page, 0.125, window, gpu)
    assert torch.isfinite(got).all()
    close(got, want, torch.bfloat16, "tiled attention with poisoned surroundings")


@pytest.mark.parametrize("shape", [(1, 96, 64), (8, 2048, 2048), (5, 1000, 96), (8, 300, 200), (16, 2048, 5632), (13, 48, 264), (3, 16, 8),
                                   (8, 4800, 1032), (2, 24, 3080), (24, 2048, 2048), (32, 1000, 264), (17, 40, 5632),
                                   (64, 6144, 2048), (33, 2048, 5632), (50, 776, 264), (64, 48, 8), (40, 11264, 2048),
                                   (65, 2048, 2048), (100, 776, 264), (128, 6144, 2048), (129, 2048, 5632), (192, 11264, 2048), (177, 40, 72),
                                   (8, 2048, 8192), (8, 16384, 2048), (64, 2048, 8192), (48, 16384, 2048),  # a feed-forward of 8,192 (block_ff_dim 12,288)
                                   (40, 998, 264), (64, 1210, 520),  # rows that are no whole groups of four features
                                   (33, 40000, 264), (64, 65536, 520), (16, 50008, 72)])  # 313 to 512 feature tiles: one wave of four CTAs an SM with rings of two stages
def test_skinny_linear_and_fused_swiglu(shape):
    """A handful of bfloat16 rows take the weight-streaming kernel, up to 192 the tensor-memory
    kernel with tokens as the MMA's N operand (tiles of at most 64 tokens, K split over a
    cluster); with a gate/up pair the activation is applied in the epilogue."""
    T, N, K = shape
    x, w = rnd((T, K), torch.bfloat16, 90), rnd((N, K), torch.bfloat16, 91, 0.05)
    bias = rnd((N,), torch.float32, 92)
    for out_dtype in (torch.bfloat16, torch.float32):
        close(ops().linear(x.cuda(), w.cuda(), out_dtype), ref.linear(x, w, out_dtype), out_dtype, f"skinny linear {shape}", rel32=1e-5)
    close(ops().linear(x.cuda(), w.cuda(), torch.float32, bias.cuda()), ref.linear(x, w, torch.float32, bias), torch.float32, "skinny bias", rel32=1e-5)
    if N % 2 == 0:
        got = ops().linear_swiglu(x.cuda(), w.cuda(), torch.bfloat16)
        close(got, ref.linear_swiglu(x, w, torch.bfloat16), torch.bfloat16, f"fused swiglu {shape}")
    big = rnd((40, K), torch.bfloat16, 93)  # above the skinny limit: product kernel + activation kernel
    if N % 2 == 0:
        close(ops().linear_swiglu(big.cuda(), w.cuda(), torch.bfloat16), ref.linear_swiglu(big, w, torch.bfloat16), torch.bfloat16, "unfused swiglu")


def test_argmax_wide_vocabulary_two_stages():
    logits = rnd((6, 65536), torch.float32, 95)
    logits[0, 100] = logits[0, 60000] = 77.0  # a tie across chunks: the lower id
    logits[1, 65535] = 88.0
    logits[2, :] = float("-inf")
    logits[3, 1023] = logits[3, 1024] = 66.0  # a tie at a chunk's edge
    got = ops().argmax(logits.cuda()).cpu().tolist()
    want = ref.argmax(torch.where(torch.isfinite(logits), logits, torch.full_like(logits, float("-inf")))).tolist()
    want[2] = 0
    assert got == want and got[0] == 100 and got[1] == 65535 and got[3] == 1023
    odd = rnd((3, 9001), torch.float32, 96)
    assert ops().argmax(odd.cuda()).cpu().tolist() == ref.argmax(odd).tolist()


@pytest.mark.parametrize("dtype", DTYPES)
def test_short_conv_few_rows_per_sequence_takes_the_serial_kernel(dtype):
    """Steps whose sequences bring at most four rows run one fused kernel (output and state);
    it must give what the two-kernel route gives, bit for bit in float32."""
    taps, hidden = 3, 300
    q_lens, starts = [1, 1, 4, 2, 1, 3], [0, 9, 2, 0, 77, 5]
    cpu, gpu, _ = make_step(q_lens, starts, 4, 64, 97, num_slots=8)
    proj = rnd((sum(q_lens), 3 * hidden), dtype, 98)
    w, b = rnd((hidden, taps), torch.float32, 99), rnd((hidden,), torch.float32, 100)
    start = rnd((8, taps - 1, hidden), torch.float32, 101)
    s_ref, s_two, s_one = start.clone(), start.clone().cuda(), start.clone().cuda()
    want = ref.short_conv(proj, w, b, s_ref, cpu)
    two = ops().short_conv(proj.cuda(), w.cuda(), b.cuda(), s_two, gpu)
    gpu.max_q_len = 4
    one = ops().short_conv(proj.cuda(), w.cuda(), b.cuda(), s_one, gpu)
    close(one, want, dtype, "serial short conv", rel32=4e-6)
    assert torch.equal(one, two) and torch.equal(s_one, s_two)
    assert torch.allclose(s_one.cpu(), s_ref, rtol=0, atol=1e-7)


@pytest.mark.parametrize("case", [(8, 2048, 2048, 3, True), (1, 96, 64, 2, False), (5, 1001, 264, 4, True), (8, 7, 1032, 3, False), (3, 300, 5632, 3, True)])
@pytest.mark.parametrize("scaled", [False, True])
def test_input_projection_with_the_convolution_in_its_epilogue(case, scaled):
    """A handful of bfloat16 rows, one per sequence: the short conv's input projection and the
    gated convolution run as one launch (a tile of the product is the B, C and x rows of five
    channels).  It must give, bit for bit, what the product kernel and the convolution kernel
    give one after the other - output and state - and leave other slots alone; channel counts
    that are no multiple of five, one to eight rows, 2..4 taps, rows with and without their
    RMS scale pending."""
    T, hidden, K, taps, bias = case
    cpu, gpu, _ = make_step([1] * T, [3 + i for i in range(T)], 4, 64, 160, num_slots=11)
    cpu.all_decode = gpu.all_decode = True
    cpu.max_q_len = gpu.max_q_len = 1
    x = rnd((T, K), torch.bfloat16, 161)
    in_proj = rnd((3 * hidden, K), torch.bfloat16, 162, 0.05)
    w = rnd((hidden, taps), torch.float32, 163)
    b = rnd((hidden,), torch.float32, 164) if bias else None
    start = rnd((11, taps - 1, hidden), torch.float32, 165)
    rows = None
    if scaled:
        squares = (0.5 + torch.rand((-(-K // 16), 16), generator=torch.Generator().manual_seed(166))) * K / 16
        rows = ops().ScaledRows(x.cuda(), squares.cuda().contiguous(), 1e-5)
        proj = ops().linear_scaled(rows, in_proj.cuda(), torch.bfloat16)
    else:
        proj = ops().linear(x.cuda(), in_proj.cuda(), torch.bfloat16)
    s_two, s_one, s_ref = start.clone().cuda(), start.clone().cuda(), start.clone()
    two = ops().short_conv(proj, w.cuda(), b.cuda() if bias else None, s_two, gpu)
    one = ops().linear_short_conv(rows if scaled else x.cuda(), in_proj.cuda(), w.cuda(), b.cuda() if bias else None, s_one, gpu)
    ops().check_kernel_status()
    assert torch.equal(one, two), f"fused and two-launch outputs differ by {(one.float() - two.float()).abs().max().item()}"
    assert torch.equal(s_one, s_two)
    # the plain convolution of the same projected rows (the products have their own tests)
    want = ref.short_conv(proj.cpu(), w, b, s_ref, cpu)
    close(one, want, torch.bfloat16, f"projection + convolution {case}")
    assert torch.allclose(s_one.cpu(), s_ref, rtol=0, atol=1e-7)
    untouched = torch.ones(11, dtype=torch.bool)
    untouched[cpu.state_slots.long()] = False
    assert torch.equal(s_one.cpu()[untouched], start[untouched]), "slots of other requests must not change"
    # a step with two rows of one sequence is not taken by the fused route: same result through the two kernels
    cpu2, gpu2, _ = make_step([2], [5], 4, 64, 167, num_slots=11)
    s_a, s_b = start.clone().cuda(), start.clone().cuda()
    xa = x[:1].repeat(2, 1).cuda()
    ya = ops().linear_short_conv(xa, in_proj.cuda(), w.cuda(), b.cuda() if bias else None, s_a, gpu2)
    yb = ops().short_conv(ops().linear(xa, in_proj.cuda(), torch.bfloat16), w.cuda(), b.cuda() if bias else None, s_b, gpu2)
    assert torch.equal(ya, yb) and torch.equal(s_a, s_b)


@pytest.mark.parametrize("shape", [(40, 600, 264), (130, 256, 512), (300, 1000, 96), (513, 2 * 5632, 2048), (777, 2 * 1000, 96), (2048, 2 * 264, 520),
                                   (520, 2 * 8192, 2048)])
def test_tensor_core_product_with_fused_swiglu(shape):
    """More than a handful of bfloat16 rows: gate and up accumulate side by side in tensor
    memory and the epilogue applies the activation (token tiles of 64, 128 and 256; feature
    counts that do not fill the last tile)."""
    T, N, K = shape
    x, w = rnd((T, K), torch.bfloat16, 110), rnd((N, K), torch.bfloat16, 111, 0.05)
    got = ops().linear_swiglu(x.cuda(), w.cuda(), torch.bfloat16)
    ops().check_kernel_status()
    close(got, ref.linear_swiglu(x, w, torch.bfloat16), torch.bfloat16, f"fused swiglu {shape}")
    unfused = ops().swiglu(ops().linear(x.cuda(), w.cuda(), torch.bfloat16))
    close(got, unfused, torch.bfloat16, "fused against product + activation kernel", scale=ref.linear_swiglu(x, w, torch.float32).abs().max().item() * 2)


@pytest.mark.parametrize("taps,hidden,bias", [(3, 2048, False), (4, 96, True), (2, 203 * 8, True)])
def test_fused_projection_and_short_conv(taps, hidden, bias):
    """The conv's input projection followed by the gated convolution through the one kernel-table
    entry the mixer uses for them."""
    k = 264
    q_lens, starts = [1, 1, 3, 2, 1, 4], [0, 9, 2, 0, 77, 5]
    cpu, gpu, _ = make_step(q_lens, starts, 4, 64, 120, num_slots=8)
    gpu.max_q_len = cpu.max_q_len = 4
    x = rnd((sum(q_lens), k), torch.bfloat16, 121)
    w_in = rnd((3 * hidden, k), torch.bfloat16, 122, 0.1)
    w = rnd((hidden, taps), torch.float32, 123)
    b = rnd((hidden,), torch.float32, 124) if bias else None
    start = rnd((8, taps - 1, hidden), torch.float32, 125)
    s_ref, s_fused, s_two = start.clone(), start.clone().cuda(), start.clone().cuda()
    want = ref.short_conv(ref.linear(x, w_in, torch.bfloat16), w, b, s_ref, cpu)
    fused = ops().linear_short_conv(x.cuda(), w_in.cuda(), w.cuda(), b.cuda() if bias else None, s_fused, gpu)
    close(fused, want, torch.bfloat16, "fused projection + conv")
    two = ops().short_conv(ops().linear(x.cuda(), w_in.cuda(), torch.bfloat16), w.cuda(), b.cuda() if bias else None, s_two, gpu)
    close(fused, two, torch.bfloat16, "fused against two kernels")
    assert torch.allclose(s_fused.cpu(), s_ref, rtol=0, atol=2.0 ** -7 * s_ref.abs().max().item())
    untouched = torch.ones(8, dtype=torch.bool)
    untouched[cpu.state_slots.long()] = False
    assert torch.equal(s_fused.cpu()[untouched], start[untouched])


@pytest.mark.parametrize("shape", [(8, 2048, 2048), (1, 96, 64), (13, 1000, 264), (16, 2048, 5632)])
def test_fused_projection_residual_add_and_norm(shape):
    """A block's output projection, the residual add and the next RMS norm through the one
    kernel-table entry the stream uses for them."""
    T, N, K = shape
    x, w = rnd((T, K), torch.bfloat16, 130), rnd((N, K), torch.bfloat16, 131, 0.05)
    res = rnd((T, N), torch.float32, 132, 2.0)
    nw = 1.0 + 0.2 * rnd((N,), torch.float32, 133)
    for round_ in range(3):
        res_ref, res_gpu = res.clone(), res.clone().cuda()
        want = ref.linear_add_rmsnorm(x, w, res_ref, nw, 1e-5, torch.bfloat16)
        got = ops().linear_add_rmsnorm(x.cuda(), w.cuda(), res_gpu, nw.cuda(), 1e-5, torch.bfloat16)
        close(got, want, torch.bfloat16, f"fused add + norm {shape} round {round_}")
        # the product is rounded to bfloat16 before it is added (as the two-kernel route stores
        # it), so the sums may differ by one unit in the last place of the product
        delta_scale = ref.linear(x, w, torch.float32).abs().max().item()
        assert (res_gpu.cpu() - res_ref).abs().max().item() <= 2.0 ** -7 * delta_scale


@pytest.mark.parametrize("shape", [(8, 2048, 2048, 6144), (1, 96, 64, 200), (3, 264, 1000, 520), (7, 4096, 512, 64), (8, 2048, 5632, 2048), (5, 8, 24, 40),
                                   (9, 2048, 2048, 6144), (16, 264, 1000, 520), (33, 2048, 5632, 2048), (64, 2048, 2048, 3072), (100, 776, 264, 200),
                                   (192, 2048, 5632, 11264), (130, 40, 72, 24),
                                   # more rows: the product into the stream as token tiles of 64, the scaled product in whichever kernel takes its shape
                                   (256, 2048, 2048, 6144), (512, 2048, 5632, 6144), (600, 1024, 1024, 3072), (1000, 1032, 520, 264), (1024, 2048, 2048, 2048),
                                   (400, 1024, 264, 1002)])  # a consumer whose width is no multiple of 8
@pytest.mark.parametrize("glu", [False, True])
@pytest.mark.parametrize("bias", [False, True])
def test_product_into_the_stream_then_scaled_product(shape, glu, bias, monkeypatch):
    """Up to 192 bfloat16 rows (the weight-streaming kernel up to 8, the tensor-memory kernel
    with one, two or three token tiles and K split over 1 to 8 CTAs above): a block's output
    projection adds into the residual stream and leaves norm-weighted rows and partial sums of
    squares; the next product applies the row scale to its accumulators.  Against product, add + RMS norm, product (or SwiGLU pair), one
    after the other; the old residual must stay as it was (other CTAs still read it)."""
    from shiso_llm_b200.kernels import ops as ops_module
    monkeypatch.setattr(ops_module, "FUSED_NORM_MAX_TOKENS", 192)  # all the rows the kernel takes, not only those the engine gives it
    T, H, K1, N2 = shape  # stream width H; the first product reads K1, the second gives N2
    x1 = rnd((T, K1), torch.bfloat16, 150)
    w1 = rnd((H, K1), torch.bfloat16, 151, 0.05)
    b1 = rnd((H,), torch.float32, 154) if bias else None
    residual = rnd((T, H), torch.float32, 152, 2.0)
    norm_w = 1.0 + 0.2 * rnd((H,), torch.float32, 153)
    w2 = rnd((2 * N2 if glu else N2, H), torch.bfloat16, 155, 0.05)
    eps = 1e-5
    res_gpu = residual.clone().cuda()
    got = ops().linear_into_stream(x1.cuda(), w1.cuda(), res_gpu, norm_w.cuda(), eps, b1.cuda() if bias else None)
    assert got is not None
    summed, rows = got
    assert torch.equal(res_gpu.cpu(), residual)
    want_sum = residual + ref.linear(x1, w1, torch.float32, b1)
    close(summed, want_sum, torch.float32, "stream after the product", rel32=1e-5)
    assert rows.partials.shape == ((-(-H // 16), 16) if T <= 8 else (-(-H // 128), T))
    mean_square = rows.partials.cpu()[:, :T].sum(0) / H
    assert torch.allclose(mean_square, (want_sum.double() ** 2).mean(-1).float(), rtol=1e-5)
    y = ops().linear_scaled(rows, w2.cuda(), torch.bfloat16, glu)
    x = ref.rmsnorm(want_sum, norm_w, eps, torch.bfloat16)
    want = ref.linear_swiglu(x, w2, torch.bfloat16) if glu else ref.linear(x, w2, torch.bfloat16)
    # x is rounded to bfloat16 on both sides but at different points (before and after the row
    # scale): single inputs differ by one unit in the last place, which the product averages out
    scale = (ref.linear_swiglu(x, w2, torch.float32) if glu else ref.linear(x, w2, torch.float32)).abs().max().item()
    close(y, want, torch.bfloat16, f"scaled product {shape} glu={glu}", scale=2 * scale)


def test_product_into_the_stream_declines_what_it_cannot_take():
    w = torch.zeros(32, 64, device="cuda", dtype=torch.bfloat16)
    nw = torch.ones(32, device="cuda")
    x = torch.zeros(1025, 64, device="cuda", dtype=torch.bfloat16)
    assert ops().linear_into_stream(x, w, torch.zeros(1025, 32, device="cuda"), nw, 1e-5) is None  # too many rows
    wide = torch.zeros(8192, 64, device="cuda", dtype=torch.bfloat16)  # 600 x 8192 is a product for the SM pairs
    assert ops().linear_into_stream(x[:600], wide, torch.zeros(600, 8192, device="cuda"), torch.ones(8192, device="cuda"), 1e-5) is None
    assert ops().linear_into_stream(x[:4].float(), w.float(), torch.zeros(4, 32, device="cuda"), nw, 1e-5) is None


def _random_shapes(seed, count):
    """Row counts on both sides of every dispatch boundary of the products, with feature and k
    counts that are multiples of 8 but of nothing larger."""
    g = torch.Generator().manual_seed(seed)
    edges = [1, 7, 8, 9, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257, 511, 512, 513, 700]
    shapes = []
    for i in range(count):
        T = edges[int(torch.randint(len(edges), (1,), generator=g))]
        N = 8 * int(torch.randint(1, 160, (1,), generator=g))
        K = 8 * int(torch.randint(1, 200, (1,), generator=g))
        shapes.append((T, N, K))
    return shapes


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_products_at_random_sizes_around_every_boundary(seed):
    """Forty random (rows, features, k) per seed, rows chosen around the boundaries between the
    product kernels: plain products (bfloat16 and float32 results, a bias) and gate/up pairs
    against the plain reference."""
    for T, N, K in _random_shapes(seed, 40):
        x, w = rnd((T, K), torch.bfloat16, 1000 + T), rnd((N, K), torch.bfloat16, 2000 + N, 0.05)
        bias = rnd((N,), torch.float32, 3000 + K)
        got = ops().linear(x.cuda(), w.cuda(), torch.float32, bias.cuda())
        close(got, ref.linear(x, w, torch.float32, bias), torch.float32, f"linear {(T, N, K)}", rel32=1e-5)
        close(ops().linear(x.cuda(), w.cuda(), torch.bfloat16), ref.linear(x, w, torch.bfloat16), torch.bfloat16, f"linear bf16 {(T, N, K)}")
        if N % 16 == 0:
            close(ops().linear_swiglu(x.cuda(), w.cuda(), torch.bfloat16), ref.linear_swiglu(x, w, torch.bfloat16), torch.bfloat16,
                  f"swiglu {(T, N, K)}")
    ops().check_kernel_status()


@pytest.mark.parametrize("seed", [1, 2])
def test_decode_attention_at_random_sizes(seed):
    """Random head counts, groups, head sizes, page sizes, lengths and windows through the
    decode kernels (the TMA kernel for heads of 64, the cp.async kernel otherwise)."""
    g = torch.Generator().manual_seed(seed)
    pick = lambda xs: xs[int(torch.randint(len(xs), (1,), generator=g))]
    for i in range(12):
        d = pick([16, 32, 48, 64, 64, 64, 96, 128])
        page = pick([8, 16, 32, 64]) if d == 64 else pick([4, 8, 16])
        kv_heads = pick([1, 2, 3, 5, 8])
        heads = kv_heads * pick([1, 2, 3, 4, 7, 16])
        starts = [int(torch.randint(0, 3000, (1,), generator=g)) for _ in range(pick([1, 3, 9]))]
        window = pick([0, 0, 17, 300, 1025])
        num_pages = sum(-(-(s + 1) // page) for s in starts) + 2
        cpu, gpu, table = make_step([1] * len(starts), starts, page, num_pages, 500 + i)
        cpu.all_decode = gpu.all_decode = True
        k = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 501 + i)
        v = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 502 + i)
        q = rnd((len(starts), heads * d), torch.bfloat16, 503 + i)
        scale = 1.0 / math.sqrt(d)
        want = ref.paged_attention(q, heads, kv_heads, d, k, v, table, page, scale, window, cpu)
        got = ops().paged_attention(q.cuda(), heads, kv_heads, d, k.cuda(), v.cuda(), table.cuda(), page, scale, window, gpu)
        close(got, want, torch.bfloat16, f"decode attention {(heads, kv_heads, d, page, starts, window)}")
    ops().check_kernel_status()


@pytest.mark.parametrize("seed", [1, 2])
def test_prompt_attention_at_random_sizes(seed):
    """Random portions (long and short, starting anywhere in their sequences), head counts,
    head sizes, pages and windows through the prompt attention kernels: the tensor-memory kernel
    where a step has heads of 64 and a portion of 128 rows or more, the tiled kernel otherwise."""
    g = torch.Generator().manual_seed(seed)
    pick = lambda xs: xs[int(torch.randint(len(xs), (1,), generator=g))]
    for i in range(8):
        d = pick([32, 64, 64, 64, 80, 128])
        page = pick([8, 16, 32, 64]) if d == 64 else pick([4, 8, 16])
        kv_heads = pick([1, 2, 4])
        heads = kv_heads * pick([1, 2, 4])
        q_lens = [pick([1, 2, 5, 40, 129, 200, 300]) for _ in range(pick([1, 2, 4]))]
        starts = [int(torch.randint(0, 600, (1,), generator=g)) for _ in q_lens]
        window = pick([0, 0, 9, 150, 700])
        num_pages = sum(-(-(s + n) // page) for s, n in zip(starts, q_lens)) + 2
        cpu, gpu, table = make_step(q_lens, starts, page, num_pages, 600 + i)
        cpu.h_q_start = gpu.h_q_start = cpu.q_start.tolist()
        cpu.max_q_len = gpu.max_q_len = max(q_lens)
        k = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 601 + i)
        v = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 602 + i)
        q = rnd((sum(q_lens), heads * d), torch.bfloat16, 603 + i)
        scale = 1.0 / math.sqrt(d)
        want = ref.paged_attention(q, heads, kv_heads, d, k, v, table, page, scale, window, cpu)
        got = ops().paged_attention(q.cuda(), heads, kv_heads, d, k.cuda(), v.cuda(), table.cuda(), page, scale, window, gpu)
        close(got, want, torch.bfloat16, f"prompt attention {(heads, kv_heads, d, page, q_lens, starts, window)}")
    ops().check_kernel_status()


@pytest.mark.parametrize("seed", [1, 2])
def test_stream_pair_at_random_sizes(seed, monkeypatch):
    """The product into the residual stream and the scaled product behind it at random row
    counts (1..192: both kernels that run the pair, one to three token tiles, every number of
    K parts), widths and depths, with and without a gate/up pair."""
    from shiso_llm_b200.kernels import ops as ops_module
    monkeypatch.setattr(ops_module, "FUSED_NORM_MAX_TOKENS", 192)
    g = torch.Generator().manual_seed(seed)
    pick = lambda xs: xs[int(torch.randint(len(xs), (1,), generator=g))]
    for i in range(16):
        T = pick([1, 3, 8, 9, 15, 16, 17, 32, 33, 64, 65, 100, 128, 129, 192])
        H = 8 * int(torch.randint(1, 300, (1,), generator=g))
        K1 = 8 * int(torch.randint(1, 300, (1,), generator=g))
        N2 = 16 * int(torch.randint(1, 100, (1,), generator=g))
        glu = bool(int(torch.randint(2, (1,), generator=g)))
        x1 = rnd((T, K1), torch.bfloat16, 700 + i)
        w1 = rnd((H, K1), torch.bfloat16, 701 + i, 0.05)
        residual = rnd((T, H), torch.float32, 702 + i, 2.0)
        norm_w = 1.0 + 0.2 * rnd((H,), torch.float32, 703 + i)
        w2 = rnd((2 * N2 if glu else N2, H), torch.bfloat16, 704 + i, 0.05)
        got = ops().linear_into_stream(x1.cuda(), w1.cuda(), residual.cuda(), norm_w.cuda(), 1e-5)
        assert got is not None
        summed, rows = got
        want_sum = residual + ref.linear(x1, w1, torch.float32)
        close(summed, want_sum, torch.float32, f"stream {(T, H, K1)}", rel32=1e-5)
        assert torch.allclose(rows.partials.cpu()[:, :T].sum(0) / H, (want_sum.double() ** 2).mean(-1).float(), rtol=1e-5)
        y = ops().linear_scaled(rows, w2.cuda(), torch.bfloat16, glu)
        x = ref.rmsnorm(want_sum, norm_w, 1e-5, torch.bfloat16)
        want = ref.linear_swiglu(x, w2, torch.bfloat16) if glu else ref.linear(x, w2, torch.bfloat16)
        scale = (ref.linear_swiglu(x, w2, torch.float32) if glu else ref.linear(x, w2, torch.float32)).abs().max().item()
        close(y, want, torch.bfloat16, f"scaled product {(T, H, K1, N2, glu)}", scale=2 * scale)
    ops().check_kernel_status()


@pytest.mark.parametrize("words", [1, 9, 300, 5000, 16384])
def test_words_between_pinned_host_memory_and_the_device_by_kernel(words):
    """A step's block and its tokens move as loads and stores of a kernel that addresses pinned
    host memory in place; memory that is not pinned, or too small, is left to the caller's copy."""
    g = torch.Generator().manual_seed(words)
    source = torch.randint(-2**31, 2**31 - 1, (words + 7,), dtype=torch.int32, generator=g).pin_memory()
    on_device = torch.zeros(words, dtype=torch.int32, device="cuda")
    assert ops().words_from_host(source, on_device) is True
    assert torch.equal(on_device.cpu(), source[:words])
    back = torch.zeros(words + 3, dtype=torch.int32).pin_memory()
    assert ops().words_to_host(on_device, back) is True
    torch.cuda.synchronize()
    assert torch.equal(back[:words], source[:words]) and not back[words:].any()
    assert ops().words_from_host(torch.zeros(words, dtype=torch.int32), on_device) is False  # pageable memory
    assert ops().words_to_host(on_device, torch.zeros(words, dtype=torch.int32)) is False
    if words > 1:
        assert ops().words_to_host(on_device, torch.zeros(words - 1, dtype=torch.int32).pin_memory()) is False
        assert ops().words_from_host(torch.zeros(words - 1, dtype=torch.int32).pin_memory(), on_device) is False
    ops().check_kernel_status()
