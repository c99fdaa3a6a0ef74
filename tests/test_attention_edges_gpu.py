"""The attention kernels that generation uses, with one key made to stand out at a place where an
off-by-one would hide among thousands of random keys: position 0, the first position a window
still shows and the one just before it (which must NOT be seen), the last key of a page and of
a 64-key tile, the first and last key of each part a decode kernel cuts a sequence into.

With random keys one key carries about 1/n of the weight, so a key dropped at an edge moves the
output by less than the bfloat16 tolerance; here the planted key takes all the weight of its
KV head's queries, so the output is that key's value when it is visible and far from it when not.
"""

import math
from types import SimpleNamespace

import pytest
import torch

from test_kernels_gpu import make_step, ops, rnd

pytestmark = pytest.mark.gpu

MARK = 3.0


def marker(d, which):
    """A value no average of random values comes near: +-3 in a pattern of its own."""
    signs = torch.tensor([1.0 if (i * (which + 3) + i // 3) % 2 == 0 else -1.0 for i in range(d)])
    return MARK * signs


def plant(k, v, table, page, seq, g, position, direction, which):
    row = table[seq, position // page].item() * page + position % page
    k.view(-1, k.shape[2], k.shape[3])[row, g] = (40.0 * direction).to(k.dtype)
    v.view(-1, v.shape[2], v.shape[3])[row, g] = marker(v.shape[3], which).to(v.dtype)


def part_edges(lo, length, page, splits):
    """Positions at the edges of the parts the two decode kernels cut ``lo..length-1`` into."""
    edges = set()
    n_keys = length - lo
    chunk = -(-n_keys // splits)  # the two-launch kernel: equal runs of keys from lo
    first_tile, last_tile = lo // 64, (length - 1) // 64  # the kernel with the merge inside: runs of 64-key tiles
    per_part = -(-(last_tile - first_tile + 1) // splits)
    for s in range(1, splits):
        for edge in (lo + s * chunk, (first_tile + s * per_part) * 64):
            edges.update((edge - 1, edge))
    return {e for e in edges if lo <= e < length}


@pytest.mark.parametrize("heads,kv_heads,d,page", [(32, 8, 64, 16), (8, 4, 64, 32), (8, 2, 32, 16), (8, 2, 128, 16), (12, 4, 96, 8)])
@pytest.mark.parametrize("window", [0, 301])
def test_decode_kernels_see_a_planted_key_exactly_where_they_should(heads, kv_heads, d, page, window):
    table_ops = ops()
    lengths = [2100, 700, 5003, 65, 64, 129, 17, 1][: max(2, 16 // kv_heads)]
    starts = [n - 1 for n in lengths]
    num_pages = sum(-(-n // page) for n in lengths) + 2
    cpu, gpu, table = make_step([1] * len(lengths), starts, page, num_pages, 300)
    gpu.all_decode = True
    capacity = table.shape[1] * page
    fused = bool(table_ops.library().shiso_decode_attention_fused_supported(heads, kv_heads, d, page))
    splits = table_ops.decode_splits(len(lengths), kv_heads, capacity, fused)
    group = heads // kv_heads
    scale = 1.0 / math.sqrt(d)
    candidates = []
    for n in lengths:
        lo = max(0, n - window) if window else 0
        spots = {0, 1, page - 1, page, 63, 64, 127, 128, n // 2, n - 2, n - 1, lo, lo + 1, lo - 1, lo - 2} | part_edges(lo, n, page, splits)
        candidates.append(sorted(p for p in spots if 0 <= p < n))
    rounds = max(-(-len(c) // kv_heads) for c in candidates)
    direction = torch.nn.functional.normalize(rnd((kv_heads, d), torch.float32, 301), dim=-1)
    checked = hidden = 0
    for r in range(rounds):
        k = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 310 + r, 0.1)
        v = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 330 + r)
        q = torch.zeros(len(lengths), heads, d)
        placed = {}
        for b, n in enumerate(lengths):
            for g in range(kv_heads):
                spot = candidates[b][(r * kv_heads + g) % len(candidates[b])]
                plant(k, v, table, page, b, g, spot, direction[g], g)
                placed[(b, g)] = spot
                q[b, g * group : (g + 1) * group] = 40.0 * direction[g]
        out = table_ops.paged_attention(q.reshape(len(lengths), -1).to(torch.bfloat16).cuda(), heads, kv_heads, d, k.cuda(), v.cuda(),
                                        table.cuda(), page, scale, window, gpu).float().cpu().reshape(len(lengths), heads, d)
        table_ops.check_kernel_status()
        for (b, g), spot in placed.items():
            lo = max(0, lengths[b] - window) if window else 0
            rows = out[b, g * group : (g + 1) * group]
            distance = (rows - marker(d, g)).abs().max().item()
            if spot >= lo:
                assert distance < 0.05, f"length {lengths[b]}, KV head {g}: the key at {spot} (window from {lo}) was not found"
                checked += 1
            else:
                assert distance > 1.0, f"length {lengths[b]}, KV head {g}: the key at {spot} lies before the window ({lo}) and was seen"
                hidden += 1
    assert checked > 20 and (hidden > 0) == bool(window)


@pytest.mark.parametrize("heads,kv_heads,d,page,start,rows", [
    (32, 8, 64, 16, 300, 320),  # long portion, heads of 64: the kernel with its products in tensor memory
    (16, 4, 64, 16, 0, 257),
    (8, 2, 64, 16, 700, 100),  # short portion: the tiled kernel
    (8, 4, 32, 8, 130, 200),  # other head sizes: the tiled kernel
    (4, 1, 128, 16, 64, 150),
])
@pytest.mark.parametrize("window", [0, 150])
def test_prompt_kernels_see_a_planted_key_exactly_where_they_should(heads, kv_heads, d, page, start, rows, window):
    """Every row of a portion asks with the same query; a row sees the planted key iff it lies at
    or after it and the window has not passed it."""
    table_ops = ops()
    end = start + rows
    num_pages = -(-end // page) + 3
    cpu, gpu, table = make_step([rows], [start], page, num_pages, 400)
    gpu.max_q_len, gpu.h_q_start = rows, [0, rows]
    group = heads // kv_heads
    scale = 1.0 / math.sqrt(d)
    spots = sorted({0, page - 1, page, 63, 64, 127, 128, start - 1, start, start + 1, start + 63, start + 64, start + 127,
                    start + 128, end - 2, end - 1, end - window, end - window - 1, start + rows // 2} & set(range(end)))
    direction = torch.nn.functional.normalize(rnd((kv_heads, d), torch.float32, 401), dim=-1)
    positions = torch.arange(start, end)
    seen = unseen = 0
    for r in range(-(-len(spots) // kv_heads)):
        k = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 410 + r, 0.1)
        v = rnd((num_pages, page, kv_heads, d), torch.bfloat16, 430 + r)
        q = torch.zeros(rows, heads, d)
        placed = {}
        for g in range(kv_heads):
            spot = spots[(r * kv_heads + g) % len(spots)]
            plant(k, v, table, page, 0, g, spot, direction[g], g)
            placed[g] = spot
            q[:, g * group : (g + 1) * group] = 40.0 * direction[g]
        out = table_ops.paged_attention(q.reshape(rows, -1).to(torch.bfloat16).cuda(), heads, kv_heads, d, k.cuda(), v.cuda(),
                                        table.cuda(), page, scale, window, gpu).float().cpu().reshape(rows, heads, d)
        table_ops.check_kernel_status()
        for g, spot in placed.items():
            distance = (out[:, g * group : (g + 1) * group] - marker(d, g)).abs().amax(dim=(1, 2))
            visible = positions >= spot
            if window:
                visible &= positions - window < spot
            assert (distance[visible] < 0.05).all(), (
                f"key at {spot}: rows at positions {positions[visible][distance[visible] >= 0.05][:5].tolist()} did not find it")
            assert (distance[~visible] > 1.0).all(), (
                f"key at {spot}: rows at positions {positions[~visible][distance[~visible] <= 1.0][:5].tolist()} saw it")
            seen += int(visible.sum())
            unseen += int((~visible).sum())
    assert seen > rows and unseen > 0
