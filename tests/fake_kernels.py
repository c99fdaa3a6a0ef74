"""Plain PyTorch stand-ins for the kernel table, one function per kernel.

Two uses.  (1) CPU tests hand this module to the engine in place of the CUDA kernel
table, so that the step function, the cache and the scheduler are exercised without a
GPU; the product itself has no such path.  (2) GPU tests compare every CUDA kernel with
the function of the same name here.  Arithmetic is done in float64 and rounded once to
the output type, so these are references, not imitations of the kernels' rounding.

Formulas: the same reference lines the kernels cite (kernels/cuda/generic/norm.cuh,
kernels/cuda/dense/dense_norm_rope.cuh, dense_attn.cuh, dense_common.cuh:120-126,166-180,
kernels/metal/dense/dense_short_conv.metal:31-68, kernels/cuda/generic/glu.cuh:35-57).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def require():
    return None


def embed(ids, table, feed_index=None, fed_tokens=None):
    ids = ids.long()
    if feed_index is not None:
        fed = fed_tokens.long()[feed_index.long().clamp(min=0)]
        ids = torch.where(feed_index.long() >= 0, fed, ids)
    return table[ids].to(torch.float32)


def gather_rows(x, rows):
    return x[rows.long()].clone()


def rmsnorm(x, w, eps, out_dtype):
    x64 = x.to(F64)
    y = x64 / torch.sqrt((x64 * x64).mean(-1, keepdim=True) + eps) * w.to(F64)
    return y.to(out_dtype)


def add_rmsnorm(residual, delta, w, eps, out_dtype, rows=None):
    if rows is None:
        residual += delta.to(residual.dtype)
        return rmsnorm(residual, w, eps, out_dtype)
    idx = rows.long()
    summed = residual[idx] + delta[idx].to(residual.dtype)
    return rmsnorm(summed, w, eps, out_dtype)


def linear(x, w, out_dtype, bias=None):
    y = x.to(F64) @ w.to(F64).T
    if bias is not None:
        y = y + bias.to(F64)
    return y.to(out_dtype)


def swiglu(gate_up):
    inter = gate_up.shape[1] // 2
    g = gate_up[:, :inter].to(F64)
    u = gate_up[:, inter:].to(F64)
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear_swiglu(x, gate_up, out_dtype):
    y = x.to(F64) @ gate_up.to(F64).T
    inter = y.shape[1] // 2
    g, u = y[:, :inter], y[:, inter:]
    return (g / (1.0 + torch.exp(-g)) * u).to(out_dtype)


class ScaledRows:
    def __init__(self, x, partials, eps):
        self.x, self.partials, self.eps = x, partials, eps


def linear_into_stream(x, w, residual, next_norm_w, eps, bias=None):
    """The pair the CUDA table offers for up to 64 bfloat16 rows; here for any type, so that
    the parts' handling of it runs on the CPU too."""
    if x.shape[0] > 64:
        return None  # as the CUDA table: short steps only
    summed = residual + linear(x, w, torch.float32, bias)
    rows = (summed.to(F64) * next_norm_w.to(F64)).to(x.dtype)
    return summed, ScaledRows(rows, (summed.to(F64) ** 2).sum(-1, keepdim=True).T.contiguous(), eps)


def linear_scaled(rows, w, out_dtype, glu=False):
    k = rows.x.shape[1]
    inv = 1.0 / torch.sqrt(rows.partials.sum(0) / k + rows.eps)
    y = (rows.x.to(F64) @ w.to(F64).T) * inv[:, None]
    if glu:
        inter = y.shape[1] // 2
        g, u = y[:, :inter], y[:, inter:]
        y = g / (1.0 + torch.exp(-g)) * u
    return y.to(out_dtype)


def linear_add_rmsnorm(x, w, residual, norm_w, eps, out_dtype):
    return add_rmsnorm(residual, linear(x, w, out_dtype), norm_w, eps, out_dtype)


def linear_short_conv(x, in_proj, taps, bias, state, step):
    """``x`` is a tensor or ``ScaledRows``, as in the CUDA table."""
    if isinstance(x, ScaledRows):
        return short_conv(linear_scaled(x, in_proj, x.x.dtype), taps, bias, state, step)
    return short_conv(linear(x, in_proj, x.dtype), taps, bias, state, step)


def short_conv(proj, taps, bias, state, step):
    """y[t] = c[t] * (sum_j taps[:, j] * u[t - (L-1) + j] + bias); u = b * x; the state of
    each sequence's slot holds the last L-1 values of u (float32) and is updated."""
    T, H3 = proj.shape
    H = H3 // 3
    L = taps.shape[1]
    p = proj.to(F64)
    b, c, x = p[:, :H], p[:, H : 2 * H], p[:, 2 * H :]
    u = b * x
    y = torch.zeros(T, H, dtype=F64)
    q_start = step.q_start.tolist()
    slots = step.state_slots.tolist()
    for s in range(step.num_seqs):
        a, e = q_start[s], q_start[s + 1]
        full = torch.cat([state[slots[s]].to(F64), u[a:e]], dim=0)  # [(L-1) + n, H]
        n = e - a
        acc = torch.zeros(n, H, dtype=F64)
        for j in range(L):
            acc += taps[:, j].to(F64)[None, :] * full[j : j + n]
        if bias is not None:
            acc += bias.to(F64)[None, :]
        y[a:e] = c[a:e] * acc
        state[slots[s]] = full[-(L - 1) :].to(state.dtype)
    return y.to(proj.dtype)


def _cache_rows(block_table, seq_of_token, positions, page_size):
    pages = block_table.long()[seq_of_token.long(), (positions // page_size).long()]
    return pages * page_size + (positions % page_size).long()


def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_w, k_w, eps, inv_freq, rotary_dim, step,
                       k_cache, v_cache, block_table, page_size, store, interleaved=False):
    T = qkv.shape[0]
    d = head_dim
    x = qkv.to(F64)
    q = x[:, : heads * d].reshape(T, heads, d)
    pos = step.positions.to(F64)

    def norm(v, w):
        if w is None:
            return v
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w.to(F64)

    def rotate(v):
        if not rotary_dim:
            return v
        half = rotary_dim // 2
        # the angle in float64 from the float32 frequency table the kernel is given: a kernel that
        # forms it in float32 is off by up to position * 2^-24 radians, which its test allows for
        angle = step.positions.to(F64)[:, None] * inv_freq.to(F64)[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        out = v.clone()
        if interleaved:  # pairs of neighbours (2i, 2i + 1)
            a, b = v[..., 0:rotary_dim:2], v[..., 1:rotary_dim:2]
            out[..., 0:rotary_dim:2] = a * cos - b * sin
            out[..., 1:rotary_dim:2] = a * sin + b * cos
            return out
        a, b = v[..., :half], v[..., half:rotary_dim]
        out[..., :half] = a * cos - b * sin
        out[..., half:rotary_dim] = a * sin + b * cos
        return out

    q = rotate(norm(q, q_w))
    if kv_heads and store:
        k = x[:, heads * d : (heads + kv_heads) * d].reshape(T, kv_heads, d)
        v = x[:, (heads + kv_heads) * d :].reshape(T, kv_heads, d)
        k = rotate(norm(k, k_w))
        rows = _cache_rows(block_table, step.seq_of_token, step.positions, page_size)
        k_cache.view(-1, kv_heads, d)[rows] = k.to(k_cache.dtype)
        v_cache.view(-1, kv_heads, d)[rows] = v.to(v_cache.dtype)
    return q.reshape(T, heads * d).to(qkv.dtype)


def paged_attention(q, heads, kv_heads, head_dim, k_cache, v_cache, block_table, page_size, scale, window, step):
    T = q.shape[0]
    d = head_dim
    group = heads // kv_heads
    q64 = q.to(F64).reshape(T, heads, d)
    kf = k_cache.view(-1, kv_heads, d)
    vf = v_cache.view(-1, kv_heads, d)
    out = torch.zeros(T, heads, d, dtype=F64)
    seq = step.seq_of_token.tolist()
    pos = step.positions.tolist()
    for t in range(T):
        lo = max(0, pos[t] + 1 - window) if window else 0
        ps = torch.arange(lo, pos[t] + 1)
        pages = block_table[seq[t]].long()[(ps // page_size)]
        rows = pages * page_size + ps % page_size
        k = kf[rows].to(F64)  # [n, kv, d]
        v = vf[rows].to(F64)
        for h in range(heads):
            g = h // group
            s = (k[:, g, :] @ q64[t, h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[:, g, :]
    return out.reshape(T, heads * d).to(q.dtype)


CARRIES_STATUS = True
GAVE_UP = "a kernel gave up waiting on a barrier; what it wrote is not valid"
STATUS_WORD = [0]  # a test sets it to imitate a kernel whose bounded wait ran out


def hand_over_status(status_out):
    if status_out is not None:
        status_out[0] = STATUS_WORD[0]
        STATUS_WORD[0] = 0


def suppress(logits, rows, ids):
    logits[rows.long(), ids.long()] = float("-inf")
    return logits


def argmax(logits, out=None, status_out=None):
    """Lowest id among the finite maxima (crates/shiso-engine/src/sampling.rs:91-154)."""
    hand_over_status(status_out)
    picks = torch.argmax(torch.where(torch.isfinite(logits), logits, torch.full_like(logits, float("-inf"))), dim=-1).to(torch.int32)
    if out is None:
        return picks
    out.copy_(picks)
    return out
