"""A plain, slow implementation of LFM2: whole sequences, no cache, one function per part.

It shares no code with the package under test: it reads the raw ``config.json``
dictionary and a ``{name: tensor}`` dictionary and evaluates the formulas that
the reference's kernels and launch order define.  The reference's model code
cannot be compiled or imported here (it is Rust, no toolchain is installed, and
its LFM2 short-conv kernel exists only as Metal source), so this file rests on
the formulas alone; each function cites the reference file and lines it restates.

Everything runs in float64 by default so that the comparison target's own
rounding is far below the float32 engine's.  ``round_to`` lets a caller imitate
an engine that stores activations in a narrower type between kernels.
"""

from __future__ import annotations

import math

import torch


def plain_ff_width(block_ff_dim, auto_adjust, multiplier, multiple_of):
    """SwiGLU width rule of the configuration (no twin in the reference, which reads
    the final width from GGUF: crates/shiso-models/src/lfm2/config.rs:177).
    8192 -> 5632 (256), 6656 -> 4608 (256), 10752 -> 7168 (256), 384 -> 256 (64)."""
    if not auto_adjust:
        return block_ff_dim
    w = int(2 * block_ff_dim / 3)
    w = int(multiplier * w)
    return multiple_of * -(-w // multiple_of)


def plain_embedding(ids, table):
    """x_t = E[id_t, :], no scale (crates/shiso-engine/src/layers.rs:1341-1357;
    embed_scale None at crates/shiso-models/src/lfm2/config.rs:185)."""
    return table[ids]


def plain_rmsnorm(x, w, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight multiplies
    directly, not (1 + w) (kernels/cuda/generic/norm.cuh:39-95)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * w


def plain_rope_half_split(v, positions, theta, rotary_dim=None):
    """Half-split rotation of ``v[T, heads, d]``: for i < d/2, angle = pos * theta^(-2i/d),
    (v_i, v_{i+d/2}) <- (v_i cos - v_{i+d/2} sin, v_i sin + v_{i+d/2} cos)
    (kernels/cuda/dense/dense_common.cuh:166-180)."""
    d = v.shape[-1]
    rot = d if rotary_dim is None else rotary_dim
    half = rot // 2
    i = torch.arange(half, dtype=torch.float64, device=v.device)
    inv_freq = theta ** (-2.0 * i / rot)
    angle = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    cos = torch.cos(angle).to(v.dtype)[:, None, :]
    sin = torch.sin(angle).to(v.dtype)[:, None, :]
    out = v.clone()
    a = v[..., :half]
    b = v[..., half:rot]
    out[..., :half] = a * cos - b * sin
    out[..., half:rot] = a * sin + b * cos
    return out


def plain_short_conv(n, w_in, conv_w, conv_b, w_out, rnd=lambda t: t):
    """Gated short convolution over a whole sequence from an empty state.

    p = W_in n, split [b | c | x]; u = b * x (gate BEFORE the conv, the state keeps u);
    y_t = c_t * (sum_j w[:, j] * u_{t-(L-1)+j} (+ bias)); out = W_out y
    (kernels/metal/dense/dense_short_conv.metal:31-68;
    crates/shiso-engine/src/short_conv.rs:146-191).  ``w[:, L-1]`` meets the current
    token (crates/shiso-models/src/lfm2/model.rs:227-232).  The bias is this build's
    option; the reference has none."""
    T, H = n.shape
    L = conv_w.shape[-1]
    conv_w = conv_w.reshape(H, L)
    p = rnd(n @ w_in.T)
    b, c, x = p[:, :H], p[:, H : 2 * H], p[:, 2 * H :]
    u = b * x
    padded = torch.cat([torch.zeros(L - 1, H, dtype=u.dtype, device=u.device), u], dim=0)
    acc = torch.zeros(T, H, dtype=u.dtype, device=u.device)
    for j in range(L):
        acc = acc + conv_w[:, j][None, :] * padded[j : j + T]
    if conv_b is not None:
        acc = acc + conv_b[None, :]
    y = rnd(c * acc)
    return rnd(y @ w_out.T)


def plain_attention(n, w_q, w_k, w_v, w_o, q_norm_w, k_norm_w, eps, theta, n_heads, n_kv_heads, window=None, rnd=lambda t: t):
    """GQA attention over a whole sequence.

    q/k/v projections without bias (crates/shiso-engine/src/dense/attn.rs:509,311-316);
    per-head RMS norm of q and k with a [d] weight BEFORE RoPE
    (kernels/cuda/dense/dense_norm_rope.cuh:42-53,96-106); half-split RoPE; k is
    cached after norm and rotation, v raw (dense_norm_rope.cuh:125-140); score =
    (q . k) / sqrt(d), KV head of query head h is h // (nh / nkv), causal and
    inclusive (kernels/cuda/dense/dense_attn.cuh:60,87-88,110); softmax; W_o."""
    T, _ = n.shape
    d = w_q.shape[0] // n_heads
    positions = torch.arange(T, device=n.device)
    q = rnd(n @ w_q.T).reshape(T, n_heads, d)
    k = rnd(n @ w_k.T).reshape(T, n_kv_heads, d)
    v = rnd(n @ w_v.T).reshape(T, n_kv_heads, d)
    q = rnd(plain_rope_half_split(plain_rmsnorm(q, q_norm_w, eps), positions, theta))
    k = rnd(plain_rope_half_split(plain_rmsnorm(k, k_norm_w, eps), positions, theta))
    group = n_heads // n_kv_heads
    out = torch.zeros(T, n_heads, d, dtype=n.dtype, device=n.device)
    scale = 1.0 / math.sqrt(d)
    for h in range(n_heads):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        allowed = positions[None, :] <= positions[:, None]
        if window is not None:
            allowed = allowed & (positions[None, :] > positions[:, None] - window)
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, g, :]
    return rnd(rnd(out).reshape(T, n_heads * d) @ w_o.T)


def plain_swiglu(n, w_gate, w_up, w_down, rnd=lambda t: t):
    """out = W_down (silu(W_gate n) * (W_up n)), silu(z) = z / (1 + e^-z), no clamp
    (crates/shiso-engine/src/ffn.rs:201-253; kernels/cuda/generic/glu.cuh:35-57)."""
    g = rnd(n @ w_gate.T)
    u = rnd(n @ w_up.T)
    m = rnd(g / (1.0 + torch.exp(-g)) * u)
    return rnd(m @ w_down.T)


def plain_forward(config, tensors, ids, dtype=torch.float64, round_to=None, return_hidden=False, device=None, rows=None,
                  layer_hook=None):
    """Logits ``[T, V]`` of one whole sequence (of the positions ``rows`` only when given).

    ``device`` moves the arithmetic (the same float64 formulas) to another device, so that a
    model of real size is a matter of seconds; tensors that already are in ``dtype`` on that
    device are used as they are.  ``layer_hook(i, x)`` is called with the residual stream
    after every layer.

    Order inside a layer: pre-norm, mixer, residual, feed-forward norm, SwiGLU,
    residual; then the final norm (the tensor named after the embedding) and the
    tied or untied head (crates/shiso-engine/src/layers.rs:1952-2301,2616-2681;
    crates/shiso-models/src/lfm2/model.rs:9-14,201-213)."""
    if round_to is None:
        rnd = lambda t: t
    else:
        rnd = lambda t: t.to(round_to).to(dtype)
    w = {k: v.to(device=device, dtype=dtype) for k, v in tensors.items()}
    H = config["hidden_size"]
    eps = config["norm_eps"]
    ids = torch.as_tensor(ids, dtype=torch.long, device=device)
    x = plain_embedding(ids, w["model.embed_tokens.weight"])
    for i, kind in enumerate(config["layer_types"]):
        p = f"model.layers.{i}"
        n = rnd(plain_rmsnorm(x, w[f"{p}.operator_norm.weight"], eps))
        if kind == "conv":
            m = plain_short_conv(
                n,
                w[f"{p}.conv.in_proj.weight"],
                w[f"{p}.conv.conv.weight"],
                w.get(f"{p}.conv.conv.bias") if config.get("conv_bias", False) else None,
                w[f"{p}.conv.out_proj.weight"],
                rnd,
            )
        elif kind == "full_attention":
            m = plain_attention(
                n,
                w[f"{p}.self_attn.q_proj.weight"],
                w[f"{p}.self_attn.k_proj.weight"],
                w[f"{p}.self_attn.v_proj.weight"],
                w[f"{p}.self_attn.out_proj.weight"],
                w[f"{p}.self_attn.q_layernorm.weight"],
                w[f"{p}.self_attn.k_layernorm.weight"],
                eps,
                config["rope_theta"],
                config["num_attention_heads"],
                config["num_key_value_heads"],
                None,
                rnd,
            )
        else:
            raise ValueError(kind)
        h = x + m
        n2 = rnd(plain_rmsnorm(h, w[f"{p}.ffn_norm.weight"], eps))
        x = h + plain_swiglu(
            n2,
            w[f"{p}.feed_forward.w1.weight"],
            w[f"{p}.feed_forward.w3.weight"],
            w[f"{p}.feed_forward.w2.weight"],
            rnd,
        )
        if layer_hook is not None:
            layer_hook(i, x)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long, device=x.device)]
    nf = rnd(plain_rmsnorm(x, w["model.embedding_norm.weight"], eps))
    tied = config.get("tie_embedding", config.get("tie_word_embeddings", True))
    head = w["model.embed_tokens.weight"] if tied else w["lm_head.weight"]
    logits = nf @ head.T
    if return_hidden:
        return logits, x
    return logits


def plain_greedy(config, tensors, prompt, steps):
    """Greedy continuation by re-running the whole sequence each step; ties go to
    the lower id (crates/shiso-engine/src/sampling.rs:91-154)."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        logits = plain_forward(config, tensors, ids)[-1]
        best = int(torch.argmax(logits))  # torch returns the first maximum
        out.append(best)
        ids.append(best)
    return out
