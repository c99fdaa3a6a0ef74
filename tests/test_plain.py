"""The plain implementation against itself: each part's stated properties, on the CPU."""

import math

import torch

import helpers
import plain_lfm2 as plain


def test_width_rule():
    assert plain.plain_ff_width(8192, True, 1.0, 256) == 5632
    assert plain.plain_ff_width(384, True, 1.0, 64) == 256
    assert plain.plain_ff_width(192, False, 1.0, 256) == 192


def test_rmsnorm_and_rope_basics():
    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.rand(12, dtype=torch.float64) + 0.5
    y = plain.plain_rmsnorm(x, w, 0.0) / w
    assert torch.allclose((y * y).mean(-1), torch.ones(5, dtype=torch.float64))
    v = torch.randn(4, 3, 8, dtype=torch.float64)
    pos = torch.tensor([0, 1, 5, 9])
    r = plain.plain_rope_half_split(v, pos, 10000.0)
    assert torch.allclose(r[0], v[0])  # position 0 is not rotated
    assert torch.allclose(r.norm(dim=-1), v.norm(dim=-1))
    # pairs are (i, i + d/2): rotating by angle pos * theta^(-2i/d)
    i = 1
    angle = 5 * 10000.0 ** (-2 * i / 8)
    a, b = v[2, 0, i], v[2, 0, i + 4]
    assert torch.allclose(r[2, 0, i], a * math.cos(angle) - b * math.sin(angle))
    assert torch.allclose(r[2, 0, i + 4], a * math.sin(angle) + b * math.cos(angle))
    # relative property: scores depend on the position difference only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s1 = (plain.plain_rope_half_split(q, torch.tensor([7]), 1e4) * plain.plain_rope_half_split(k, torch.tensor([3]), 1e4)).sum()
    s2 = (plain.plain_rope_half_split(q, torch.tensor([14]), 1e4) * plain.plain_rope_half_split(k, torch.tensor([10]), 1e4)).sum()
    assert torch.allclose(s1, s2)


def test_short_conv_is_causal_and_gates_before_the_conv():
    torch.manual_seed(0)
    H, L, T = 6, 3, 9
    n = torch.randn(T, H, dtype=torch.float64)
    w_in, w_out = torch.randn(3 * H, H, dtype=torch.float64), torch.eye(H, dtype=torch.float64)
    conv = torch.randn(H, L, dtype=torch.float64)
    y = plain.plain_short_conv(n, w_in, conv, None, w_out)
    n2 = n.clone()
    n2[6:] += 1.0
    y2 = plain.plain_short_conv(n2, w_in, conv, None, w_out)
    assert torch.allclose(y[:6], y2[:6]) and not torch.allclose(y[6], y2[6])
    # by hand at t = 4: c_4 * sum_j conv[:, j] * (b * x)_{4 - 2 + j}
    p = n @ w_in.T
    u = p[:, :H] * p[:, 2 * H :]
    want = p[4, H : 2 * H] * (conv[:, 0] * u[2] + conv[:, 1] * u[3] + conv[:, 2] * u[4])
    assert torch.allclose(y[4], want)
    want0 = p[0, H : 2 * H] * (conv[:, 2] * u[0])  # the last tap meets the current token
    assert torch.allclose(y[0], want0)


def test_attention_is_causal_groups_heads_and_normalises():
    torch.manual_seed(1)
    H, nh, nkv, d, T = 16, 4, 2, 4, 7
    n = torch.randn(T, H, dtype=torch.float64)
    ws = [torch.randn(r, H, dtype=torch.float64) * 0.3 for r in (nh * d, nkv * d, nkv * d)]
    w_o = torch.eye(H, dtype=torch.float64)
    ones = torch.ones(d, dtype=torch.float64)
    out = plain.plain_attention(n, *ws, w_o, ones, ones, 1e-6, 1e4, nh, nkv)
    n2 = n.clone()
    n2[5] += 2.0
    out2 = plain.plain_attention(n2, *ws, w_o, ones, ones, 1e-6, 1e4, nh, nkv)
    assert torch.allclose(out[:5], out2[:5]) and not torch.allclose(out[5:], out2[5:])
    # the first token attends to itself only: its output is its own value, per KV group
    v0 = (n[0] @ ws[2].T).reshape(nkv, d)
    assert torch.allclose(out[0].reshape(nh, d), v0.repeat_interleave(nh // nkv, dim=0))
    # a window of 1 makes every token attend to itself only
    outw = plain.plain_attention(n, *ws, w_o, ones, ones, 1e-6, 1e4, nh, nkv, window=1)
    v = (n @ ws[2].T).reshape(T, nkv, d).repeat_interleave(nh // nkv, dim=1)
    assert torch.allclose(outw.reshape(T, nh, d), v)


def test_swiglu():
    n = torch.randn(3, 4, dtype=torch.float64)
    g, u, dn = torch.randn(5, 4, dtype=torch.float64), torch.randn(5, 4, dtype=torch.float64), torch.randn(4, 5, dtype=torch.float64)
    a, b = n @ g.T, n @ u.T
    assert torch.allclose(plain.plain_swiglu(n, g, u, dn), (torch.nn.functional.silu(a) * b) @ dn.T)


def test_whole_model_prefix_property_and_tied_head():
    for name in ("A", "B"):
        doc, seed = helpers.TINY[name]
        tensors = helpers.make_tensors(doc, seed)
        ids = helpers.random_prompt(20, doc["vocab_size"], 1)
        full = plain.plain_forward(doc, tensors, ids)
        assert full.shape == (20, doc["vocab_size"])
        assert torch.allclose(plain.plain_forward(doc, tensors, ids[:11]), full[:11], atol=1e-12)
        f32 = plain.plain_forward(doc, tensors, ids, dtype=torch.float32)
        assert (f32.double() - full).abs().max() < 1e-5
    doc, seed = helpers.TINY["A"]
    tensors = helpers.make_tensors(doc, seed)
    logits, hidden = plain.plain_forward(doc, tensors, [1, 2, 3], return_hidden=True)
    nf = plain.plain_rmsnorm(hidden, tensors["model.embedding_norm.weight"].double(), doc["norm_eps"])
    assert torch.allclose(logits, nf @ tensors["model.embed_tokens.weight"].double().T)


def test_plain_implementation_has_not_drifted():
    """tests/golden/plain_tiny.json pins a few logits of this file's functions (it is not an
    output of the reference, which cannot be run here)."""
    import importlib.util
    import json
    import os

    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "golden", "make_golden.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    stored = json.load(open(os.path.join(here, "golden", "plain_tiny.json")))
    fresh = module.golden()
    for name in ("A", "B"):
        assert fresh[name]["tokens"] == stored[name]["tokens"]
        assert fresh[name]["argmax"] == stored[name]["argmax"] and fresh[name]["greedy"] == stored[name]["greedy"]
        for a, b in zip(fresh[name]["logits"], stored[name]["logits"]):
            assert all(abs(x - y) < 1e-9 for x, y in zip(a, b))
