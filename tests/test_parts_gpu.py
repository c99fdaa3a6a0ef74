"""Each part alone on the GPU, built from a PartSpec with sizes of its own (none of them the
tiny models'), against the plain function of the same formula."""

import math

import pytest
import torch

import plain_lfm2 as plain
from shiso_llm_b200.cache import CacheManager
from shiso_llm_b200.engine.batch import StepBuilder, StepEntry
from shiso_llm_b200.parts import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, BuildEnv, LayerSpec, PartSpec, Stream,
)
from shiso_llm_b200.weights import random_tensors
from shiso_llm_b200.weights.loader import target_dtype

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def env(dtype):
    from shiso_llm_b200.kernels import ops

    ops.require()
    return BuildEnv(dtype=dtype, device=torch.device("cuda:0"), ops=ops)


def bind(part, dtype, seed, std=0.05):
    specs = part.tensor_specs()
    stored = random_tensors(specs, seed, std, "bfloat16", 0.1)
    by = {s.name: s for s in specs}
    part.bind({k: v.to("cuda", target_dtype(by[k], v.dtype, dtype)) for k, v in stored.items()})
    return {k: v.double() for k, v in stored.items()}


def step_for(needs, lengths, dtype, page=4):
    """A cache manager and a step in which sequence i brings lengths[i] tokens from position 0."""
    cache = CacheManager(needs, page, 64, len(lengths) + 1, dtype, "cuda:0")
    builder = StepBuilder(cache, "cuda:0", sum(lengths), len(lengths))
    entries = [StepEntry(i, [0] * n, []) for i, n in enumerate(lengths)]
    starts = [cache.append(i, n) for i, n in enumerate(lengths)]
    return cache, builder.build(entries, starts)


def agree(got, want, dtype, what):
    if hasattr(got, "materialize"):
        got = got.materialize()  # an output projection handed over unevaluated
    err = (got.double().cpu() - want).abs().max().item()
    scale = want.abs().max().item()
    bound = (3e-6 if dtype == torch.float32 else 2.0 ** -6) * scale
    assert err <= bound, f"{what}: {err:.3e} > {bound:.3e}"


def rows(n, width, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, width, generator=g).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    norm = NORMS.build(PartSpec("rmsnorm", {"tensor": "n.weight", "size": 176, "eps": 1e-4}), env(dtype))
    w = bind(norm, dtype, 1)
    x = rows(9, 176, torch.float32, 2)
    agree(norm.apply(x.cuda()), plain.plain_rmsnorm(x.double(), w["n.weight"], 1e-4), dtype, "norm")
    delta = rows(9, 176, dtype, 3)
    res = x.clone().cuda()
    got = norm.add_apply(res, delta.cuda())
    agree(got, plain.plain_rmsnorm(x.double() + delta.double(), w["n.weight"], 1e-4), dtype, "add+norm")
    agree(res, x.double() + delta.double(), torch.float32, "stored sum")


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    e = env(dtype)
    emb = EMBEDDINGS.build(PartSpec("token_embedding", {"tensor": "e.weight", "vocab_size": 333, "hidden_size": 80}), e)
    w = bind(emb, dtype, 4)
    _, step = step_for([], [5], dtype)
    step.token_ids.copy_(torch.tensor([0, 332, 7, 7, 100], dtype=torch.int32))
    agree(emb.forward(step), w["e.weight"][[0, 332, 7, 7, 100]], torch.float32, "embedding")
    tied = HEADS.build(PartSpec("linear_head", {"vocab_size": 333, "hidden_size": 80, "tied_to": "e.weight", "tensor": None}), e)
    tied.bind({"e.weight": emb.table()})
    x = rows(3, 80, dtype, 5)
    got = tied.forward(x.cuda())
    assert got.dtype == torch.float32
    agree(got, x.double() @ w["e.weight"].T, torch.float32 if dtype == torch.float32 else dtype, "tied head")
    own = HEADS.build(PartSpec("linear_head", {"vocab_size": 333, "hidden_size": 80, "tied_to": None, "tensor": "h.weight"}), e)
    wh = bind(own, dtype, 6)
    agree(own.forward(x.cuda()), x.double() @ wh["h.weight"].T, torch.float32 if dtype == torch.float32 else dtype, "own head")


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    ff = FEED_FORWARDS.build(PartSpec("swiglu", {"hidden_size": 80, "intermediate_size": 208, "gate": "g", "up": "u", "down": "d"}), env(dtype))
    w = bind(ff, dtype, 7, 0.1)
    x = rows(11, 80, dtype, 8)
    rnd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype).double())
    agree(ff.forward(x.cuda(), None), plain.plain_swiglu(x.double(), w["g"], w["u"], w["d"], rnd), dtype, "swiglu")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,bias", [(5, True), (2, False)])
def test_short_conv_part(dtype, taps, bias):
    spec = PartSpec("short_conv", {"hidden_size": 112, "taps": taps, "bias": bias, "in_proj": "i", "conv": "c", "conv_bias": "b", "out_proj": "o"})
    mixer = MIXERS.build(spec, env(dtype))
    w = bind(mixer, dtype, 9, 0.2)
    lengths = [7, 1, 12]
    cache, step = step_for([mixer.cache_spec()], lengths, dtype)
    x = rows(sum(lengths), 112, dtype, 10)
    got = mixer.forward(x.cuda(), step, cache.view(0)).materialize()
    rnd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype).double())
    at = 0
    for i, n in enumerate(lengths):
        want = plain.plain_short_conv(x[at : at + n].double(), w["i"], w["c"], w["b"] if bias else None, w["o"], rnd)
        agree(got[at : at + n], want, dtype, f"short conv sequence {i}")
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(6, 2, 48), (5, 1, 16), (2, 2, 80), (4, 2, 24)])
def test_attention_part(dtype, heads, kv_heads, head_dim):
    hidden = 96

    def norm(name):
        return PartSpec("rmsnorm", {"tensor": name, "size": head_dim, "eps": 1e-5})

    spec = PartSpec("gqa_attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim, "scale": None,
        "window": None, "q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "o", "q_norm": norm("qn"),
        "k_norm": norm("kn"), "position": PartSpec("rope_half_split", {"theta": 5000.0, "rotary_dim": head_dim}),
    })
    mixer = MIXERS.build(spec, env(dtype))
    w = bind(mixer, dtype, 11, 0.15)
    lengths = [19, 1, 6]
    cache, step = step_for([mixer.cache_spec()], lengths, dtype)
    x = rows(sum(lengths), hidden, dtype, 12)
    got = mixer.forward(x.cuda(), step, cache.view(0)).materialize()
    rnd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype).double())
    at = 0
    for i, n in enumerate(lengths):
        want = plain.plain_attention(x[at : at + n].double(), w["q"], w["k"], w["v"], w["o"], w["qn"], w["kn"], 1e-5,
                                     5000.0, heads, kv_heads, None, rnd)
        agree(got[at : at + n], want, dtype, f"attention sequence {i}")
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block(dtype):
    hidden = 64
    layer = LayerSpec(
        "L", PartSpec("pre_norm"),
        PartSpec("short_conv", {"hidden_size": hidden, "taps": 3, "bias": False, "in_proj": "i", "conv": "c", "conv_bias": None, "out_proj": "o"}),
        PartSpec("rmsnorm", {"tensor": "n1", "size": hidden, "eps": 1e-5}),
        PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 96, "gate": "g", "up": "u", "down": "d"}),
        PartSpec("rmsnorm", {"tensor": "n2", "size": hidden, "eps": 1e-5}),
    )
    block = BLOCKS.build(layer.block, env(dtype), layer)
    w = bind(block, dtype, 13, 0.2)
    cache, step = step_for([block.mixer_part().cache_spec()], [10], dtype)
    x = rows(10, hidden, torch.float32, 14)
    stream = Stream(x.clone().cuda())
    block.forward(stream, step, cache.view(0))
    rnd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype).double())
    h = x.double() + plain.plain_short_conv(rnd(plain.plain_rmsnorm(x.double(), w["n1"], 1e-5)), w["i"], w["c"], None, w["o"], rnd)
    out = h + plain.plain_swiglu(rnd(plain.plain_rmsnorm(h, w["n2"], 1e-5)), w["g"], w["u"], w["d"], rnd)
    got = stream.residual.double().cpu() + stream.take_pending().double().cpu()
    agree(got, out, dtype, "block output")
