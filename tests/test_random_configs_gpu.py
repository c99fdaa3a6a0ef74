"""Configurations and scheduler settings drawn at random (from fixed seeds) through the entry point.

The two tiny configurations of ``helpers`` are fixed; this file draws others: head sizes in steps
of 16, any number of heads and groups, widths and vocabularies that are no power of two, every
convolution length, pages of 4 to 32 tokens, and for each a scheduler of its own (live requests,
token budget, portion size, a pool that holds barely one request so that requests are put back,
captured graphs and lookahead on or off, greedy or temperature sampling).  Every logits row a token
was picked from is compared with the plain implementation on that request's own tokens, in 32-bit
and in bfloat16, so a wrong row cannot hide behind a continuation that differs.  The larger
configurations have the widths at which the tensor-memory kernels run (heads of 64, prompts of a
thousand tokens, dozens of live requests).
"""

import random

import pytest
import torch

import helpers
import plain_lfm2
from shiso_llm_b200 import LLM, SamplingParams
from tolerances import check_logits

pytestmark = pytest.mark.gpu


def _layer_types(rng, layers, both):
    types = [rng.choice(["conv", "full_attention"]) for _ in range(layers)]
    if "full_attention" not in types:
        types[rng.randrange(layers)] = "full_attention"
    if both and "conv" not in types:
        types[rng.randrange(layers)] = "conv"
    return types


def small_config(rng):
    head_dim = rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128])
    heads = rng.choice([1, 2, 3, 4, 5, 6, 8])
    layers = rng.randint(2, 5)
    return {
        "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
        "vocab_size": rng.choice([131, 500, 777, 1000, 1531, 2048, 3001]),
        "hidden_size": heads * head_dim, "num_hidden_layers": layers,
        "num_attention_heads": heads,
        "num_key_value_heads": rng.choice([d for d in range(1, heads + 1) if heads % d == 0]),
        "layer_types": _layer_types(rng, layers, False),
        "conv_L_cache": rng.randint(2, 5), "conv_bias": rng.random() < 0.5,
        "block_ff_dim": rng.choice([72, 150, 192, 264, 384, 520, 1002]),
        "block_auto_adjust_ff_dim": rng.random() < 0.5, "block_multiple_of": rng.choice([8, 24, 64, 256]),
        "block_ffn_dim_multiplier": rng.choice([1.0, 0.75, 1.3]),
        "norm_eps": rng.choice([1e-5, 1e-6, 3e-5]), "rope_theta": rng.choice([1e4, 1e6, 5e5]),
        "tie_embedding": rng.random() < 0.5,
    }


def large_config(rng):
    head_dim = rng.choice([64, 64, 64, 32, 128, 96])
    heads = rng.choice([8, 12, 16, 24, 32])
    layers = rng.randint(2, 4)
    return {
        "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
        "vocab_size": rng.choice([8192, 32003, 65536, 10007]),
        "hidden_size": heads * head_dim, "num_hidden_layers": layers,
        "num_attention_heads": heads,
        "num_key_value_heads": rng.choice([d for d in range(1, heads + 1) if heads % d == 0]),
        "layer_types": _layer_types(rng, layers, True),
        "conv_L_cache": rng.randint(2, 4), "conv_bias": rng.random() < 0.3,
        "block_ff_dim": rng.choice([1000, 1536, 2304, 4608, 5632, 3000]),
        "block_auto_adjust_ff_dim": False, "block_multiple_of": 256, "block_ffn_dim_multiplier": 1.0,
        "norm_eps": rng.choice([1e-5, 1e-6]), "rope_theta": rng.choice([1e4, 1e6]),
        "tie_embedding": rng.random() < 0.7,
    }


def draw(seed, large):
    rng = random.Random(1000 + seed)
    document = large_config(rng) if large else small_config(rng)
    page = rng.choice([4, 8, 16, 32])
    lengths = [rng.choice([1, 2, 5, 17, 33, 64, 100, 150, 257] + ([600, 1100] if large else []))
               for _ in range(rng.randint(3, 30 if large else 14))]
    new = rng.choice([8, 20, 40])
    ctx = -(-(max(lengths) + new) // page) * page
    seqs = rng.choice([1, 2, 4, 8, 12] + ([24, 70] if large else []))
    pool = ctx + (rng.choice([0, 64, 128]) if rng.random() < 0.5 else seqs * ctx)
    settings = dict(
        ctx=ctx, page_size=page, max_num_seqs=seqs,
        max_num_batched_tokens=rng.choice([16, 32, 100, 256, 512] + ([1024, 2048] if large else [])),
        prefill_chunk=rng.choice([None, 2, 13, 64]), kv_cache_tokens=-(-pool // page) * page,
        cuda_graphs=rng.random() < 0.7, lookahead=rng.random() < 0.7, allow_small_pool=True,
    )
    return document, lengths, new, settings, rng.choice([0.0, 0.0, 0.8])


CASES = [pytest.param(seed, False, id=f"small-{seed}") for seed in (0, 3, 5, 8, 13, 21, 34, 55)] + [
    pytest.param(seed, True, id=f"large-{seed}") for seed in (1, 4, 39, 115, 295, 328)
]


@pytest.mark.parametrize("seed,large", CASES)
def test_a_drawn_configuration_under_a_drawn_scheduler(tmp_path, seed, large):
    document, lengths, new, settings, temperature = draw(seed, large)
    tensors = helpers.make_folder(tmp_path, document, seed)
    on_device = {name: t.cuda().double() for name, t in tensors.items()}
    prompts = [helpers.random_prompt(n, document["vocab_size"], 100 * seed + i) for i, n in enumerate(lengths)]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(str(tmp_path), dtype=dtype, **settings)
        seen = {}  # (request, position) -> the logits row its token was picked from

        def tap(plan, logits, seen=seen):
            rows = logits.float().cpu()
            for row, entry in zip(rows, [e for e in plan.entries if e.samples]):
                seen[(entry.request.id, entry.start + entry.count - 1)] = row

        llm.logits_tap = tap
        outs = llm.generate(prompts, SamplingParams(temperature=temperature, seed=seed, max_new_tokens=new))
        for out, prompt in zip(outs, prompts):
            assert len(out.token_ids) == new and out.finish_reason == "length"
            places = range(len(prompt) - 1, len(prompt) + new - 1)
            want = plain_lfm2.plain_forward(document, on_device, prompt + out.token_ids[:-1], device="cuda", rows=places).cpu()
            got = torch.stack([seen[(out.request_id, p)] for p in places])
            check_logits(got, want, dtype, f"seed {seed} {dtype}, the request of {len(prompt)} tokens under {settings}")
        llm.engine.cache.check()
        assert llm.engine.cache.slots.free_slots == settings["max_num_seqs"]
        del llm
