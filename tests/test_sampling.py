"""Host samplers: invariants the reference states (crates/shiso-engine/src/sampling.rs:4-17)."""

import numpy as np
import pytest

from shiso_llm_b200.sampling import (
    SamplingParams, Xorshift64Star, argmax, candidate_mask, keyed_sample, keyed_uniform, stream_sample, suppress,
)


def row(seed=0, n=500, scale=3.0):
    return (np.random.default_rng(seed).standard_normal(n) * scale).astype(np.float32)


def test_argmax_ties_to_the_lower_id_and_skips_non_finite():
    r = row()
    r[40] = r[400] = 99.0
    assert argmax(r) == 40
    r[3] = np.inf
    r[4] = np.nan
    assert argmax(r) == 40
    assert argmax(np.full(10, -np.inf, dtype=np.float32)) == 0


def test_greedy_draws_nothing_and_stochastic_draws_once():
    rng = Xorshift64Star(5)
    before = rng.state
    assert stream_sample(row(), SamplingParams(temperature=0.0), rng) == argmax(row())
    assert rng.state == before
    for params in (SamplingParams(temperature=0.7), SamplingParams(temperature=1.0, top_k=20),
                   SamplingParams(temperature=1.0, top_p=0.5), SamplingParams(temperature=1.0, min_p=0.1, top_k=50)):
        a, b = Xorshift64Star(9), Xorshift64Star(9)
        stream_sample(row(), params, a)
        b.next_u64()
        assert a.state == b.state


def test_xorshift_zero_seed_and_range():
    z = Xorshift64Star(0)
    assert z.state == 0x9E3779B97F4A7C15
    assert all(0.0 <= Xorshift64Star(s).next_f32() < 1.0 for s in range(1, 50))


def test_candidates():
    r = row(1)
    order = np.argsort(-r)
    m = candidate_mask(r, SamplingParams(temperature=1.0, top_k=5))
    assert set(np.nonzero(m)[0]) == set(order[:5])
    tie = r.copy()
    tie[order[5]] = tie[order[4]]  # a tie at the edge of top-k stays in
    assert candidate_mask(tie, SamplingParams(temperature=1.0, top_k=5)).sum() == 6
    p = np.exp((r - r.max()).astype(np.float64))
    p /= p.sum()
    m = candidate_mask(r, SamplingParams(temperature=1.0, top_p=0.6))
    kept = np.nonzero(m)[0]
    assert p[kept].sum() >= 0.6 and p[kept].sum() - p[kept].min() < 0.6 + 1e-6  # a minimal nucleus
    assert set(kept) == set(order[: len(kept)])
    m = candidate_mask(r, SamplingParams(temperature=0.5, min_p=0.2))
    assert set(np.nonzero(m)[0]) == set(np.nonzero(np.exp((r - r.max()) / 0.5) >= 0.2)[0])
    r[7] = -np.inf
    assert not candidate_mask(r, SamplingParams(temperature=1.0))[7]


def test_keyed_sample_depends_only_on_row_key_and_position():
    r = row(2)
    params = SamplingParams(temperature=0.8, top_k=40, top_p=0.9)
    a = keyed_sample(r, params, key=1, position=17)
    assert a == keyed_sample(r.copy(), params, key=1, position=17)
    picks = {keyed_sample(r, params, key=1, position=p) for p in range(64)}
    assert len(picks) > 3 and all(candidate_mask(r, params)[list(picks)])
    assert keyed_sample(r, SamplingParams(temperature=0.0), 1, 17) == argmax(r)


def test_keyed_sample_follows_the_softmax():
    r = np.array([2.0, 1.0, 0.0, -1.0, -np.inf], dtype=np.float32)
    params = SamplingParams(temperature=1.0)
    counts = np.zeros(5)
    n = 4000
    for position in range(n):
        counts[keyed_sample(r, params, key=3, position=position)] += 1
    p = np.exp(r[:4] - 2.0)
    p /= p.sum()
    assert counts[4] == 0 and np.abs(counts[:4] / n - p).max() < 0.03
    u = keyed_uniform(3, 5, np.arange(1000))
    assert u.min() > 0.0 and u.max() < 1.0 and abs(u.mean() - 0.5) < 0.05


def test_stream_sample_respects_top_k_and_top_p():
    r = row(4)
    order = list(np.argsort(-r))
    rng = Xorshift64Star(1)
    picks = {stream_sample(r, SamplingParams(temperature=1.5, top_k=3), rng) for _ in range(200)}
    assert picks <= set(order[:3]) and len(picks) > 1
    picks = {stream_sample(r, SamplingParams(temperature=1.0, top_p=1e-6), rng) for _ in range(50)}
    assert picks == {order[0]}


def test_parameter_clamps():
    assert SamplingParams(top_p=0.0).clamped()[2] == 1.0 and SamplingParams(top_p=1.5).clamped()[2] == 1.0
    assert SamplingParams(min_p=-1.0).clamped()[3] == 0.0 and SamplingParams(top_k=5000).clamped()[1] == 1024
    with pytest.raises(ValueError):
        SamplingParams(top_k=-1)


def test_suppressed_ids_are_never_picked():
    """``bad_token_ids`` become -inf before any pick, greedy or not; an id past the row is
    ignored and the caller's row is not changed (crates/shiso-engine/src/sampling.rs:156-174)."""
    r = row(6)
    best, second = np.argsort(-r)[:2]
    assert keyed_sample(r, SamplingParams(temperature=0.0, bad_token_ids=[int(best)]), 0, 0) == second
    assert r[best] > r[second]  # untouched
    cut = suppress(r, [int(best), 10**6])
    assert np.isneginf(cut[best]) and np.isfinite(cut).sum() == len(r) - 1
    bad = [int(i) for i in np.argsort(-r)[:20]]
    params = SamplingParams(temperature=1.2, top_k=30, bad_token_ids=bad, seed=3)
    picks = {keyed_sample(r, params, 3, p) for p in range(200)}
    assert picks and not picks & set(bad) and picks <= set(int(i) for i in np.argsort(-r)[20:50])
    rng = Xorshift64Star(2)
    assert not {stream_sample(r, params, rng) for _ in range(100)} & set(bad)
    assert keyed_sample(r, SamplingParams(temperature=0.0, bad_token_ids=list(range(len(r)))), 0, 0) == 0  # nothing left
    with pytest.raises(ValueError):
        SamplingParams(bad_token_ids=[-1])
