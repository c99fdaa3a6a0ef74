"""Host samplers over one row of float32 logits.

``argmax`` and ``keyed_sample`` state, in plain NumPy, exactly the rules the device
kernels implement, and serve when logits are already on the host.  ``stream_sample`` is
the reference's sequential sampler driven by its xorshift64* stream
(crates/shiso-engine/src/sampling.rs:432-633; crates/shiso-core/src/ids.rs:200-252); it
exists only here, because a stream that advances draw by draw cannot be shared by the
rows of a batch.

The keyed rule (crates/shiso-engine/src/sampling.rs:720-912): the token is
argmax(logit / T + G(key, position, id)) over the allowed candidates, G a Gumbel variate
from a hash of (key, position, id), so the draw does not depend on the batch or on how
the work was cut.  Candidates are described by thresholds here (ties stay in):
top-k keeps logits >= the k-th largest; top-p keeps logits >= the logit at which the
mass summed from the top over the top-k set first reaches top_p of it; min-p keeps
exp((l - max) / T) >= min_p.  Masses are 2^-40 fixed-point integers.
"""

from __future__ import annotations

import numpy as np

from .params import SamplingParams

_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_POSMUL = np.uint64(0xD1B54A32D192ED03)


def _mix(x):
    x = x ^ (x >> np.uint64(30))
    x = x * _M1
    x = x ^ (x >> np.uint64(27))
    x = x * _M2
    return x ^ (x >> np.uint64(31))


def keyed_uniform(key: int, position: int, ids: np.ndarray) -> np.ndarray:
    """Uniforms in (0, 1) from (key, position, id): three rounds of the splitmix64
    finalizer, top 24 bits, offset half a step (sampling.rs:893-912)."""
    with np.errstate(over="ignore"):
        x = _mix(np.uint64(key & 0xFFFFFFFFFFFFFFFF) + _GOLDEN)
        x = _mix(x ^ (np.uint64(position) * _POSMUL))
        x = _mix(x ^ ids.astype(np.uint64))
    return ((x >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)


def argmax(logits) -> int:
    """Lowest id attaining the highest finite logit; 0 when nothing is finite."""
    row = np.asarray(logits, dtype=np.float32)
    finite = np.isfinite(row)
    if not finite.any():
        return 0
    return int(np.argmax(np.where(finite, row, -np.inf)))


def suppress(logits, ids) -> np.ndarray:
    """A copy of the row with -inf at every id of ``ids``, so that no pick after it can choose
    one; an id past the row is ignored (crates/shiso-engine/src/sampling.rs:156-174)."""
    row = np.array(logits, dtype=np.float32, copy=True)
    for i in ids:
        if 0 <= i < row.shape[0]:
            row[i] = -np.inf
    return row


def _fixed_mass(scaled: np.ndarray) -> np.ndarray:
    return (np.exp(scaled.astype(np.float32)).astype(np.float32) * np.float32(1099511627776.0)).astype(np.uint64)


def candidate_mask(logits, params: SamplingParams) -> np.ndarray:
    """Which ids the request's top-k, top-p and min-p allow."""
    row = np.asarray(logits, dtype=np.float32)
    temperature, top_k, top_p, min_p = params.clamped()
    finite = np.isfinite(row)
    keep = finite.copy()
    top = row[argmax(row)]
    inv_t = np.float32(1.0) / np.float32(temperature)
    if top_k > 0 and finite.sum() > top_k:
        kth = np.sort(row[finite])[::-1][top_k - 1]
        keep &= row >= kth
    if top_p < 1.0:
        scaled = (row - top) * inv_t
        mass = np.where(keep, _fixed_mass(np.where(keep, scaled, 0)), np.uint64(0))
        total = int(mass.sum(dtype=np.uint64))
        target = int(np.ceil(np.float64(np.float32(top_p)) * np.float64(total)))
        order = np.argsort(-row[keep], kind="stable")
        values = row[keep][order]
        running = np.cumsum(mass[keep][order].astype(object))
        reached = np.nonzero(running >= target)[0]
        cut = values[reached[0]] if len(reached) else values[-1]
        keep &= row >= cut
    if min_p > 0.0:
        scaled = (row - top) * inv_t
        floor = np.log(np.float32(min_p))
        best = argmax(row)
        allowed = scaled >= floor
        allowed[best] = True
        keep &= allowed
    return keep


def keyed_sample(logits, params: SamplingParams, key: int, position: int) -> int:
    row = np.asarray(logits, dtype=np.float32)
    if params.bad_token_ids:
        row = suppress(row, params.bad_token_ids)
    if params.greedy or not np.isfinite(row).any():
        return argmax(row)
    keep = candidate_mask(row, params)
    ids = np.nonzero(keep)[0]
    top = row[argmax(row)]
    inv_t = np.float32(1.0) / np.float32(params.temperature)
    u = keyed_uniform(key, position, ids)
    score = (row[ids] - top) * inv_t - np.log(-np.log(u))
    return int(ids[int(np.argmax(score))])  # first maximum: the lower id on a tie


class Xorshift64Star:
    """The reference's stream: xorshift64* with a zero seed replaced by the golden-ratio
    constant; a uniform is the top 24 bits over 2^24 (crates/shiso-core/src/ids.rs:200-252)."""

    def __init__(self, seed: int):
        self.state = (seed & 0xFFFFFFFFFFFFFFFF) or 0x9E3779B97F4A7C15

    def next_u64(self) -> int:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / 16777216.0


def stream_sample(logits, params: SamplingParams, rng: Xorshift64Star) -> int:
    """Temperature softmax with optional top-k, min-p and top-p, one uniform per sample,
    none for greedy: keep the k largest (ties to the lower id), weights
    exp((l - max) / T), stop at the min-p floor, stop once the cumulative share reaches
    top_p, draw r = u * kept mass and walk in descending order
    (crates/shiso-engine/src/sampling.rs:521-591); without top-k and with top_p >= 1 the
    walk is in vocabulary order (sampling.rs:432-478)."""
    row = np.asarray(logits, dtype=np.float32)
    if params.bad_token_ids:
        row = suppress(row, params.bad_token_ids)
    finite = np.isfinite(row)
    if params.greedy or not finite.any():
        return argmax(row)
    temperature, top_k, top_p, min_p = params.clamped()
    best = argmax(row)
    ids = np.nonzero(finite)[0]
    weights = np.exp((row[ids] - row[best]) / np.float32(temperature)).astype(np.float32)
    if top_k == 0 and top_p >= 1.0 and min_p == 0.0:
        total = np.float32(weights.sum(dtype=np.float32))
        r = np.float32(rng.next_f32()) * total
        for i, w in zip(ids, weights):
            r -= w
            if r <= 0:
                return int(i)
        return int(ids[-1])
    order = np.lexsort((ids, -row[ids]))  # descending logit, ties to the lower id
    if top_k > 0:
        order = order[: min(top_k, len(order))]
    ids, weights = ids[order], weights[order]
    total = float(weights.sum(dtype=np.float64))
    kept, kept_mass = 0, 0.0
    for i, w in enumerate(weights):
        if i > 0 and w / total < min_p * (weights[0] / total):
            break
        kept_mass += float(w)
        kept += 1
        if kept_mass / total >= top_p:
            break
    r = rng.next_f32() * kept_mass
    for i in range(kept):
        r -= float(weights[i])
        if r <= 0:
            return int(ids[i])
    return int(ids[kept - 1])
