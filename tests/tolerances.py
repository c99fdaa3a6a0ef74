"""Tolerances of the model-level comparisons, fixed before any GPU run.

float32: the plain implementation evaluated in float32 instead of float64 moves the tiny
models' logits by about 5e-7 (logits are of order 1); the engine orders its sums
differently and uses rsqrtf/sincosf/expf, so 2e-5 * max(1, max|logit|) leaves a factor of
a few tens and is far below what any indexing fault produces.

bfloat16: rounding the plain implementation's activations to bfloat16 at the points where
the engine stores them moves the logits by at most 0.033 * std and 0.006 * std in the
root mean square.  The budget is three times that: max 0.1 * std, rms 0.02 * std, and the
best token must agree wherever the reference's lead over the runner-up exceeds twice
the max budget.

bfloat16 at full depth (``check_logits_deep``, the 16-layer LFM2-1.2B shape): the same
imitation - the plain implementation with its activations rounded to bfloat16 where the engine
stores them - measured on the CPU at 192 and 640 positions gives, against float64: error rms
0.0245 * std in every row, max 0.140 * std (what a Gaussian of that rms yields over 10^7
values), worst change of log-probability over the plain implementation's top 64 tokens 0.070
and 0.092, smallest overlap of the two top-64 sets 58 of 64, argmax equal on 96 % of the rows
(the random model's lead over the runner-up is often a hundredth of std).  Budgets are twice
the imitation's figures: rms 0.05 * std per row, max 0.3 * std, log-probability 0.2 (entries
below -12 are ignored, as in crates/shiso-models/tests/lfm2_forward.rs:44-48), overlap 52, and
the best token must agree where the lead exceeds 0.6 * std.  A fault of indexing (a wrong key,
page or state) moves a row by the order of std itself.
"""

import torch

FP32_REL = 2e-5
BF16_MAX_OVER_STD = 0.1
BF16_RMS_OVER_STD = 0.02


def check_logits(got, ref, dtype, what=""):
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = (got - ref).abs()
    if dtype == "float32":
        bound = FP32_REL * max(1.0, ref.abs().max().item())
        worst = err.max().item()
        if worst > bound:
            at = torch.nonzero(err > bound)[0].tolist()
            raise AssertionError(f"{what}: float32 logits differ by {worst:.3e} > {bound:.3e}; first bad (row, id) = {at}")
        assert (got.argmax(-1) == ref.argmax(-1)).all() or _ties_only(got, ref, bound), f"{what}: argmax differs"
    else:
        std = ref.std().item()
        worst, rms = err.max().item(), err.pow(2).mean().sqrt().item()
        if worst > BF16_MAX_OVER_STD * std:
            bad_rows = torch.nonzero(err.max(-1).values > BF16_MAX_OVER_STD * std).flatten().tolist()
            raise AssertionError(
                f"{what}: bfloat16 logits differ by {worst:.3e} > {BF16_MAX_OVER_STD * std:.3e}; first bad rows {bad_rows[:8]}"
            )
        assert rms <= BF16_RMS_OVER_STD * std, f"{what}: bfloat16 rms error {rms:.3e} > {BF16_RMS_OVER_STD * std:.3e}"
        top2 = ref.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 2 * BF16_MAX_OVER_STD * std
        assert (got.argmax(-1)[clear] == ref.argmax(-1)[clear]).all(), f"{what}: argmax differs on a clear row"


DEEP_RMS_OVER_STD = 0.05
DEEP_MAX_OVER_STD = 0.3
DEEP_LOGP = 0.2
DEEP_TOP = 64
DEEP_OVERLAP = 52
DEEP_LOGP_FLOOR = -12.0


def check_logits_deep(got, ref, dtype="bfloat16", what=""):
    """The bfloat16 budget of the full-depth model: per-row rms and max error, top-64 overlap
    and the worst change of log-probability over the reference's top 64."""
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    std = ref.std().item()
    err = (got - ref).abs()
    row_rms = err.pow(2).mean(-1).sqrt()
    worst_row = int(row_rms.argmax())
    assert row_rms.max().item() <= DEEP_RMS_OVER_STD * std, (
        f"{what}: row {worst_row} has rms error {row_rms.max().item() / std:.4f} * std > {DEEP_RMS_OVER_STD}"
    )
    assert err.max().item() <= DEEP_MAX_OVER_STD * std, f"{what}: max error {err.max().item() / std:.4f} * std > {DEEP_MAX_OVER_STD}"
    logp_ref, logp_got = torch.log_softmax(ref, -1), torch.log_softmax(got, -1)
    top = ref.topk(DEEP_TOP, -1).indices
    kept = logp_ref.gather(1, top) >= DEEP_LOGP_FLOOR
    delta = (logp_ref.gather(1, top) - logp_got.gather(1, top)).abs() * kept
    assert delta.max().item() <= DEEP_LOGP, f"{what}: log-probability of a top-{DEEP_TOP} token moved by {delta.max().item():.4f} > {DEEP_LOGP}"
    top_got = got.topk(DEEP_TOP, -1).indices
    overlap = min(len(set(a.tolist()) & set(b.tolist())) for a, b in zip(top, top_got))
    assert overlap >= DEEP_OVERLAP, f"{what}: only {overlap} of the top {DEEP_TOP} tokens are shared"
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2 * DEEP_MAX_OVER_STD * std
    assert (got.argmax(-1)[clear] == ref.argmax(-1)[clear]).all(), f"{what}: argmax differs on a clear row"
    return {"rms_over_std": row_rms.max().item() / std, "max_over_std": err.max().item() / std,
            "logp": delta.max().item(), "overlap": overlap}


def _ties_only(got, ref, bound):
    rows = torch.nonzero(got.argmax(-1) != ref.argmax(-1)).flatten()
    for r in rows.tolist():
        a, b = got[r].argmax().item(), ref[r].argmax().item()
        if abs(ref[r, a] - ref[r, b]) > 2 * bound:
            return False
    return True
