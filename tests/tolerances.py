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


def _ties_only(got, ref, bound):
    rows = torch.nonzero(got.argmax(-1) != ref.argmax(-1)).flatten()
    for r in rows.tolist():
        a, b = got[r].argmax().item(), ref[r].argmax().item()
        if abs(ref[r, a] - ref[r, b]) > 2 * bound:
            return False
    return True
