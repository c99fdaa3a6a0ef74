"""Writes tests/golden/plain_tiny.json: a few logits of the plain implementation on the two
tiny configurations.

The reference's own model code cannot be run here (it is Rust, no toolchain is installed, and
its LFM2 short-conv kernel exists only as Metal source), so these numbers are NOT outputs of
the reference: they pin the plain implementation under tests/ (which rests on the reference's
formulas) against accidental change.  Run from the repository root:

    python tests/golden/make_golden.py
"""

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import helpers  # noqa: E402
import plain_lfm2  # noqa: E402


def golden():
    out = {}
    for name in ("A", "B"):
        document, seed = helpers.TINY[name]
        tensors = helpers.make_tensors(document, seed)
        tokens = helpers.random_prompt(24, document["vocab_size"], 5)
        logits = plain_lfm2.plain_forward(document, tensors, tokens)
        picks = [0, 1, 7, 100, document["vocab_size"] - 1]
        out[name] = {
            "tokens": tokens,
            "rows": [0, 11, 23],
            "ids": picks,
            "logits": [[float(logits[r, i]) for i in picks] for r in (0, 11, 23)],
            "argmax": [int(logits[r].argmax()) for r in (0, 11, 23)],
            "greedy": plain_lfm2.plain_greedy(document, tensors, tokens[:9], 6),
        }
    return out


if __name__ == "__main__":
    with open(os.path.join(HERE, "plain_tiny.json"), "w") as f:
        json.dump(golden(), f, indent=1)
    print("wrote", os.path.join(HERE, "plain_tiny.json"))
