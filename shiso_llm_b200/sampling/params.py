"""Per-request sampling parameters.

Field names and meanings follow the reference's ``SamplingParams`` and request fields
(crates/shiso-core/src/model.rs:530-567; crates/shiso-ir/src/request.rs:33-85):
``temperature <= 0`` means greedy and draws nothing; ``top_k`` 0 / None is off;
``top_p`` outside (0, 1] is treated as 1; ``min_p`` below 0 as 0.  The neutral setting
is (1.0, off, 1.0, 0.0).  ``bad_token_ids`` are ids the request may never emit: their
logits are set to -inf before any pick, greedy or not
(crates/shiso-engine/src/sampling.rs:156-174).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

TOP_K_LIMIT = 1024  # crates/shiso-engine/src/sampling.rs:27


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0
    max_new_tokens: int = 16
    stop_token_ids: Sequence[int] = field(default_factory=tuple)
    ignore_eos: bool = False
    bad_token_ids: Sequence[int] = field(default_factory=tuple)

    def __post_init__(self):
        if self.max_new_tokens < 0:
            raise ValueError(f"max_new_tokens = {self.max_new_tokens} must not be negative")
        if self.top_k is not None and self.top_k < 0:
            raise ValueError(f"top_k = {self.top_k} must not be negative")
        self.bad_token_ids = tuple(int(t) for t in self.bad_token_ids)
        if any(t < 0 for t in self.bad_token_ids):
            raise ValueError(f"bad_token_ids = {self.bad_token_ids}: token ids are not negative")

    @property
    def greedy(self) -> bool:
        return not self.temperature > 0.0

    def clamped(self):
        """(temperature, top_k, top_p, min_p) as the samplers use them
        (clamps of crates/shiso-engine/src/sampling.rs:607-625)."""
        top_p = self.top_p if 0.0 < self.top_p <= 1.0 else 1.0
        min_p = max(self.min_p, 0.0)
        top_k = min(int(self.top_k or 0), TOP_K_LIMIT)
        return float(self.temperature), top_k, float(top_p), float(min_p)
