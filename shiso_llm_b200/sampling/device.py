"""Sampling on the device for the rows of one step."""

from __future__ import annotations

from typing import Sequence

import torch

from .params import SamplingParams


class DeviceSampler:
    """Turns per-request parameters into the arrays the sampling kernel reads and picks one
    token per logits row.  Rows that are all greedy take the argmax kernel."""

    def __init__(self, ops, device):
        self.ops = ops
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], positions: Sequence[int]) -> list[int]:
        """``logits[R, V]`` float32 on the device; ``positions[r]`` is the position the
        sampled token will occupy in its sequence.  Returns host ints."""
        return self.sample_into(logits, params, positions, None).tolist()

    def sample_into(self, logits, params: Sequence[SamplingParams], positions: Sequence[int], out,
                    status_out=None) -> torch.Tensor:
        """The same, leaving the picks on the device: in ``out`` (int32 ``[R]``) when one is
        given.  Nothing waits for the device.  Rows whose request names ``bad_token_ids`` have
        those logits set to -inf first, in place.  ``status_out`` (one int32 on the device) is
        handed to the picking kernel, which leaves the status word of the kernels' bounded
        waits there (``ops.check_kernel_status``)."""
        if logits.shape[0] != len(params):
            raise ValueError(f"{logits.shape[0]} rows of logits for {len(params)} requests")
        extra = {} if status_out is None else {"status_out": status_out}
        if any(p.bad_token_ids for p in params):
            pairs = [(r, t) for r, p in enumerate(params) for t in p.bad_token_ids]
            both = torch.tensor(pairs, dtype=torch.int32).t().contiguous().to(self.device, non_blocking=True)
            self.ops.suppress(logits, both[0], both[1])
        if all(p.greedy for p in params):
            return self.ops.argmax(logits, out, **extra)
        clamped = [p.clamped() for p in params]
        host = torch.tensor(
            [[c[0] if not p.greedy else 0.0, c[2], c[3]] for c, p in zip(clamped, params)], dtype=torch.float32
        )
        ints = torch.tensor([[c[1], pos] for c, pos in zip(clamped, positions)], dtype=torch.int32)
        keys = torch.tensor([_as_signed(p.seed) for p in params], dtype=torch.int64)
        dev = self.device
        floats = host.to(dev, non_blocking=True)
        ints = ints.to(dev, non_blocking=True)
        picks = self.ops.sample(
            logits,
            floats[:, 0].contiguous(),
            ints[:, 0].contiguous(),
            floats[:, 1].contiguous(),
            floats[:, 2].contiguous(),
            keys.to(dev, non_blocking=True),
            ints[:, 1].contiguous(),
            out,
            **extra,
        )
        return picks


def _as_signed(seed: int) -> int:
    seed &= 0xFFFFFFFFFFFFFFFF
    return seed - (1 << 64) if seed >= (1 << 63) else seed
