"""GPU time per launch, for finding where a step spends it.

While a region is open every call into the kernel library is bracketed by two CUDA events on
the launching stream, and the time filed under a launch is the time between them.  Steps run
kernel by kernel while a region is open (no graph replay, no lookahead), and the host takes
longer to issue a launch than the device to run a small kernel, so the device idles between
launches: a report therefore carries three figures per step - the sum of its rows, the span
from the first launch's start to the last one's end, and the host's wall time - and the
captured step a user sees is shorter than all three.  What the table is for is the shares.
(A kernel's row includes the few microseconds between the host's recording the first event and
its launch reaching the device; kernels of that size are better read from `ncu`.)  The
counterpart in the reference is its per-launch profiler behind ``--profile-dir``
(crates/shiso-core/src/profile.rs:1-80, crates/shiso-runtime/src/options.rs:139-146); rows are
keyed as there by what ran and at which shape, because the same kernel at a decode shape and
at a prompt shape is two questions.
"""

from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class LaunchRow:
    kernel: str
    shape: str
    launches: int = 0
    calls: int = 0
    total_us: float = 0.0

    @property
    def mean_us(self) -> float:
        return self.total_us / self.calls if self.calls else 0.0


@dataclass
class LaunchTable:
    """Samples of one kind of step (say, decode steps), added up by (kernel, shape)."""

    name: str
    rows: dict = field(default_factory=dict)
    steps: int = 0
    device_us: float = 0.0  # the rows' sum
    span_us: float = 0.0    # from the first launch's start to the last one's end, summed over steps
    wall_us: float = 0.0    # the host's clock around the same steps

    def add_step(self, samples, wall_us: float, span_us: float = 0.0) -> None:
        """``samples``: (kernel, shape, launches, microseconds) in launch order."""
        self.steps += 1
        self.wall_us += wall_us
        self.span_us += span_us
        for kernel, shape, launches, us in samples:
            row = self.rows.get((kernel, shape))
            if row is None:
                row = self.rows[(kernel, shape)] = LaunchRow(kernel, shape)
            row.launches += launches
            row.calls += 1
            row.total_us += us
            self.device_us += us

    def sorted_rows(self):
        return sorted(self.rows.values(), key=lambda r: -r.total_us)

    def report(self) -> dict:
        steps = max(1, self.steps)
        return {
            "steps": self.steps,
            "device_us_per_step": self.device_us / steps,
            "span_us_per_step": self.span_us / steps,
            "wall_us_per_step": self.wall_us / steps,
            "rows": [
                {
                    "kernel": r.kernel, "shape": r.shape, "launches_per_step": r.launches / steps,
                    "us_per_step": r.total_us / steps, "mean_us": r.mean_us,
                    "share": r.total_us / self.device_us if self.device_us else 0.0,
                }
                for r in self.sorted_rows()
            ],
        }

    def text(self) -> str:
        rep = self.report()
        lines = [
            f"{self.name}: {rep['steps']} steps; a step's launches take {rep['device_us_per_step']:.1f} us in all, "
            f"{rep['span_us_per_step']:.1f} us from the first one's start to the last one's end (kernel by kernel, "
            f"no graph), {rep['wall_us_per_step']:.1f} us by the host's clock",
            f"{'us/step':>10} {'share':>6} {'launches':>8} {'mean us':>8}  kernel",
        ]
        for r in rep["rows"]:
            shape = f" [{r['shape']}]" if r["shape"] else ""
            lines.append(f"{r['us_per_step']:10.1f} {100 * r['share']:5.1f}% {r['launches_per_step']:8.1f} {r['mean_us']:8.1f}  {r['kernel']}{shape}")
        return "\n".join(lines)


class StepProfiler:
    """Files every profiled step under its kind - ``decode`` when every sequence brings one
    token, ``prompt`` otherwise - and writes ``launches.json`` / ``launches.txt``."""

    def __init__(self, folder: Optional[str] = None):
        self.folder = folder
        self.tables = {"decode": LaunchTable("decode steps"), "prompt": LaunchTable("steps with prompt portions")}

    def add(self, kind: str, samples, wall_us: float, span_us: float = 0.0) -> None:
        self.tables[kind].add_step(samples, wall_us, span_us)

    def report(self) -> dict:
        return {kind: table.report() for kind, table in self.tables.items() if table.steps}

    def text(self) -> str:
        return "\n\n".join(table.text() for table in self.tables.values() if table.steps)

    def write(self) -> Optional[str]:
        if not self.folder:
            return None
        os.makedirs(self.folder, exist_ok=True)
        with open(os.path.join(self.folder, "launches.json"), "w") as f:
            json.dump(self.report(), f, indent=1)
        with open(os.path.join(self.folder, "launches.txt"), "w") as f:
            f.write(self.text() + "\n")
        return self.folder


class Region:
    """The open region of the kernel library: ``ops`` records an event before every call into
    the library (``before``) and one after every launch (``mark``)."""

    def __init__(self, torch):
        self.torch = torch
        self.marks = []  # (kernel, shape, launches, event before, event after)
        self.pending = None
        torch.cuda.synchronize()  # queued work is not counted
        self.began = time.perf_counter()

    def before(self) -> None:
        self.pending = self.torch.cuda.Event(enable_timing=True)
        self.pending.record()

    def mark(self, kernel: str, shape: str, launches: int) -> None:
        after = self.torch.cuda.Event(enable_timing=True)
        after.record()
        start = self.pending if self.pending is not None else (self.marks[-1][4] if self.marks else after)
        self.pending = None
        self.marks.append((kernel, shape, launches, start, after))

    def close(self):
        """(samples in launch order, the host's microseconds around the region, the microseconds
        from the first launch's start to the last one's end)."""
        self.torch.cuda.synchronize()
        wall_us = (time.perf_counter() - self.began) * 1e6
        samples = [(kernel, shape, launches, start.elapsed_time(after) * 1e3) for kernel, shape, launches, start, after in self.marks]
        span_us = self.marks[0][3].elapsed_time(self.marks[-1][4]) * 1e3 if self.marks else 0.0
        return samples, wall_us, span_us
