"""Weights by tensor name, checked against what the model's parts ask for.

Every part lists the tensors it needs (``TensorSpec``).  The loader opens every
``*.safetensors`` file of the model folder, compares the directory with that
list, and raises ONE ``WeightError`` that names every missing tensor, every
tensor nobody asked for, every wrong shape and every unusable dtype, before a
byte is copied to the device.  The reference stops at the first absent tensor
(crates/shiso-models/src/lfm2/model.rs:253-259) and checks shapes tensor by
tensor (model.rs:284-300); here the whole picture is reported at once.

Precision: 16-bit floating tensors are kept in bfloat16 when the compute dtype
is bfloat16 and widened when it is float32; a tensor stored in 32-bit stays in
32-bit; small vectors (norm weights, conv taps, biases) are handed to the
kernels as float32, which holds every bfloat16 value exactly; integer tables
become int32.
"""

from __future__ import annotations

import glob
import os
from typing import Iterable

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile
from .spec import INDEX, MATRIX, VECTOR, TensorSpec

_FLOATS = (torch.float32, torch.bfloat16, torch.float16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    """The checkpoint does not hold exactly the tensors the model needs."""

    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_dtype, other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        self.other = list(other)
        lines = [f"{where}: the checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name}: expected {list(want)}, file has {list(got)}")
        for name, why in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name}: {why}")
        for why in self.other:
            lines.append(f"  {why}")
        super().__init__("\n".join(lines))


def target_dtype(spec: TensorSpec, stored: torch.dtype, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor has on the device."""
    if spec.role == INDEX:
        return torch.int32
    if spec.role == VECTOR:
        return torch.float32
    if stored == torch.float32 or compute_dtype == torch.float32:
        return torch.float32
    return torch.bfloat16


def weight_files(model_dir: str) -> list[str]:
    return sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))


def load_weights(
    model_dir: str,
    specs: Iterable[TensorSpec],
    compute_dtype: torch.dtype,
    device,
) -> dict[str, torch.Tensor]:
    """Loads exactly the tensors ``specs`` names; anything else is an error."""
    specs = list(specs)
    paths = weight_files(model_dir)
    if not paths:
        raise WeightError(model_dir, [s.name for s in specs], [], [], [], ["no *.safetensors file in the folder"])

    files = []
    home: dict[str, SafetensorsFile] = {}
    other = []
    for path in paths:
        try:
            f = SafetensorsFile(path)
        except SafetensorsError as e:
            raise WeightError(model_dir, [], [], [], [], [str(e)]) from e
        files.append(f)
        for name in f.names():
            if name in home:
                other.append(f"tensor {name} appears in {os.path.basename(home[name].path)} and {os.path.basename(path)}")
            home[name] = f

    wanted = {s.name: s for s in specs}
    if len(wanted) != len(specs):
        seen, twice = set(), []
        for s in specs:
            if s.name in seen:
                twice.append(s.name)
            seen.add(s.name)
        other.append("the model asks twice for: " + ", ".join(sorted(set(twice))))

    missing = sorted(n for n in wanted if n not in home)
    unexpected = sorted(n for n in home if n not in wanted)
    wrong_shape, wrong_dtype = [], []
    for name, spec in wanted.items():
        if name not in home:
            continue
        entry = home[name].entries[name]
        if entry.shape != tuple(spec.shape) and entry.shape not in spec.alt_shapes:
            wrong_shape.append((name, spec.shape, entry.shape))
        if spec.role == INDEX:
            if entry.dtype not in _INTS:
                wrong_dtype.append((name, f"an integer table stored as {entry.dtype}"))
        elif entry.dtype not in _FLOATS:
            wrong_dtype.append((name, f"stored as {entry.dtype}; expected F32, BF16 or F16"))
    if missing or unexpected or wrong_shape or wrong_dtype or other:
        for f in files:
            f.close()
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype, other)

    out: dict[str, torch.Tensor] = {}
    for name, spec in wanted.items():
        view = home[name].tensor(name)
        dtype = target_dtype(spec, view.dtype, compute_dtype)
        tensor = view.to(device=device, dtype=dtype, copy=True).reshape(spec.shape).contiguous()
        out[name] = tensor
    for f in files:
        f.close()
    return out
