"""Random weights: a model folder made from a configuration and a seed.

Every matrix is drawn from N(0, std) and every norm weight is 1.0 (or jittered
around 1.0 when a test wants a wrong norm weight to show), from one seeded
generator visited in sorted tensor-name order, so a (config, seed) pair always
yields the same folder.  The folder is written as ``config.json`` plus
``model.safetensors`` and is then loaded by name like any checkpoint.  The
reference has no such mode; its kernel tests use an LCG signal instead
(crates/shiso-kerneltest/src/oracle.rs:58-68).
"""

from __future__ import annotations

import json
import os
from typing import Iterable, Mapping

import torch

from .safetensors_io import write_safetensors
from .spec import INDEX, NORMAL, ONES, VECTOR, ZEROS, TensorSpec

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def random_tensors(
    specs: Iterable[TensorSpec],
    seed: int,
    std: float = 0.02,
    storage_dtype: str = "bfloat16",
    norm_jitter: float = 0.0,
) -> dict[str, torch.Tensor]:
    if storage_dtype not in _STORAGE:
        raise ValueError(f"storage dtype {storage_dtype!r}: expected one of {sorted(_STORAGE)}")
    dtype = _STORAGE[storage_dtype]
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out = {}
    for spec in sorted(specs, key=lambda s: s.name):
        if spec.role == INDEX:
            raise ValueError(f"{spec.name}: integer tables have no random initialisation")
        if spec.init == NORMAL:
            t = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * std
        elif spec.init == ONES:
            t = torch.ones(spec.shape, dtype=torch.float32)
            if norm_jitter:
                t = t + norm_jitter * torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        elif spec.init == ZEROS:
            t = torch.zeros(spec.shape, dtype=torch.float32)
        else:
            raise ValueError(f"{spec.name}: unknown initialisation {spec.init!r}")
        out[spec.name] = t.to(dtype)
    return out


def write_model_folder(model_dir: str, config_document: Mapping, tensors: Mapping[str, torch.Tensor]) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config_document), f, indent=2)
        f.write("\n")
    write_safetensors(os.path.join(model_dir, "model.safetensors"), dict(tensors), {"format": "pt"})


def random_device_tensors(specs: Iterable[TensorSpec], seed: int, compute_dtype, device, std: float = 0.02) -> dict:
    """Random weights made on the device, in the types the loader would hand out (matrices
    in the compute type, vectors in float32): the same distribution as ``random_tensors``
    without the trip through a file, for benchmarks of large shapes."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for spec in sorted(specs, key=lambda s: s.name):
        dtype = torch.float32 if spec.role == VECTOR else compute_dtype
        if spec.init == NORMAL:
            t = torch.empty(spec.shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=gen)
        elif spec.init == ONES:
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
        else:
            t = torch.zeros(spec.shape, dtype=torch.float32, device=device)
        out[spec.name] = t.to(dtype)
    return out
