"""What a part says about each tensor it needs."""

from __future__ import annotations

from dataclasses import dataclass

MATRIX = "matrix"  # a projection or embedding table: kept in the compute dtype when stored in 16 bits
VECTOR = "vector"  # norm weights, conv taps, biases: small, read in 32-bit by the kernels
INDEX = "index"  # integer tables: kept as int32

NORMAL = "normal"
ONES = "ones"
ZEROS = "zeros"


@dataclass(frozen=True)
class TensorSpec:
    """One tensor of the checkpoint: its name, exact shape, role and how random weights fill it.

    ``alt_shapes`` lists other stored shapes with the same element count that mean the
    same tensor (a depthwise conv weight stored ``[H, 1, L]`` for ``[H, L]``).
    """

    name: str
    shape: tuple[int, ...]
    role: str = MATRIX
    init: str = NORMAL
    alt_shapes: tuple[tuple[int, ...], ...] = ()
