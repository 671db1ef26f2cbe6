"""What a model expects to find in its weight files: one TensorSpec per tensor."""
from __future__ import annotations

from dataclasses import dataclass

MATRIX = "matrix"      # operand of a matrix product or the embedding table: held in the engine's dtype
VECTOR = "vector"      # norm weights and other small tensors: 32-bit if stored so, else as stored
TABLE = "table"        # integer tables: held as int32

NORMAL = "normal"            # random mode: N(0, 0.02)
NORM_WEIGHT = "norm_weight"  # random mode: 1 + U(-0.1, 0.1)


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple
    role: str = MATRIX
    init: str = NORMAL
    optional: bool = False      # may be absent from the files (a tied output head)
    ignored: bool = False       # may be present but is not used (a stored copy of a tied head)
