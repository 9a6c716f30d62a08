"""What a part says about each tensor it needs."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One named tensor of a checkpoint.

    role      "matrix": operand of a matrix product, held in the compute dtype;
              "vector": gain or bias, a tensor stored in 32-bit stays in 32-bit;
              "table":  integer table, held as int32.
    init      how the random-weights mode draws it: "normal" (N(0, std)),
              "gain" (1 + N(0, std)), "zeros" or "ones".
    optional  may be absent from the checkpoint (the part says what it does then).
    same_as   when present in the checkpoint it must equal this other tensor
              (a head tied to the embedding that is stored a second time).
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    optional: bool = False
    same_as: str = ""
