"""What a part says about a tensor it wants from the weight file."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TensorSpec:
    """One named tensor: its shape, and how random-weights mode draws it.

    init: the name of the law random-weights mode draws it by (weights.random_init.INIT_LAWS:
    "matrix" normal with std 0.02, "norm_weight" 1 + that, "integer_table"; parts may register more).
    optional: the file may leave it out; the part then finds no entry under the name.
    """
    name: str
    shape: tuple[int, ...]
    init: str = "matrix"
    optional: bool = False
