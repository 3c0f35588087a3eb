"""What a part says about a tensor it wants from the weight file."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TensorSpec:
    """One named tensor: its shape, and how random-weights mode draws it.

    init: "matrix" (normal, std 0.02), "norm_weight" (1 + normal*0.02), "integer_table".
    optional: the file may leave it out (the loader then gives None); alias_of names the tensor
    used in its place (a tied output head reads the embedding, as the reference falls back to the
    embedding when output.weight is absent, model_f32.go:147-162).
    """
    name: str
    shape: tuple[int, ...]
    init: str = "matrix"
    optional: bool = False
