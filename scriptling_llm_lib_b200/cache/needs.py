"""What a mixer asks of the cache for its layer."""
from __future__ import annotations

from dataclasses import dataclass

import torch

PAGE = 64  # tokens per page; the kernels are compiled with the same number


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values for every position ("full") or for the last `window` positions ("window")."""
    kind: str
    kv_heads: int
    head_dim: int
    window: int | None = None

    def __post_init__(self):
        if self.kind not in ("full", "window"):
            raise ValueError(f"cache kind {self.kind!r}; known: full, window")
        if (self.kind == "window") != (self.window is not None):
            raise ValueError("a window cache needs a window, a full cache has none")


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size (a recurrent mixer's carry): zeroed when a slot is opened."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32
