"""What a mixer asks of the cache for its layer."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

PAGE = 64  # tokens per page; the kernel libraries are compiled with the same number and say so when loaded

# kind of cache -> first position that a query at position >= length can still see (pages wholly
# below it are given back to the pool at once). "full" keeps everything; "window" the last
# `window` positions. A mixer with another retention rule registers its kind here.
CACHE_KINDS: dict[str, Callable[["CacheNeed", int], int]] = {}


def register_cache_kind(kind: str, first_needed: Callable[["CacheNeed", int], int], replace: bool = False) -> None:
    if kind in CACHE_KINDS and not replace:
        raise ValueError(f"cache kind {kind!r} is already registered")
    CACHE_KINDS[kind] = first_needed


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values per position: `kind` says which positions must be kept ("full": all;
    "window": the last `window`; or a registered kind of the mixer's own)."""
    kind: str
    kv_heads: int
    head_dim: int
    window: int | None = None

    def __post_init__(self):
        if self.kind not in CACHE_KINDS:
            raise ValueError(f"cache kind {self.kind!r}; known: {', '.join(sorted(CACHE_KINDS))}")
        if (self.kind == "window") != (self.window is not None) and self.kind in ("full", "window"):
            raise ValueError("a window cache needs a window, a full cache has none")

    def first_needed(self, length: int) -> int:
        return CACHE_KINDS[self.kind](self, length)


register_cache_kind("full", lambda need, length: 0)
register_cache_kind("window", lambda need, length: length - need.window + 1)


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size (a recurrent mixer's carry): zeroed when a slot is opened."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32
