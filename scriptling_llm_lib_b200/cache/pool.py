"""Host-side bookkeeping of pages and slots: nothing is lost, held twice or freed twice."""
from __future__ import annotations


class CacheFull(RuntimeError):
    """The step needs more pages or slots than are free; nothing was changed."""


class FreeList:
    """Ids 0..n-1, handed out lowest first; `free` refuses an id that is not held."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def free(self, i: int) -> None:
        if not (0 <= i < self.n) or not self._held[i]:
            raise ValueError(f"{self.what} {i} is not held; it cannot be freed")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]
