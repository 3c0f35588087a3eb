"""The cache: a slot for each live sequence, paged keys and values for each cache unit, and
per-sequence state of fixed size beside them.

The reference keeps, per layer and KV head, one growing array of rotated keys and one of values
for its single sequence (float32_ops.go:11-14, model_f32.go:310-317, :445-448). Here a *cache
unit* is what one entry of the model's schedule writes; units with the same need (all keys / a
window of them, same head count and width) form a *group* with storage of its own:
`k, v: [unit, page, kv_head, PAGE, head_dim]`. A sequence holds a slot; in each group the slot owns
a list of pages, position p living in page p // PAGE. One page id serves all units of the group.
Pages come from the group's pool as the sequence grows and go back when it is closed, or, in a
window group, as soon as no later query can see them. Nothing relies on cleared memory: every read
is bounded by the sequence's length.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .needs import PAGE, CacheNeed, StateNeed

SEQ_STATE_WORDS = 8      # int32 words of a sequence's record (lib_sampling.cu has the same layout)
SEQ_POS, SEQ_GENERATED, SEQ_LAST_TOKEN, SEQ_FLAGS, SEQ_KEY, SEQ_COUNTER = 0, 1, 2, 3, 4, 6
SEQ_FLAG_FINISHED = 1
from .pool import CacheFull, FreeList


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


@dataclass
class KVGroup:
    need: CacheNeed
    units: list[int]
    pool: FreeList
    k: torch.Tensor            # [len(units), n_pages, kv_heads, PAGE, head_dim]
    v: torch.Tensor
    pages: dict[int, list[int]] = field(default_factory=dict)   # slot -> page id per page index (-1: given back)

    def unit_storage(self, unit: int):
        i = self.units.index(unit)
        return self.k[i], self.v[i]

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, pages_for(new_len) - len(self.pages[slot]))

    def grow(self, slot: int, new_len: int) -> None:
        lst = self.pages[slot]
        while len(lst) < pages_for(new_len):
            lst.append(self.pool.alloc())

    def release_unseen(self, slot: int, length: int) -> None:
        """Give back the pages no query at a position >= length can see (the need's kind says which)."""
        first_seen = self.need.first_needed(length)
        if first_seen <= 0:
            return
        lst = self.pages[slot]
        for i, pg in enumerate(lst):
            if pg >= 0 and (i + 1) * PAGE - 1 < first_seen:
                self.pool.free(pg)
                lst[i] = -1

    def release_all(self, slot: int) -> None:
        for pg in self.pages.pop(slot):
            if pg >= 0:
                self.pool.free(pg)


class SequenceCache:
    """Slots, page groups and fixed-size state for one model on one device."""

    def __init__(self, cache_needs: dict[int, CacheNeed | None], state_needs: dict[int, StateNeed | None],
                 n_slots: int, n_pages: int, dtype: torch.dtype, device):
        if n_slots < 1 or n_pages < 1:
            raise ValueError("the cache needs at least one slot and one page")
        self.n_slots, self.n_pages, self.dtype, self.device = n_slots, n_pages, dtype, device
        self.slots = FreeList(n_slots, "cache slot")
        self.length = [0] * n_slots
        by_need: dict[CacheNeed, list[int]] = {}
        for unit, need in cache_needs.items():
            if need is not None:
                by_need.setdefault(need, []).append(unit)
        self.groups: list[KVGroup] = []
        self.group_of_unit: dict[int, int] = {}
        for need, units in by_need.items():
            # one page more than the pool hands out: padded rows of a replayed decode step write there
            shape = (len(units), n_pages + 1, need.kv_heads, PAGE, need.head_dim)
            g = KVGroup(need, units, FreeList(n_pages, f"cache page ({need.kind})"),
                        torch.empty(shape, dtype=dtype, device=device), torch.empty(shape, dtype=dtype, device=device))
            for u in units:
                self.group_of_unit[u] = len(self.groups)
            self.groups.append(g)
        # the fixed-size record of every sequence, on the device: tokens held, tokens generated, last token,
        # flags, sampling key (2 words), draw counter (2 words). The sampler's kernel reads key and counter
        # from it and advances it; `length` above and the generation loop's bookkeeping are its host mirror.
        # One spare row serves the padding rows of replayed decode steps.
        self.seq_state = torch.zeros((n_slots + 1, SEQ_STATE_WORDS), dtype=torch.int32, device=device)
        self.state: dict[int, torch.Tensor] = {
            unit: torch.zeros((n_slots + 1, *need.shape), dtype=need.dtype, device=device)   # last: spare, for padding
            for unit, need in state_needs.items() if need is not None}

    # ------------------------------------------------------------------ slots
    def open(self) -> int:
        slot = self.slots.alloc()
        self.length[slot] = 0
        for g in self.groups:
            g.pages[slot] = []
        for st in self.state.values():
            st[slot].zero_()
        self.seq_state[slot].zero_()
        return slot

    def seed(self, slots: list[int], seeds: list[int]) -> None:
        """Start the sampling streams of freshly opened sequences: key = the sequence's 64-bit seed,
        draw counter 0 (one small copy for the batch)."""
        rec = np.zeros((len(slots), SEQ_STATE_WORDS), dtype=np.int64)
        for i, sd in enumerate(seeds):
            rec[i, SEQ_KEY], rec[i, SEQ_KEY + 1] = sd & 0xFFFFFFFF, (sd >> 32) & 0xFFFFFFFF
        rec = torch.from_numpy(rec.astype(np.uint32).view(np.int32))
        self.seq_state.index_copy_(0, torch.as_tensor(slots, dtype=torch.long, device=self.device), rec.to(self.device))

    def close(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise ValueError(f"cache slot {slot} is not held; it cannot be closed")
        for g in self.groups:
            g.release_all(slot)
        self.slots.free(slot)
        self.length[slot] = 0

    # ------------------------------------------------------------------ growth
    def reserve(self, growth: list[tuple[int, int]]) -> None:
        """Pages for `n_new` more tokens of each (slot, n_new); either all are had or CacheFull is
        raised and nothing has changed."""
        for g in self.groups:
            want = sum(g.pages_needed(slot, self.length[slot] + n) for slot, n in growth)
            if want > g.pool.n_free:
                raise CacheFull(f"the step needs {want} more cache pages of {PAGE} tokens in the {g.need.kind} group; "
                                f"{g.pool.n_free} of {g.pool.n} are free")
        for g in self.groups:
            for slot, n in growth:
                g.grow(slot, self.length[slot] + n)

    def advance(self, growth: list[tuple[int, int]]) -> None:
        for slot, n in growth:
            self.length[slot] += n
            for g in self.groups:
                g.release_unseen(slot, self.length[slot])

    # ------------------------------------------------------------------ views for a step
    def block_table(self, group: int, slots: list[int], width: int | None = None) -> np.ndarray:
        g = self.groups[group]
        w = max(1, max(len(g.pages[s]) for s in slots)) if width is None else width
        bt = np.full((len(slots), w), -1, dtype=np.int32)
        for i, s in enumerate(slots):
            lst = g.pages[s]
            bt[i, :len(lst)] = lst
        return bt

    def tokens_capacity(self) -> int:
        return self.n_pages * PAGE
