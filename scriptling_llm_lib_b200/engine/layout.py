"""A model as data: its layers, the order they run in, and what surrounds them.

The reference runs blocks 0..L-1 once each over one cache per block (model_f32.go:371-373). Here
the order is a list of schedule entries; an entry names the layer to run and the cache unit it
uses, so a layer can appear twice (with a unit for each appearance) or read the unit that another
entry wrote (`writes_cache=False`).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import PartSpec
from ..parts.block import LayerSpec


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int
    cache_unit: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelLayout:
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec                 # resolved through the EMBEDDINGS registry
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec                # NORMS; adds the last pending addend and norms the wanted rows
    head: PartSpec                      # HEADS
    stop_ids: tuple[int, ...] = ()
    ignorable_tensors: tuple[str, ...] = field(default=())   # may be in the file without being used

    def check(self) -> None:
        written: set[int] = set()
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}; the model has {len(self.layers)}")
            if e.writes_cache:
                if e.cache_unit in written:
                    raise ValueError(f"cache unit {e.cache_unit} is written by two schedule entries")
                written.add(e.cache_unit)
            elif e.cache_unit not in written:
                raise ValueError(f"schedule entry reads cache unit {e.cache_unit} before any entry has written it")


def sequential_schedule(n_layers: int) -> tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(i, i, True) for i in range(n_layers))
