"""The decoder as built parts: embedding, blocks, final norm, output head.

Everything here is driven by a ModelLayout; no size, name or role is written down in this file:
the embedding, the final norm and the head come from their registries like the layers' parts, and
what a layer needs of the cache or whether its decode step can be captured is asked of its block."""
from __future__ import annotations

from ..cache.needs import CacheNeed, StateNeed
from ..parts.base import EMBEDDINGS, HEADS, NORMS
from ..parts.block import build_block
from ..weights.spec import TensorSpec
from .layout import ModelLayout


class DecoderModel:
    def __init__(self, layout: ModelLayout):
        layout.check()
        self.layout = layout
        self.embedding = EMBEDDINGS.build(layout.embedding)
        self.blocks = [build_block(spec) for spec in layout.layers]
        self.final_norm = NORMS.build(layout.final_norm)
        self.head = HEADS.build(layout.head)

    def parts(self):
        out = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        out.extend([self.final_norm, self.head])
        return out

    def tensor_specs(self) -> list[TensorSpec]:
        specs, seen = [], set()
        for p in self.parts():
            for s in p.tensor_specs():
                if s.name in seen:
                    raise ValueError(f"two parts ask for the tensor {s.name!r}")
                seen.add(s.name)
                specs.append(s)
        return specs

    def bind(self, tensors: dict, dtype, device) -> None:
        for p in self.parts():
            p.bind(tensors, dtype, device)

    def prepare(self, max_positions: int, device) -> None:
        for p in self.parts():
            p.prepare(max_positions, device)

    def graph_safe(self) -> bool:
        """True when every block says its decode step launches the same work whatever the values
        (no host reads, no shapes that depend on data), so the step can be captured and replayed."""
        return all(b.graph_safe() for b in self.blocks)

    def cache_needs(self) -> dict[int, CacheNeed | None]:
        """Need of every cache unit, asked of the block of the entry that writes it."""
        return {e.cache_unit: self.blocks[e.layer].cache_need() for e in self.layout.schedule if e.writes_cache}

    def state_needs(self) -> dict[int, StateNeed | None]:
        return {e.cache_unit: self.blocks[e.layer].state_need() for e in self.layout.schedule if e.writes_cache}

    def elements_read_per_step(self) -> int:
        """Weight elements one decode step reads whatever the batch: every scheduled layer's parts
        (a layer that runs twice is read twice), the final norm and the head."""
        n = sum(p.elements_read_per_step() for e in self.layout.schedule for p in self.blocks[e.layer].parts())
        return n + self.embedding.elements_read_per_step() + self.final_norm.elements_read_per_step() + \
            self.head.elements_read_per_step()
