"""The decoder as built parts: embedding, blocks, final norm, output head.

Everything here is driven by a ModelLayout; no size or name is written down in this file."""
from __future__ import annotations

from ..cache.needs import CacheNeed, StateNeed
from ..parts.base import NORMS
from ..parts.block import build_block
from ..parts.embedding import OutputHead, TokenEmbedding
from ..weights.spec import TensorSpec
from .layout import ModelLayout


class DecoderModel:
    def __init__(self, layout: ModelLayout):
        layout.check()
        self.layout = layout
        self.embedding = TokenEmbedding(layout.vocab_size, layout.hidden_size, layout.embedding_name)
        self.blocks = [build_block(spec) for spec in layout.layers]
        self.final_norm = NORMS.build(layout.final_norm)
        self.head = OutputHead(layout.vocab_size, layout.hidden_size, layout.head_name,
                               self.embedding if layout.head_name is None else None)

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
        for b in self.blocks:
            for p in b.parts():
                p.prepare(max_positions, device)

    def graph_safe(self) -> bool:
        """True when every part says its decode step launches the same work whatever the values
        (no host reads, no shapes that depend on data), so the step can be captured and replayed."""
        return all(getattr(p, "graph_safe", False) for b in self.blocks for p in (b.mixer, b.feed_forward))

    def cache_needs(self) -> dict[int, CacheNeed | None]:
        """Need of every cache unit, taken from the mixer of the entry that writes it."""
        return {e.cache_unit: self.blocks[e.layer].mixer.cache_need() for e in self.layout.schedule if e.writes_cache}

    def state_needs(self) -> dict[int, StateNeed | None]:
        return {e.cache_unit: self.blocks[e.layer].mixer.state_need() for e in self.layout.schedule if e.writes_cache}
