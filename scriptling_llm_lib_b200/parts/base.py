"""The parts a model is put together from, and the registries that name them.

A layer is an arrangement (a block) of named parts: norms, a mixer, a feed-forward, or whatever
the arrangement asks for. Around the layers stand an embedding, a final norm and an output head,
parts like the others. Each part takes its sizes and constants as parameters, publishes the
tensors it wants (`tensor_specs`), takes them (`bind`) and runs on the rows it is given
(`forward`). No part knows which model it is in: tensor names, widths, eps, theta and head counts
all arrive through the constructor. A model's layout names a part by its registered kind, layer
by layer, so different layers can have different mixers and feed-forwards.

Interfaces (duck-typed; the base classes document them):

  Embedding.forward(ids, ctx) -> x            the float32 residual stream [T, hidden] of the step's tokens
  Head.forward(normed, ctx) -> logits         float32 [n, vocab] for the rows it is given
  Block.forward(residual, delta, ctx, unit, writes) -> delta
                                              an arrangement: runs its parts on the stream; also parts(),
                                              graph_safe(), cache_need(), state_need() (see block.py)

  Mixer.cache_need() -> CacheNeed | None      keys/values the layer keeps per position
  Mixer.state_need() -> StateNeed | None      per-sequence state of fixed size
  Mixer.forward(x, ctx, unit, writes) -> y    x, y: [T, hidden] in the engine's dtype; `unit` is the
                                              cache unit to read, `writes` whether to append to it.
                                              y may also be float32 [P, T, hidden]: partial sums
                                              that add up to the output (the next norm adds them)
  FeedForward.forward(x, ctx) -> y            the same two forms of y
  Norm.forward(residual, delta, ctx, rows=None) -> normed
                                              residual float32 [T, hidden], updated in place by
                                              += delta when rows is None; rows picks rows to norm;
                                              delta: None or either form of y
  PositionEncoding.prepare(max_positions, device); .rotation() or .transform(...)   see below

A norm between two products can be folded into them (optional, and only where all three agree): a
row's 1/rms is one number, so (v / rms * w) W^T = (1 / rms) * ((v * w) W^T). A norm that can be
folded says so with `fold_terms()`; a mixer or feed-forward whose last product can take the first
half (add its result to the residual stream, write v * w, leave the sums of v^2) accepts
`forward(..., fold=FoldRequest)` and says when with `can_fold(ctx, rows)`; one whose first product
can take the second half (scale its output rows) accepts a `Folded` as its input and says when with
`takes_folded(ctx, rows)`. A block asks all three before it requests anything; parts that say
nothing are never handed either.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..cache.needs import CacheNeed, StateNeed
from ..weights.spec import TensorSpec


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name with its parameters: pure data, part of a model's layout."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)


class Part:
    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def elements_read_per_step(self) -> int:
        """Weight elements a decode step has to read for this part whatever the batch (a roofline's
        numerator): by default every tensor it owns, once."""
        n = 0
        for s in self.tensor_specs():
            k = 1
            for d in s.shape:
                k *= d
            n += k
        return n

    def bind(self, tensors: dict, dtype, device) -> None:
        """Take this part's tensors (by the names it published) for an engine of `dtype`."""

    def prepare(self, max_positions: int, device) -> None:
        """Build host-made tables once the engine knows its longest sequence."""


@dataclass
class FoldRequest:
    """Asks a part's last product to finish the sublayer itself: add the result to `residual`
    (float32 [T, width], in place) and prepare the input of the product behind the norm with
    this `weight` (float32 [width]) and `eps`."""
    residual: Any
    weight: Any
    eps: float


@dataclass
class Folded:
    """The input of the product behind a folded norm: x = (residual * norm weight) in the engine's
    dtype [T, width], not yet divided by the rows' rms; sumsq float32 [P, T] partial sums of
    residual^2 over the width. The product multiplies its output rows by rsqrt(sum / width + eps)."""
    x: Any
    sumsq: Any
    width: int
    eps: float


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def forward(self, x, ctx, unit: int, writes: bool):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class Norm(Part):
    def forward(self, residual, delta, ctx, rows=None):
        raise NotImplementedError

    def fold_terms(self):
        """(weight float32 [width], eps) if this norm is y = v / sqrt(mean(v^2) + eps) * weight and may be
        folded into the products around it; None otherwise."""
        return None


class PositionEncoding(Part):
    """How a mixer's queries and keys learn their positions. A mixer without one (None in its
    parameters) uses queries and keys as projected. An encoding is one of two kinds:

      rotation() -> (table, rotary_width, interleaved)
          a rotation of pairs by an angle per position and pair: table float32
          [positions, rotary_width / 2, 2] of (cos, sin). The mixer's kernels do the rotating, fused
          into the products and the decode attention where the widths allow.
      transform(qkv, ctx, n_heads, n_kv_heads, head_dim) -> None
          anything else: rewrite the query heads (columns [0, n_heads * head_dim)) and the key heads
          (the next n_kv_heads * head_dim columns) of the step's rows in place, using ctx.tok_pos.
          `rotation()` then returns None.

    Neither writes the cache: storing keys and values is the mixer's own step."""

    def rotation(self):
        return None

    def transform(self, qkv, ctx, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ids, ctx):
        raise NotImplementedError


class Head(Part):
    def forward(self, normed, ctx):
        raise NotImplementedError


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, type] = {}

    def register(self, kind: str, cls: type, replace: bool = False) -> type:
        if kind in self._items and not replace:
            raise ValueError(f"{self.what} {kind!r} is already registered")
        self._items[kind] = cls
        return cls

    def build(self, part: PartSpec, **extra):
        try:
            cls = self._items[part.kind]
        except KeyError:
            raise ValueError(f"unknown {self.what} {part.kind!r}; registered: {', '.join(sorted(self._items))}") from None
        return cls(**part.params, **extra)

    def kinds(self) -> list[str]:
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
ARRANGEMENTS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
