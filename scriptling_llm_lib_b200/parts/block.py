"""How a layer's parts are arranged around the residual stream.

A layer is data: the name of an arrangement and the parts it is made of, by role. An arrangement
(a block class) builds its parts from their registries, runs them in its order, and answers for
the layer: which parts it has, whether its decode step can be captured, what it needs of the cache.
The engine asks the block, never a part by name, so an arrangement with other roles (no
feed-forward, two mixers, four norms) is a class of its own and nothing else changes.

"pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)) (model_f32.go:382-500), roles
`mixer_norm`, `mixer`, `feed_forward_norm`, `feed_forward`. The residual stream is float32; a block
hands its last sublayer's output on as a pending `delta`, which the next norm adds while it reads
the row, so no separate pass over the stream is needed.

Where the norm between two sublayers and the products on either side of it all agree (see base.py:
FoldRequest, Folded), the norm needs no kernel: the block asks the sublayer before it to finish the
residual sum and prepare the norm's output, and hands the result through the norm to the sublayer
behind it. Across layers the same holds for a layer's first norm: a block that sets `folds_entry`
tells through `entry_fold(ctx, rows, residual)` what the layer before it may prepare, and accepts
that layer's request as `forward(..., next_fold=...)`.

A block's interface:
  parts() -> list of its parts                  for tensor specs, bind, prepare
  forward(residual, delta, ctx, unit, writes) -> delta
  graph_safe() -> bool                          its decode step launches the same work whatever the values
  cache_need() -> CacheNeed | None              what the cache unit it writes must hold
  state_need() -> StateNeed | None              per-sequence state of fixed size
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping

from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, FoldRequest, PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer as data: the arrangement and its parts by role."""
    arrangement: str
    parts: Mapping[str, PartSpec] = field(default_factory=dict)


def pre_norm_layer(mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec) -> LayerSpec:
    return LayerSpec("pre_norm", dict(mixer=mixer, feed_forward=feed_forward, mixer_norm=mixer_norm,
                                      feed_forward_norm=feed_forward_norm))


import os
_NO_FOLD = bool(os.environ.get("SLLM_NO_FOLD"))


def fold_request(norm, before, behind, ctx, rows: int, residual):
    """A FoldRequest for `norm` if it, the part `before` it and the part `behind` it all can; else None.
    What the three answer depends on a step only through its kind (how many rows, decode or not), so
    the answer is kept per kind, with the norm (which lives and dies with its neighbours)."""
    if _NO_FOLD:
        return None
    memo = norm.__dict__.setdefault("_fold_memo", {})
    key = (id(before), id(behind), min(rows, 256), bool(ctx.is_decode), ctx.dtype)
    try:
        terms = memo[key]
    except KeyError:
        terms = norm.fold_terms() if hasattr(norm, "fold_terms") else None
        can = getattr(before, "can_fold", None)
        takes = getattr(behind, "takes_folded", None)
        if terms is None or can is None or takes is None or not can(ctx, rows) or not takes(ctx, rows):
            terms = None
        memo[key] = terms
    return None if terms is None else FoldRequest(residual, terms[0], terms[1])


class Block:
    """Base of the arrangements: answers for the layer out of `parts()`; an arrangement with one
    mixer need only name it `self.mixer`."""
    mixer = None
    folds_entry = False          # True: forward takes next_fold=..., and entry_fold says what may be prepared for it

    def parts(self) -> list:
        raise NotImplementedError

    def forward(self, residual, delta, ctx, unit, writes):
        raise NotImplementedError

    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def cache_need(self):
        return self.mixer.cache_need() if self.mixer is not None else None

    def state_need(self):
        return self.mixer.state_need() if self.mixer is not None else None


def _role(spec: LayerSpec, role: str) -> PartSpec:
    try:
        return spec.parts[role]
    except KeyError:
        raise ValueError(f"the {spec.arrangement!r} arrangement needs a part in the role {role!r}; "
                         f"the layer has {', '.join(sorted(spec.parts)) or 'none'}") from None


class PreNormBlock(Block):
    def __init__(self, spec: LayerSpec):
        self.mixer_norm = NORMS.build(_role(spec, "mixer_norm"))
        self.mixer = MIXERS.build(_role(spec, "mixer"))
        self.feed_forward_norm = NORMS.build(_role(spec, "feed_forward_norm"))
        self.feed_forward = FEED_FORWARDS.build(_role(spec, "feed_forward"))

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    folds_entry = True

    def entry_fold(self, ctx, rows: int, residual, before):
        """What the sublayer `before` this layer may prepare of this layer's first norm (or None)."""
        return fold_request(self.mixer_norm, before, self.mixer, ctx, rows, residual)

    def last_part(self):
        return self.feed_forward

    def forward(self, residual, delta, ctx, unit, writes, next_fold=None):
        """residual float32 [T, hidden] (updated in place), delta: pending addend or None (or the
        prepared output of this layer's first norm). Returns the new pending addend; `next_fold`
        (a function of the part that would do it) asks the last sublayer to prepare the next
        layer's first norm instead."""
        rows = residual.shape[0]
        n = self.mixer_norm.forward(residual, delta, ctx)
        fold = fold_request(self.feed_forward_norm, self.mixer, self.feed_forward, ctx, rows, residual)
        a = self.mixer.forward(n, ctx, unit, writes, fold=fold) if fold is not None else self.mixer.forward(n, ctx, unit, writes)
        n2 = self.feed_forward_norm.forward(residual, a, ctx)
        fold = next_fold(self.feed_forward) if next_fold is not None else None
        return self.feed_forward.forward(n2, ctx, fold=fold) if fold is not None else self.feed_forward.forward(n2, ctx)


ARRANGEMENTS.register("pre_norm", PreNormBlock)


def build_block(spec: LayerSpec):
    return ARRANGEMENTS.build(PartSpec(spec.arrangement), spec=spec)
