"""How a layer's parts are arranged around the residual stream.

"pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)) (model_f32.go:382-500). The residual
stream is float32; a block hands its last sublayer's output on as a pending `delta`, which the next
norm adds while it reads the row, so no separate pass over the stream is needed.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer as data: which parts, with which parameters, in which arrangement."""
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    arrangement: str = "pre_norm"


class PreNormBlock:
    def __init__(self, spec: LayerSpec):
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, residual, delta, ctx, unit, writes):
        """residual float32 [T, hidden] (updated in place), delta: pending addend or None.
        Returns the new pending addend."""
        n = self.mixer_norm.forward(residual, delta, ctx)
        a = self.mixer.forward(n, ctx, unit, writes)
        n2 = self.feed_forward_norm.forward(residual, a, ctx)
        return self.feed_forward.forward(n2, ctx)


ARRANGEMENTS.register("pre_norm", PreNormBlock)


def build_block(spec: LayerSpec):
    return ARRANGEMENTS.build(PartSpec(spec.arrangement), spec=spec)
