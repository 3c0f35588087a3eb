"""Dense SiLU-gated feed-forward: y = (silu(x Wg^T) * (x Wu^T)) Wd^T, no biases
(model_f32.go:476-493). Gate and up rows are stacked so one product serves both."""
from __future__ import annotations

import torch

from .base import FEED_FORWARDS, FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
    def __init__(self, hidden: int, intermediate: int, gate_name: str, up_name: str, down_name: str):
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_up = Linear([gate_name, up_name], [intermediate, intermediate], hidden)
        self.down = Linear([down_name], [hidden], intermediate)

    def tensor_specs(self):
        return self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, tensors, dtype, device):
        self.gate_up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)

    def forward(self, x, ctx):
        gu = self.gate_up.forward(x, ctx)
        h = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        ctx.kernels.swiglu(gu, h)
        return self.down.forward(h, ctx)


FEED_FORWARDS.register("swiglu", SwiGLU)
