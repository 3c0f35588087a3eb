"""RMSNorm fused with the residual sum that precedes it.

y = (v / sqrt(mean(v^2) + eps)) * w with v = residual + delta; weight used as is, no bias, no mean
subtraction (float32_ops.go:159-172). The sum of squares, the division and the residual sum are
float32 whatever the engine's dtype.
"""
from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import NORMS, Folded, Norm


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_name: str):
        self.width, self.eps, self.weight_name = width, float(eps), weight_name
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.width,), init="norm_weight")]

    def bind(self, tensors, dtype, device):
        self.weight = tensors[self.weight_name]
        self.weight_f32 = self.weight if self.weight.dtype == torch.float32 else self.weight.float()
        self._fold_memo = {}

    def fold_terms(self):
        return self.weight_f32, self.eps

    def forward(self, residual, delta, ctx, rows=None):
        if isinstance(delta, Folded):          # the product before this norm has done its work already
            return delta
        n = residual.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, self.width), dtype=ctx.dtype, device=residual.device)
        ctx.kernels.add_rmsnorm(residual, delta, rows, self.weight, y, self.eps)
        return y


NORMS.register("rmsnorm", RMSNorm)
