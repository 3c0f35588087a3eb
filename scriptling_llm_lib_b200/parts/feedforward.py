"""Dense SiLU-gated feed-forward: y = (silu(x Wg^T) * (x Wu^T)) Wd^T, no biases
(model_f32.go:476-493). Gate and up rows are stacked so one product serves both; when the
intermediate width is a multiple of 8 the stacked rows are kept in tiles of 16 (8 gate rows, the 8
matching up rows), so that one tensor-core tile holds both halves of a pair and the gate can be
applied before anything is written."""
from __future__ import annotations

import torch

from .base import FEED_FORWARDS, FeedForward, Folded
from .linear import Linear


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, gate_name: str, up_name: str, down_name: str):
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_up = Linear([gate_name, up_name], [intermediate, intermediate], hidden)
        self.down = Linear([down_name], [hidden], intermediate)

    def tensor_specs(self):
        return self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, tensors, dtype, device):
        self.gate_up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)
        F = self.intermediate
        self.tiled = F % 8 == 0
        if self.tiled:
            w = self.gate_up.weight
            self.gate_up.weight = w.view(2, F // 8, 8, self.hidden).permute(1, 0, 2, 3).reshape(2 * F, self.hidden).contiguous()

    def takes_folded(self, ctx, rows: int) -> bool:
        return self.tiled and self.gate_up.fold_path(ctx, rows, ctx.dtype) is not None

    def can_fold(self, ctx, rows: int) -> bool:
        return self.down.fold_path(ctx, rows, ctx.dtype, finishing=True) is not None

    def forward(self, x, ctx, fold=None):
        if isinstance(x, Folded) or fold is not None:
            plain = x.x if isinstance(x, Folded) else x
            rows = plain.shape[0]
            h = torch.empty((rows, self.intermediate), dtype=torch.bfloat16, device=plain.device)
            if isinstance(x, Folded) or (self.tiled and self.gate_up.fold_path(ctx, rows, ctx.dtype) is not None):
                self.gate_up.forward_folded(x, ctx, swiglu_out=h)
            else:
                h = self._hidden(x, ctx)
            return self.down.forward_folded(h, ctx, fold=fold) if fold is not None else self.down.forward(h, ctx, partials_ok=True)
        return self.down.forward(self._hidden(x, ctx), ctx, partials_ok=True)

    def _hidden(self, x, ctx):
        h = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        w = self.gate_up.weight
        fast = self.tiled and x.dtype == torch.bfloat16 and w.dtype == x.dtype
        if fast and ctx.kernels.tensor_core.prefers_skinny(x, w, "swiglu", ctx.engine.sm_count):
            ctx.kernels.tensor_core.gemm_skinny(x, w, h, ctx.err_flag, swiglu=True)
        elif fast and ctx.kernels.decode.prefers(x, w, ctx.engine.sm_count):
            ctx.kernels.decode.gemm_small_m(x, w, h, swiglu=True)
        elif fast and ctx.kernels.tensor_core.takes(x, w):
            ctx.kernels.tensor_core.gemm(x, w, h, ctx.err_flag, swiglu=True)
        else:
            gu = self.gate_up.forward(x, ctx)
            ctx.kernels.swiglu(gu, h, tiled=self.tiled)
        return h


FEED_FORWARDS.register("swiglu", SwiGLU)
