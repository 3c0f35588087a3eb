"""Token embedding and output head.

x[i, :] = E[id_i, :], no scaling (model_f32.go:363-369); logits = n W^T with W the embedding when
the head is tied (model_f32.go:147-162, :519-524). The reference skips ids outside the table and
leaves stale data in the row; here such an id is an error before anything runs.
"""
from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .linear import Linear


class TokenEmbedding:
    def __init__(self, vocab: int, width: int, name: str):
        self.vocab, self.width, self.name = vocab, width, name
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.width))]

    def bind(self, tensors, dtype, device):
        self.table = tensors[self.name]

    def forward(self, ids, ctx):
        out = torch.empty((ids.shape[0], self.width), dtype=torch.float32, device=ids.device)
        if self.table.dtype == ctx.dtype:
            ctx.kernels.embed_rows(ids, self.table, out, ctx.err_flag)
        else:
            ctx.kernels_f32.embed_rows(ids, self.table, out, ctx.err_flag)
        return out


class OutputHead:
    """Logits in float32 for the rows it is given."""

    def __init__(self, vocab: int, width: int, name: str | None, tied_to: TokenEmbedding | None):
        self.vocab, self.width, self.tied_to = vocab, width, tied_to
        self.linear = Linear([name if name else tied_to.name], [vocab], width)

    def tensor_specs(self):
        return [] if self.tied_to is not None else self.linear.tensor_specs()

    def bind(self, tensors, dtype, device):
        if self.tied_to is not None:
            self.linear.weight = self.tied_to.table
        else:
            self.linear.bind(tensors, dtype, device)

    def forward(self, normed, ctx):
        return self.linear.forward(normed, ctx, out_dtype=torch.float32)
