"""Token embedding and output head.

x[i, :] = E[id_i, :], no scaling (model_f32.go:363-369); logits = n W^T with W the embedding when
the head is tied (model_f32.go:147-162, :519-524). The reference skips ids outside the table and
leaves stale data in the row; here such an id is an error before anything runs. Both are parts
like the others, named in a layout by kind ("token_embedding", "linear_head"): a model that scales
its embedding or caps its logits registers parts of its own.
"""
from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import EMBEDDINGS, HEADS, Embedding, Head, PartSpec
from .linear import Linear


class TokenEmbedding(Embedding):
    def __init__(self, vocab: int, width: int, name: str):
        self.vocab, self.width, self.name = vocab, width, name
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.width))]

    def elements_read_per_step(self) -> int:
        return 0                                    # a step reads one row per token, not the table

    def bind(self, tensors, dtype, device):
        self.table = tensors[self.name]

    def forward(self, ids, ctx):
        out = torch.empty((ids.shape[0], self.width), dtype=torch.float32, device=ids.device)
        if self.table.dtype == ctx.dtype:
            ctx.kernels.embed_rows(ids, self.table, out, ctx.err_flag)
        else:
            ctx.kernels_f32.embed_rows(ids, self.table, out, ctx.err_flag)
        return out


class OutputHead(Head):
    """Logits in float32 for the rows it is given. `tied`: the matrix is another part's tensor (the
    embedding's), named by `weight_name`, and is not asked of the weight file a second time."""

    def __init__(self, vocab: int, width: int, weight_name: str, tied: bool = False):
        self.vocab, self.width, self.tied = vocab, width, tied
        self.linear = Linear([weight_name], [vocab], width)

    def tensor_specs(self):
        return [] if self.tied else self.linear.tensor_specs()

    def elements_read_per_step(self) -> int:
        return self.vocab * self.width

    def bind(self, tensors, dtype, device):
        self.linear.bind(tensors, dtype, device)

    def forward(self, normed, ctx):
        return self.linear.forward(normed, ctx, out_dtype=torch.float32)


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("linear_head", OutputHead)


def token_embedding(vocab: int, width: int, name: str) -> PartSpec:
    return PartSpec("token_embedding", dict(vocab=vocab, width=width, name=name))


def linear_head(vocab: int, width: int, weight_name: str, tied: bool = False) -> PartSpec:
    return PartSpec("linear_head", dict(vocab=vocab, width=width, weight_name=weight_name, tied=tied))
