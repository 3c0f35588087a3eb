"""Grouped-query causal attention over the paged cache.

q = x Wq^T, k = x Wk^T, v = x Wv^T; Q and K rotated by the position encoding; K, V appended to
the cache; query head h reads key/value head h // (H/G); score = (q.k) / sqrt(head_dim); keys
after the query are masked; max-subtracted softmax; out = sum p v; y = out Wo^T
(model_f32.go:391-470, float32_ops.go:190-235, :252-260). A `window` (absent in the reference)
also masks keys `window` or more positions behind the query and lets the cache give old pages
back. With `writes=False` the layer projects queries only and reads the unit another layer wrote.

The position encoding is optional (`position=None`: queries and keys as projected). Storing keys
and values in the cache is this mixer's own step, whatever the encoding: for an encoding that is a
rotation by a table the store and the rotation are one kernel (or part of the q|k|v product's
epilogue, or of the decode attention kernel, where the widths allow); any other encoding rewrites
the step's query and key rows in place first (`transform`) and the store copies.
"""
from __future__ import annotations

import math

import torch

from ..cache.needs import CacheNeed
from ..csrc.bindings import DecodeKernels, PrefillAttentionTC
from .base import MIXERS, POSITION_ENCODINGS, Folded, Mixer, PartSpec
from .linear import Linear


class Attention(Mixer):
    @property
    def graph_safe(self) -> bool:
        """The decode step launches the same work whatever the values; an encoding that rewrites rows
        itself (`transform`) has to say the same of its own work."""
        return self.position is None or self.position.rotation() is not None or bool(getattr(self.position, "graph_safe", False))

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, position: PartSpec | None,
                 q_name: str, k_name: str, v_name: str, o_name: str, window: int | None = None,
                 scale: float | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} key/value heads")
        if head_dim % 16:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take head widths in steps of 16")
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim, self.window = hidden, n_heads, n_kv_heads, head_dim, window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = POSITION_ENCODINGS.build(position) if position is not None else None
        qw, kw = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv = Linear([q_name, k_name, v_name], [qw, kw, kw], hidden)
        self.out = Linear([o_name], [hidden], qw)
        self.q_only: Linear | None = None

    def tensor_specs(self):
        return self.qkv.tensor_specs() + self.out.tensor_specs()

    def bind(self, tensors, dtype, device):
        self.qkv.bind(tensors, dtype, device)
        self.out.bind(tensors, dtype, device)
        self.q_only = self.qkv.rows(0, self.n_heads * self.head_dim)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def _store(self, qkv, ctx, rotation, n_kv, kpages, vpages, block_table) -> None:
        """Give the step's queries and keys their positions and append keys and values to the cache
        (n_kv == 0: queries only). `rotation`: the encoding's table, or None."""
        if self.position is not None and rotation is None:
            self.position.transform(qkv, ctx, self.n_heads, n_kv, self.head_dim)
        if rotation is None and n_kv == 0:
            return
        table, rot, interleaved = rotation if rotation is not None else (None, 0, False)
        ctx.kernels.rope_kv_write(qkv, ctx.tok_pos, ctx.tok_seq, block_table, table, kpages, vpages, self.n_heads, n_kv,
                                  self.head_dim, rot, interleaved)

    def cache_need(self):
        return CacheNeed("window" if self.window else "full", self.n_kv_heads, self.head_dim, self.window)

    def takes_folded(self, ctx, rows: int) -> bool:
        """The q|k|v product can scale its own output rows: in a decode step of few rows, and in a long
        prompt step (the tensor-core product, with or without the rotation in its epilogue)."""
        path = self.qkv.fold_path(ctx, rows, ctx.dtype)
        return path is not None and self.q_only.fold_path(ctx, rows, ctx.dtype) == path and (ctx.is_decode or path == "tiles")

    def can_fold(self, ctx, rows: int) -> bool:
        """The output product can finish the sublayer: add to the residual stream and prepare the next norm."""
        path = self.out.fold_path(ctx, rows, ctx.dtype, finishing=True)
        return path is not None and (ctx.is_decode or path == "tiles")

    def forward(self, x, ctx, unit, writes, fold=None):
        if isinstance(x, Folded):
            folded, x = x, x.x
        else:
            folded = None
        kpages, vpages, block_table = ctx.unit_kv(unit)
        fast_decode = ctx.is_decode and x.dtype == torch.bfloat16 and self.head_dim in DecodeKernels.HEAD_DIMS
        rotation = self.position.rotation() if self.position is not None else None
        tc = ctx.kernels.tensor_core if x.dtype == torch.bfloat16 else None
        # a rotation can ride in the decode attention kernel, or in the q|k|v product of a long prompt step
        fusion = rotation if (fast_decode and rotation is not None and DecodeKernels.rotation_fusable(*rotation[1:])) else None
        fused_product = None
        if (tc is not None and writes and not fast_decode and rotation is not None and x.shape[0] > tc.SKINNY_MAX_M
                and tc.rotation_fusable(self.head_dim, *rotation[1:]) and self.qkv.weight.dtype == torch.bfloat16
                and tc.takes(x, self.qkv.weight)):
            fused_product = rotation
        if fused_product is not None:
            # a long prompt step: the q|k|v product rotates and fills the cache in its own epilogue
            qkv = torch.empty((x.shape[0], self.n_heads * self.head_dim), dtype=x.dtype, device=x.device)
            tc.gemm_qkv_rope(x, self.qkv.weight, qkv, ctx.err_flag, ctx.tok_pos, ctx.tok_seq, block_table, fused_product[0],
                             kpages, vpages, self.n_heads, self.n_kv_heads, self.head_dim, fused_product[1], fused_product[2],
                             owed=(folded.sumsq, folded.width, folded.eps) if folded is not None else None)
        else:
            proj = self.qkv if writes else self.q_only
            qkv = proj.forward_folded(folded, ctx) if folded is not None else proj.forward(x, ctx)
            if fusion is None:
                self._store(qkv, ctx, rotation, self.n_kv_heads if writes else 0, kpages if writes else None,
                            vpages if writes else None, block_table)
        attn = torch.empty((x.shape[0], self.n_heads * self.head_dim), dtype=x.dtype, device=x.device)
        if fast_decode:
            n_split = ctx.decode_splits(self.n_heads, self.n_kv_heads, self.head_dim)
            scratch = torch.empty((ctx.n_seqs * self.n_heads * n_split * (self.head_dim + 2),), dtype=torch.float32,
                                  device=x.device)
            tickets = ctx.engine.tickets(ctx.n_seqs * self.n_kv_heads)
            if fusion is not None:      # rotation and cache write happen inside the attention kernel
                ctx.kernels.decode.attn_decode_rope(qkv, attn, ctx.seq_pos0, block_table, kpages, vpages, scratch, tickets,
                                                    fusion[0], fusion[1], fusion[2], writes, ctx.n_seqs, self.n_heads,
                                                    self.n_kv_heads, self.head_dim, self.window, self.scale, n_split)
            else:
                ctx.kernels.decode.attn_decode(qkv, attn, ctx.seq_pos0, block_table, kpages, vpages, scratch, ctx.n_seqs,
                                               self.n_heads, self.n_kv_heads, self.head_dim, self.window, self.scale,
                                               n_split, tickets=tickets)
        elif x.dtype == torch.bfloat16 and self.head_dim in PrefillAttentionTC.HEAD_DIMS:
            ctx.kernels.prefill_attention_tc.attn(qkv, attn, ctx.seq_start, ctx.seq_pos0, block_table, kpages, vpages,
                                                  ctx.n_seqs, ctx.max_new, self.n_heads, self.n_kv_heads, self.head_dim,
                                                  self.window, self.scale, ctx.err_flag)
        elif ctx.is_decode and ctx.kernels.attn_decode_split_takes(self.head_dim, qkv.stride(0)):
            # one query per sequence on the generic path (the whole 32-bit decode step): keys split over blocks
            n_split = ctx.kernels.attn_decode_splits(ctx.n_seqs, self.n_heads, self.n_kv_heads, ctx.max_pages, ctx.engine.sm_count)
            part = torch.empty((ctx.n_seqs * self.n_heads * n_split * (self.head_dim + 2),), dtype=torch.float32,
                               device=x.device) if n_split > 1 else None
            ctx.kernels.attn_decode_split(qkv, attn, ctx.seq_pos0, block_table, kpages, vpages, part, ctx.n_seqs,
                                          self.n_heads, self.n_kv_heads, self.head_dim, self.window, self.scale, n_split)
        else:
            ctx.kernels.attn_paged(qkv, attn, ctx.seq_start, ctx.seq_pos0, block_table, kpages, vpages, ctx.n_seqs,
                                   ctx.max_new, self.n_heads, self.n_kv_heads, self.head_dim, self.window, self.scale)
        if fold is not None:
            return self.out.forward_folded(attn, ctx, fold=fold)
        return self.out.forward(attn, ctx, partials_ok=True)


MIXERS.register("attention", Attention)
