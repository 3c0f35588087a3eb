"""y = x W^T for one or several weight tensors stacked along the output dimension.

The reference runs Q, K, V (and gate, up) as separate products over the same input
(model_f32.go:391-396, :479-482); stacking their rows into one matrix gives the same numbers from
one pass over the input. Weights are [out, in] row-major as in the file (float32_ops.go:462-482).
"""
from __future__ import annotations

import torch

from ..weights.spec import TensorSpec
from .base import Folded, FoldRequest


class Linear:
    def __init__(self, names: list[str], out_features: list[int], in_features: int):
        self.names, self.out_features, self.in_features = list(names), list(out_features), in_features
        self.weight: torch.Tensor | None = None
        self._fold_ok = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(n, (o, self.in_features)) for n, o in zip(self.names, self.out_features)]

    def bind(self, tensors: dict, dtype, device) -> None:
        parts = [tensors[n] for n in self.names]
        if len({p.dtype for p in parts}) != 1:
            raise ValueError(f"tensors {self.names} are stored in different precisions and cannot be stacked")
        self.weight = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()
        self._fold_ok = None

    def rows(self, first: int, count: int) -> "Linear":
        """A view of `count` output rows from `first` (the query rows of a stacked q|k|v)."""
        sub = Linear([f"{self.names[0]}[{first}:{first + count}]"], [count], self.in_features)
        sub.weight = self.weight[first:first + count]
        return sub

    def fold_path(self, ctx, rows: int, dtype, finishing: bool = False):
        """Which kernel of this product, on `rows` rows of `dtype`, can take over a half of a norm:
        "few" (the decode step's few-rows kernel), "tiles" (the tensor-core kernels of a long prompt
        step) or None. `finishing`: the half that adds to the residual stream and prepares the norm's
        output (needs whole tiles of output columns); else the half that scales its output rows."""
        w = self.weight
        if dtype != torch.bfloat16 or w is None:
            return None
        if self._fold_ok is None:       # what does not change once the weights are bound
            self._fold_ok = bool(w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.stride(0) % 8 == 0 and w.stride(1) == 1
                                 and w.data_ptr() % 16 == 0)
        if not self._fold_ok:
            return None
        tc = ctx.kernels.tensor_core
        if rows <= ctx.kernels.decode.FOLD_MAX_M:
            return "few" if not finishing or w.shape[0] % 16 == 0 else None
        if rows >= tc.FOLD_MIN_M:
            return "tiles" if not finishing or (w.shape[0] % 32 == 0 and w.shape[0] > 128 and not tc.ONE_SM_FORCED) else None
        return None

    def forward_folded(self, x, ctx, fold: FoldRequest | None = None, swiglu_out=None):
        """The product with one or both halves of a norm folded in (only where `fold_path` said so).
        `x`: a Folded (its rows are owed their scale) or a plain tensor. `fold`: finish the sublayer
        (residual += y) and return the Folded input of the product behind the next norm; else
        returns y, or with `swiglu_out` fills it with silu(gate) * up."""
        owed = (x.sumsq, x.width, x.eps) if isinstance(x, Folded) else None
        a = x.x if isinstance(x, Folded) else x
        w = self.weight
        few = a.shape[0] <= ctx.kernels.decode.FOLD_MAX_M
        tc = ctx.kernels.tensor_core
        if fold is not None:
            n_out = w.shape[0]
            xb = torch.empty((a.shape[0], n_out), dtype=torch.bfloat16, device=a.device)
            sumsq = torch.empty((-(-n_out // (16 if few else tc.FOLD_SPAN)), a.shape[0]), dtype=torch.float32, device=a.device)
            if few:
                ctx.kernels.decode.gemm_small_m(a, w, fold.residual, owed=owed, fold=(fold.weight, xb, sumsq))
            else:
                tc.gemm(a, w, fold.residual, ctx.err_flag, owed=owed, fold=(fold.weight, xb, sumsq))
            return Folded(xb, sumsq, n_out, fold.eps)
        out = swiglu_out if swiglu_out is not None else torch.empty((a.shape[0], w.shape[0]), dtype=a.dtype, device=a.device)
        if few:
            ctx.kernels.decode.gemm_small_m(a, w, out, swiglu=swiglu_out is not None, owed=owed)
        else:
            tc.gemm(a, w, out, ctx.err_flag, swiglu=swiglu_out is not None, owed=owed)
        return out

    def forward(self, x: torch.Tensor, ctx, out_dtype=None, partials_ok: bool = False) -> torch.Tensor:
        """y [T, out] in `out_dtype` (default: x's). With `partials_ok` the result may instead be
        float32 [P, T, out] partial sums that add up to y (the reader, a norm, adds them): a product
        with few rows and few columns is split over K to fill the GPU."""
        w = self.weight
        out_dtype = out_dtype or x.dtype
        if w.dtype == x.dtype:
            if x.dtype == torch.bfloat16 and ctx.kernels.tensor_core.prefers_skinny(x, w, "partials" if partials_ok else "plain", ctx.engine.sm_count):
                tc = ctx.kernels.tensor_core
                split = tc.skinny_split(w.shape[0], w.shape[1], ctx.engine.sm_count) if partials_ok else 1
                shape = (split, x.shape[0], w.shape[0]) if split > 1 else (x.shape[0], w.shape[0])
                out = torch.empty(shape, dtype=torch.float32 if split > 1 else out_dtype, device=x.device)
                tc.gemm_skinny(x, w, out, ctx.err_flag)
                return out
            if x.dtype == torch.bfloat16 and ctx.kernels.decode.prefers(x, w, ctx.engine.sm_count):
                split = ctx.kernels.decode.split_for(w.shape[0], w.shape[1], ctx.engine.sm_count) if partials_ok else 1
                shape = (split, x.shape[0], w.shape[0]) if split > 1 else (x.shape[0], w.shape[0])
                out = torch.empty(shape, dtype=torch.float32 if split > 1 else out_dtype, device=x.device)
                ctx.kernels.decode.gemm_small_m(x, w, out)
                return out
            if x.dtype == torch.bfloat16 and ctx.kernels.tensor_core.takes(x, w):
                out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
                ctx.kernels.tensor_core.gemm(x, w, out, ctx.err_flag)
                return out
            split = ctx.kernels.gemm_nt_split(x.shape[0], w.shape[0], w.shape[1], ctx.engine.sm_count) if partials_ok else 1
            shape = (split, x.shape[0], w.shape[0]) if split > 1 else (x.shape[0], w.shape[0])
            out = torch.empty(shape, dtype=torch.float32 if split > 1 else out_dtype, device=x.device)
            ctx.kernels.gemm_nt(x, w, out)
            return out
        if w.dtype == torch.float32 and x.dtype == torch.bfloat16:
            # a matrix kept in 32-bit inside a bfloat16 model: widen the rows, multiply in 32-bit
            x32 = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            ctx.casts.to_f32(x, x32)
            out32 = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
            ctx.kernels_f32.gemm_nt(x32, w, out32)
            if out_dtype == torch.float32:
                return out32
            out = torch.empty(out32.shape, dtype=torch.bfloat16, device=x.device)
            ctx.casts.to_bf16(out32, out)
            return out
        raise ValueError(f"weight {self.names} is {w.dtype} but the engine runs in {x.dtype}")
