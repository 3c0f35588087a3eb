"""ctypes bindings of the kernel libraries: torch tensors in, launches on torch's current stream.

`KernelSet(dtype)` gives the launchers of one element type (float32: the true 32-bit set;
bfloat16: the serving set). Every wrapper checks device, dtype and contiguity before it passes a
pointer on, and raises on a non-zero return code. There is no CPU path: a tensor that is not on a
CUDA device is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load_library



class KernelError(RuntimeError):
    pass


def _ptr(t: torch.Tensor | None, dtype=None, name="tensor"):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on a CUDA device only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return c_void_p(t.data_ptr())


try:        # the raw handle of torch's current stream without building a Stream object (a launch costs microseconds)
    _raw_stream, _current_device = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:      # a torch without these entry points: the public, slower way
    _raw_stream = _current_device = None


def _stream():
    if _raw_stream is not None:
        return c_void_p(_raw_stream(_current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = [0]   # kernels enqueued through these bindings since import (a bench reads the difference)


def _check(code: int, what: str):
    LAUNCHES[0] += 1
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: arguments refused by the launcher (code {code})")
    raise KernelError(f"{what}: CUDA error {code} ({_cuda_error_name(code)})")


def _cuda_error_name(code: int) -> str:
    try:
        rt = ctypes.CDLL("libcudart.so")
        rt.cudaGetErrorString.restype = ctypes.c_char_p
        return rt.cudaGetErrorString(code).decode()
    except OSError:
        return "see cudaError_t"


_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}


class KernelSet:
    """Launchers for activations and weights of one element type."""

    def __init__(self, dtype: torch.dtype):
        if dtype not in _SUFFIX:
            raise KernelError(f"no kernels for {dtype}; supported: float32, bfloat16")
        self.dtype = dtype
        self.suffix = _SUFFIX[dtype]
        self.lib = load_library(self.suffix)
        self._fns: dict[str, object] = {}

    def _fn(self, name):
        fn = self._fns.get(name)
        if fn is None:
            fn = getattr(self.lib, f"sllm_{name}_{self.suffix}")
            fn.restype = c_int
            self._fns[name] = fn
        return fn

    # ------------------------------------------------------------------ embedding
    def embed_rows(self, ids, table, out, err_flag):
        T, d = out.shape
        _check(self._fn("embed_rows")(_ptr(ids, torch.int32, "ids"), _ptr(table, self.dtype, "table"),
                                      _ptr(out, torch.float32, "out"), c_int(T), c_int(d), c_int(table.shape[0]),
                                      _ptr(err_flag, torch.int32, "err"), _stream()), "embed_rows")

    # ------------------------------------------------------------------ norm
    def add_rmsnorm(self, x, delta, rows, weight, y, eps):
        """x float32 [T,d] residual (+= delta when rows is None); y [n,d] normed output. delta: None,
        [T,d] of this set's dtype, or float32 [P,T,d] partial sums that add up to the addend."""
        d = x.shape[-1]
        n = y.shape[0]
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"norm weight has dtype {weight.dtype}")
        n_parts, stride = 0, 0
        if delta is not None and delta.dim() == 3:
            if delta.dtype != torch.float32 or tuple(delta.shape[1:]) != tuple(x.shape):
                raise KernelError(f"partial sums must be float32 [P, {x.shape[0]}, {d}], found {delta.dtype} {tuple(delta.shape)}")
            n_parts, stride = delta.shape[0], x.shape[0] * d
        elif delta is not None and (delta.dtype != self.dtype or tuple(delta.shape) != tuple(x.shape)):
            raise KernelError(f"addend must be {self.dtype} {tuple(x.shape)}, found {delta.dtype} {tuple(delta.shape)}")
        _check(self._fn("add_rmsnorm")(_ptr(x, torch.float32, "x"), _ptr(delta, None, "delta"), c_int(n_parts),
                                       c_longlong(stride), _ptr(rows, torch.int32, "rows"), _ptr(weight, None, "weight"),
                                       c_int(1 if weight.dtype == torch.float32 else 0), _ptr(y, self.dtype, "y"),
                                       c_int(n), c_int(d), c_float(eps), _stream()), "add_rmsnorm")

    # ------------------------------------------------------------------ matrix products
    def gemm_nt(self, a, w, out):
        """out[M,N] = a[M,K] @ w[N,K]^T; `out` is of this set's dtype or float32. A float32 `out` of
        shape [P,M,N] receives P partial sums (K cut into P parts); the reader adds them."""
        M, K = a.shape
        N = w.shape[0]
        ksplit = out.shape[0] if out.dim() == 3 else 1
        if w.shape[1] != K or tuple(out.shape[-2:]) != (M, N) or (out.dim() == 3 and out.dtype != torch.float32):
            raise KernelError(f"gemm_nt shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
        out_f32 = 1 if (out.dtype == torch.float32 and self.dtype != torch.float32) else 0
        _check(self._fn("gemm_nt")(_ptr(a, self.dtype, "a"), _ptr(w, self.dtype, "w"),
                                   _ptr(out, torch.float32 if out_f32 else self.dtype, "out"), c_int(M), c_int(N),
                                   c_int(K), c_int(a.stride(0)), c_int(w.stride(0)), c_int(N), c_int(out_f32),
                                   c_int(ksplit), _stream()), "gemm_nt")

    @staticmethod
    def gemm_nt_split(m: int, n_out: int, k: int, sm_count: int) -> int:
        """Into how many parts the generic product cuts K when its reader takes partial sums: none for
        up to 8 rows (a block per four columns fills the GPU already) or when the 128-column tiles
        fill it; else enough parts for about two blocks per SM, each at least 256 deep."""
        if m <= 8 or k % 4:
            return 1
        tiles = -(-n_out // 128) * -(-m // (64 if m <= 64 else 128))
        if tiles >= sm_count:
            return 1
        return max(1, min(2 * sm_count // tiles, k // 256, 16))

    # ------------------------------------------------------------------ rotary + cache write
    def rope_kv_write(self, qkv, tok_pos, tok_seq, block_table, cos_sin, kpages, vpages, n_heads, n_kv, head_dim, rot,
                      interleaved):
        T, ld = qkv.shape
        _check(self._fn("rope_kv_write")(_ptr(qkv, self.dtype, "qkv"), c_int(ld), _ptr(tok_pos, torch.int32, "tok_pos"),
                                         _ptr(tok_seq, torch.int32, "tok_seq"),
                                         _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
                                         _ptr(cos_sin, torch.float32, "cos_sin"),
                                         _ptr(kpages, self.dtype if kpages is not None else None, "kpages"),
                                         _ptr(vpages, self.dtype if vpages is not None else None, "vpages"), c_int(T),
                                         c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(rot),
                                         c_int(1 if interleaved else 0), _stream()), "rope_kv_write")

    # ------------------------------------------------------------------ attention
    def attn_paged(self, q, out, seq_start, seq_pos0, block_table, kpages, vpages, n_seqs, max_new, n_heads, n_kv,
                   head_dim, window, scale):
        _check(self._fn("attn_paged")(_ptr(q, self.dtype, "q"), c_int(q.shape[1]), _ptr(out, self.dtype, "out"),
                                      _ptr(seq_start, torch.int32, "seq_start"), _ptr(seq_pos0, torch.int32, "seq_pos0"),
                                      _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
                                      _ptr(kpages, self.dtype, "kpages"), _ptr(vpages, self.dtype, "vpages"),
                                      c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv), c_int(head_dim),
                                      c_int(window or 0), c_float(scale), _stream()), "attn_paged")

    def attn_decode_split(self, q, out, seq_pos0, block_table, kpages, vpages, part, n_seqs, n_heads, n_kv, head_dim,
                          window, scale, n_split):
        """One query per sequence, each sequence's keys split over `n_split` blocks (then merged);
        `part`: float32 scratch of n_seqs * n_heads * n_split * (head_dim + 2) elements, or None for one split."""
        need = n_seqs * n_heads * n_split * (head_dim + 2) if n_split > 1 else 0
        if need and (part is None or part.numel() < need):
            raise KernelError(f"attn_decode_split scratch holds {0 if part is None else part.numel()} floats, needs {need}")
        _check(self._fn("attn_decode_split")(_ptr(q, self.dtype, "q") if q.is_contiguous() else c_void_p(q.data_ptr()),
                                             c_int(q.stride(0)), _ptr(out, self.dtype, "out"),
                                             _ptr(seq_pos0, torch.int32, "seq_pos0"),
                                             _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
                                             _ptr(kpages, self.dtype, "kpages"), _ptr(vpages, self.dtype, "vpages"),
                                             _ptr(part, torch.float32, "part"), c_int(n_seqs), c_int(n_heads), c_int(n_kv),
                                             c_int(head_dim), c_int(window or 0), c_float(scale), c_int(n_split), _stream()),
               "attn_decode_split")

    @staticmethod
    def attn_decode_split_takes(head_dim: int, q_ld: int) -> bool:
        return head_dim % 4 == 0 and 4 <= head_dim <= 512 and q_ld % 4 == 0

    @staticmethod
    def attn_decode_splits(n_seqs: int, n_heads: int, n_kv: int, pages: int, sm_count: int) -> int:
        """Blocks per (sequence, key/value head, pass over the keys; a pass serves up to four of the
        query heads that share the key/value head): enough for about six blocks of four warps per SM,
        at most one per page."""
        passes = -(-(n_heads // n_kv) // 4)       # (wide heads, above 128: two heads a pass; the estimate stays)
        want = -(-6 * sm_count // max(1, n_seqs * n_kv * passes))
        return max(1, min(want, pages, 64))

    # ------------------------------------------------------------------ feed-forward
    def swiglu(self, gate_up, out, tiled=False):
        T, F = out.shape
        if tuple(gate_up.shape) != (T, 2 * F):
            raise KernelError(f"swiglu shapes: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
        _check(self._fn("swiglu")(_ptr(gate_up, self.dtype, "gate_up"), _ptr(out, self.dtype, "out"), c_int(T), c_int(F),
                                  c_int(1 if tiled else 0), _stream()), "swiglu")

    # ------------------------------------------------------------------ fast bfloat16 kernels
    @property
    def tensor_core(self) -> "TensorCoreGemm":
        if self.dtype != torch.bfloat16:
            raise KernelError("the tensor-core GEMM is bfloat16 only")
        if getattr(self, "_tc", None) is None:
            self._tc = TensorCoreGemm()
        return self._tc

    @property
    def prefill_attention_tc(self) -> "PrefillAttentionTC":
        if self.dtype != torch.bfloat16:
            raise KernelError("the tensor-core attention is bfloat16 only")
        if getattr(self, "_fa_tc", None) is None:
            self._fa_tc = PrefillAttentionTC()
        return self._fa_tc

    @property
    def decode(self) -> "DecodeKernels":
        if self.dtype != torch.bfloat16:
            raise KernelError("the decode kernels are bfloat16 only")
        if getattr(self, "_decode", None) is None:
            self._decode = DecodeKernels()
        return self._decode


class TensorCoreGemm:
    """bfloat16 GEMM on tcgen05 tensor cores with TMA-fed shared memory (the prompt step's products)."""

    def __init__(self):
        self.lib = load_library("gemm_tcgen05")
        for n in ("sllm_gemm_tc_bf16", "sllm_gemm_tc_fold_bf16", "sllm_gemm_tc_skinny_bf16", "sllm_gemm_tc_qkv_rope_bf16",
                  "sllm_gemm_tc_qkv_rope_fold_bf16"):
            getattr(self.lib, n).restype = c_int

    @staticmethod
    def takes(a, w) -> bool:
        return (a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1
                and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    @staticmethod
    def _owed_args(owed, M):
        if owed is None:
            return c_void_p(None), c_int(0), c_int(0), c_float(0.0)
        sq, width, eps = owed
        if sq.dtype != torch.float32 or sq.dim() != 2 or sq.shape[1] != M or not sq.is_contiguous():
            raise KernelError(f"sums of squares {tuple(sq.shape)} {sq.dtype} for {M} rows")
        return _ptr(sq, torch.float32, "sumsq"), c_int(sq.shape[0]), c_int(width), c_float(eps)

    FOLD_SPAN = 128      # columns to a partial sum of squares that a folded product leaves
    FOLD_MIN_M = 129     # the product that finishes a sublayer for a folded norm runs on the two-SM tiles only
    ONE_SM_FORCED = os.environ.get("SLLM_GEMM_ONE_SM", "0") not in ("", "0")      # a debugging switch of the library

    def gemm(self, a, w, out, err_flag, swiglu=False, owed=None, fold=None):
        """out[M,N] = a @ w^T in bfloat16 or float32; swiglu: out[M,N/2] = silu(gate)*up for w's rows
        tiled 8 gate / 8 up. `err_flag` (int32 on the device) is set if a wait in the kernel timed out.
        `owed` = (sumsq float32 [P, M], width, eps): the rows of `a` are a norm's v * weight whose scale
        rsqrt(sum of v^2 / width + eps) is applied to the output rows instead. `fold` = (norm_weight
        float32 [N], xb bfloat16 [M, N], sumsq_out float32 [ceil(N / 128), M]): `out` is the float32
        residual stream [M, N] (M >= FOLD_MIN_M, N > 128 and a multiple of 32); it receives the product,
        and xb and sumsq_out what the product behind the following norm is owed."""
        M, K = a.shape
        N = w.shape[0]
        if fold is not None:
            norm_w, xb, sq_out = fold
            if (swiglu or out.dtype != torch.float32 or tuple(out.shape) != (M, N) or N % 32 or N <= 128 or M < self.FOLD_MIN_M
                    or tuple(norm_w.shape) != (N,) or norm_w.dtype != torch.float32 or tuple(xb.shape) != (M, N)
                    or xb.dtype != torch.bfloat16 or not xb.is_contiguous() or tuple(sq_out.shape) != (-(-N // self.FOLD_SPAN), M)
                    or not sq_out.is_contiguous() or w.shape[1] != K or out.stride(1) != 1):
                raise KernelError(f"gemm_tc fold: residual {tuple(out.shape)} {out.dtype}, norm weight {tuple(norm_w.shape)}, "
                                  f"xb {tuple(xb.shape)}, sums {tuple(sq_out.shape)} for M={M}, N={N}")
            _check(self.lib.sllm_gemm_tc_fold_bf16(
                c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
                c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(1), c_int(2), *self._owed_args(owed, M),
                _ptr(norm_w, torch.float32, "norm_w"), _ptr(xb, torch.bfloat16, "xb"), _ptr(sq_out, torch.float32, "sumsq_out"),
                _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_tc")
            return
        want = (M, N // 2) if swiglu else (M, N)
        if tuple(out.shape) != want or w.shape[1] != K or out.stride(1) != 1:
            raise KernelError(f"gemm_tc shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_tc dtypes: a {a.dtype}, w {w.dtype}, out {out.dtype}")
        if not (a.is_cuda and w.is_cuda and out.is_cuda):
            raise KernelError("gemm_tc runs on a CUDA device only")
        _check(self.lib.sllm_gemm_tc_fold_bf16(
            c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
            c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(1 if swiglu else 0), *self._owed_args(owed, M), c_void_p(None), c_void_p(None), c_void_p(None),
            _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_tc")


    QKV_ROPE_HEAD_DIMS = (64, 128)

    @classmethod
    def rotation_fusable(cls, head_dim: int, rot: int, interleaved: bool) -> bool:
        """Whether the q|k|v product's epilogue can rotate by a (cos, sin) table and fill the cache
        itself: its 32-column chunks must hold whole pairs, or both halves of a fully rotated head."""
        return head_dim in cls.QKV_ROPE_HEAD_DIMS and (interleaved or rot == head_dim)

    def gemm_qkv_rope(self, a, w, qkv, err_flag, tok_pos, tok_seq, block_table, cos_sin, kpages, vpages, n_heads, n_kv,
                      head_dim, rot, interleaved, owed=None):
        """qkv[:, :n_heads*head_dim] = rotated queries of a @ w^T (w rows: q | k | v heads); the rotated
        keys and the values go to each row's place in the cache pages and not to `qkv`. `owed`: as in `gemm`."""
        M, K = a.shape
        N = (n_heads + 2 * n_kv) * head_dim
        if tuple(w.shape) != (N, K) or qkv.shape[0] != M or qkv.shape[1] < n_heads * head_dim or qkv.stride(1) != 1:
            raise KernelError(f"gemm_qkv_rope shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, qkv {tuple(qkv.shape)}")
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16:
            raise KernelError("gemm_qkv_rope works in bfloat16")
        _check(self.lib.sllm_gemm_tc_qkv_rope_fold_bf16(
            c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(qkv.data_ptr()), c_int(M), c_int(K), c_int(a.stride(0)),
            c_int(w.stride(0)), c_int(qkv.stride(0)), _ptr(tok_pos, torch.int32, "tok_pos"), _ptr(tok_seq, torch.int32, "tok_seq"),
            _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), _ptr(cos_sin, torch.float32, "cos_sin"),
            _ptr(kpages, torch.bfloat16, "kpages"), _ptr(vpages, torch.bfloat16, "vpages"), c_int(n_heads), c_int(n_kv),
            c_int(head_dim), c_int(rot), c_int(1 if interleaved else 0), *self._owed_args(owed, M),
            _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_qkv_rope")

    SKINNY_MAX_M = 128

    def gemm_skinny(self, a, w, out, err_flag, swiglu=False):
        """The same product for at most 128 rows of `a`, with the weights as the tensor cores' 128-row
        operand and a grid over (128 weight rows, K splits). out [M,N] bfloat16 or float32, or
        [M,N/2] with swiglu; float32 [P,M,N]: K split P ways, out receives the partial sums."""
        M, K = a.shape
        N = w.shape[0]
        ksplit = out.shape[0] if out.dim() == 3 else 1
        want = (M, N // 2) if swiglu else ((ksplit, M, N) if out.dim() == 3 else (M, N))
        if out.dim() == 3 and out.dtype != torch.float32:
            raise KernelError("partial sums are written in float32")
        if tuple(out.shape) != want or w.shape[1] != K or not out.is_contiguous():
            raise KernelError(f"gemm_skinny shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_skinny dtypes: a {a.dtype}, w {w.dtype}, out {out.dtype}")
        if not (a.is_cuda and w.is_cuda and out.is_cuda):
            raise KernelError("gemm_skinny runs on a CUDA device only")
        _check(self.lib.sllm_gemm_tc_skinny_bf16(
            c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
            c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(-2)), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(1 if swiglu else 0), c_int(ksplit), _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_skinny")

    def prefers_skinny(self, a, w, kind: str, sm_count: int) -> bool:
        """True where the few-rows kernel is the fastest of the three products for a [M,K] x [N,K]^T
        (measured on the layer shapes of 1-8 B models): 9..128 rows; always when the reader takes
        partial sums ("partials": K is split to fill the GPU); with the SiLU gate ("swiglu") up to 64
        rows; a plain product ("plain") from 33 rows on and only while its N/128 blocks fit one wave
        of the GPU's `sm_count` SMs."""
        M, N = a.shape[0], w.shape[0]
        if not (8 < M <= self.SKINNY_MAX_M and self.takes(a, w)):
            return False
        if kind == "partials":
            return True
        if kind == "swiglu":
            return M <= 64
        return M > 32 and N <= 128 * sm_count

    @staticmethod
    def skinny_split(n_out: int, k: int, sm_count: int) -> int:
        """Over how many blocks to split K so that the (n_out / 128) x split grid about fills the GPU."""
        tiles = -(-n_out // 128)
        return max(1, min(sm_count // tiles, k // 256, 16))


class PrefillAttentionTC:
    """tcgen05 causal attention of a prompt step over the paged cache (bfloat16, head width 64 or 128)."""
    HEAD_DIMS = (64, 128)

    def __init__(self):
        self.lib = load_library("attn_prefill_tcgen05")
        self.lib.sllm_attn_prefill_tc_bf16.restype = c_int

    def attn(self, q, out, seq_start, seq_pos0, block_table, kpages, vpages, n_seqs, max_new, n_heads, n_kv, head_dim,
             window, scale, err_flag):
        _check(self.lib.sllm_attn_prefill_tc_bf16(
            _ptr(q, torch.bfloat16, "q"), c_int(q.shape[1]), c_int(q.shape[0]), _ptr(out, torch.bfloat16, "out"),
            _ptr(seq_start, torch.int32, "seq_start"), _ptr(seq_pos0, torch.int32, "seq_pos0"),
            _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
            _ptr(kpages, torch.bfloat16, "kpages"), _ptr(vpages, torch.bfloat16, "vpages"), c_longlong(kpages.shape[0]),
            c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(window or 0), c_float(scale),
            _ptr(err_flag, torch.int32, "err_flag"), _stream()), "attn_prefill_tc")


class DecodeKernels:
    """Weight-streaming small-M product and split-key attention for the bfloat16 decode step."""
    HEAD_DIMS = (16, 32, 64, 128, 256)
    MAX_M = 64

    def __init__(self):
        self.lib = load_library("decode_bf16")
        for n in ("sllm_gemm_small_m_bf16", "sllm_gemm_small_m_fold_bf16", "sllm_attn_decode_bf16",
                  "sllm_attn_decode_merged_bf16", "sllm_attn_decode_rope_bf16"):
            getattr(self.lib, n).restype = c_int
        self.lib.sllm_attn_decode_scratch_bytes.restype = c_longlong
        self.lib.sllm_attn_decode_uses_mma.restype = c_int

    @staticmethod
    def takes(a, w) -> bool:
        K = a.shape[1]
        return (a.shape[0] <= DecodeKernels.MAX_M and K % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)

    @staticmethod
    def prefers(a, w, sm_count: int) -> bool:
        """True when this kernel is the faster one for the shape: always up to 16 rows; beyond that
        only while the output is too narrow to give the 128 x 256 tensor-core tiles enough blocks
        (fewer than a third of the SMs; measured at 148: 48 tiles)."""
        return DecodeKernels.takes(a, w) and (a.shape[0] <= 16 or 3 * -(-w.shape[0] // 256) <= sm_count)

    @staticmethod
    def rotation_fusable(rot: int, interleaved: bool) -> bool:
        """Whether the decode attention kernel can rotate queries and the new key by a (cos, sin)
        table itself: its 16-byte vectors must not straddle the rotary width or its half."""
        return rot >= 2 and rot % (8 if interleaved else 16) == 0

    MAX_SPLITS = 64      # beyond this the merging block falls back to a slow loop

    def attention_splits(self, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int, pages: int, sm_count: int) -> int:
        """Over how many blocks a decode step splits each sequence's keys: about as many blocks as are
        resident at once (a second wave that is far from full costs a whole one), never more than the
        longest sequence has pages. The tensor-core kernel (grouped queries, or very few sequences)
        has fatter blocks: its registers allow four per SM at width 64, two at width 128, and it wants
        at least four pages each. The one-head kernel is built for seven per SM (three where it serves
        several query heads per key/value head at other widths); a tenth more blocks than that still
        beat leaving a quarter of the places empty (measured at context 4,096: 12 sequences 64.5 us
        with 1,152 blocks against 74.6 with 768; 6 sequences 36.1 with 1,152 against 37.2 with 960;
        16 sequences 84.6 with 1,024 against 98.8 with 1,536)."""
        pairs = max(1, n_seqs * n_kv_heads)
        if self.lib.sllm_attn_decode_uses_mma(c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim)):
            want, cap = ((4 if head_dim <= 64 else 2) * sm_count) // pairs, max(1, pages // 4)
        else:
            want, cap = ((39 if n_heads == n_kv_heads else 17) * sm_count) // (5 * pairs), pages
        n = max(1, min(want, cap, DecodeKernels.MAX_SPLITS))
        per = -(-pages // n)                   # pages a block takes; the fewest blocks that need no more each
        return max(1, -(-pages // per)) if pages > 0 else n

    FOLD_MAX_M = 16      # rows up to which a product can take over one half of a norm

    def gemm_small_m(self, a, w, out, swiglu=False, owed=None, fold=None):
        """out[M,N] = a @ w^T (bfloat16 or float32 out); swiglu: out[M,N/2] = silu(gate)*up for w rows
        tiled 8 gate / 8 up; out float32 [P,M,N]: K split P ways, out receives the partial sums.
        `owed` = (sumsq float32 [P, M], width, eps): the rows of `a` are a norm's v * weight whose scale
        rsqrt(sum of v^2 / width + eps) is applied to the output rows instead. `fold` = (norm_weight
        float32 [N], xb bfloat16 [M, N], sumsq_out float32 [ceil(N / 16), M]): `out` is the float32
        residual stream [M, N]; it receives the product, and xb and sumsq_out what the product after
        the following norm is owed (M <= FOLD_MAX_M)."""
        M, K = a.shape
        N = w.shape[0]
        if owed is not None or fold is not None:
            return self._gemm_small_m_fold(a, w, out, swiglu, owed, fold)
        ksplit = out.shape[0] if out.dim() == 3 else 1
        want = (M, N // 2) if swiglu else ((ksplit, M, N) if out.dim() == 3 else (M, N))
        if out.dim() == 3 and out.dtype != torch.float32:
            raise KernelError("partial sums are written in float32")
        if tuple(out.shape) != want or w.shape[1] != K:
            raise KernelError(f"gemm_small_m shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_small_m output dtype {out.dtype}")
        _check(self.lib.sllm_gemm_small_m_bf16(
            _ptr(a, torch.bfloat16, "a") if a.is_contiguous() else c_void_p(a.data_ptr()),
            _ptr(w, torch.bfloat16, "w"), _ptr(out, None, "out"), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
            c_int(w.stride(0)), c_int(out.stride(-2)), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(1 if swiglu else 0), c_int(ksplit), _stream()), "gemm_small_m")

    def _gemm_small_m_fold(self, a, w, out, swiglu, owed, fold):
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.dim() != 2 or (fold is not None and swiglu):
            raise KernelError(f"gemm_small_m shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        sumsq_in, n_in, width, eps = c_void_p(None), 0, 0, 0.0
        if owed is not None:
            sq, width, eps = owed
            if sq.dtype != torch.float32 or sq.dim() != 2 or sq.shape[1] != M or not sq.is_contiguous():
                raise KernelError(f"gemm_small_m: sums of squares {tuple(sq.shape)} {sq.dtype} for {M} rows")
            sumsq_in, n_in = _ptr(sq, torch.float32, "sumsq"), sq.shape[0]
        if fold is not None:
            norm_w, xb, sq_out = fold
            tiles = -(-N // 16)
            if (M > self.FOLD_MAX_M or out.dtype != torch.float32 or tuple(out.shape) != (M, N) or tuple(norm_w.shape) != (N,)
                    or tuple(xb.shape) != (M, N) or not xb.is_contiguous() or tuple(sq_out.shape) != (tiles, M)
                    or not sq_out.is_contiguous()):
                raise KernelError(f"gemm_small_m fold: residual {tuple(out.shape)} {out.dtype}, norm weight {tuple(norm_w.shape)}, "
                                  f"xb {tuple(xb.shape)}, sums {tuple(sq_out.shape)} for M={M}, N={N}")
            tail = (_ptr(norm_w, torch.float32, "norm_w"), _ptr(xb, torch.bfloat16, "xb"), _ptr(sq_out, torch.float32, "sumsq_out"))
            epilogue = 2
        else:
            want = (M, N // 2) if swiglu else (M, N)
            if tuple(out.shape) != want or out.dtype not in (torch.bfloat16, torch.float32):
                raise KernelError(f"gemm_small_m out {tuple(out.shape)} {out.dtype}, want {want}")
            tail = (c_void_p(None), c_void_p(None), c_void_p(None))
            epilogue = 1 if swiglu else 0
        _check(self.lib.sllm_gemm_small_m_fold_bf16(
            _ptr(a, torch.bfloat16, "a") if a.is_contiguous() else c_void_p(a.data_ptr()),
            _ptr(w, torch.bfloat16, "w"), _ptr(out, None, "out"), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
            c_int(w.stride(0)), c_int(out.stride(-2)), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(epilogue), c_int(1), sumsq_in, c_int(n_in), c_int(width), c_float(eps), *tail, _stream()), "gemm_small_m")

    def attn_decode_rope(self, qkv, out, seq_pos0, block_table, kpages, vpages, scratch, tickets, cos_sin, rot,
                         interleaved, write_kv, n_seqs, n_heads, n_kv, head_dim, window, scale, n_split):
        """Rotary positions, cache write and attention of a decode step in one kernel: `qkv` holds the
        unrotated [q | k | v] rows of the step (only q when write_kv is false)."""
        need = self.lib.sllm_attn_decode_scratch_bytes(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(n_split))
        if scratch.numel() * scratch.element_size() < need or tickets.numel() < n_seqs * n_kv:
            raise KernelError("attn_decode_rope: scratch or tickets too small")
        width = (n_heads + 2 * n_kv) * head_dim if write_kv else n_heads * head_dim
        if qkv.shape[1] < width:
            raise KernelError(f"attn_decode_rope: rows of {qkv.shape[1]} columns, need {width}")
        _check(self.lib.sllm_attn_decode_rope_bf16(
            _ptr(qkv, torch.bfloat16, "qkv"), c_int(qkv.shape[1]), _ptr(out, torch.bfloat16, "out"),
            _ptr(seq_pos0, torch.int32, "seq_pos0"), _ptr(block_table, torch.int32, "block_table"),
            c_int(block_table.shape[1]), _ptr(kpages, torch.bfloat16, "kpages"), _ptr(vpages, torch.bfloat16, "vpages"),
            _ptr(scratch, torch.float32, "scratch"), _ptr(tickets, torch.int32, "tickets"),
            _ptr(cos_sin, torch.float32, "cos_sin"), c_int(rot), c_int(1 if interleaved else 0), c_int(1 if write_kv else 0),
            c_int(n_seqs), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(window or 0), c_float(scale), c_int(n_split),
            _stream()), "attn_decode_rope")

    def split_for(self, n_out: int, k: int, sm_count: int) -> int:
        """Over how many blocks to split K so that a product with few output rows still fills the GPU."""
        tiles = -(-n_out // 16)
        return max(1, min(8, (4 * sm_count) // tiles, k // 512))

    def attn_decode(self, q, out, seq_pos0, block_table, kpages, vpages, scratch, n_seqs, n_heads, n_kv, head_dim,
                    window, scale, n_split, tickets=None):
        """`tickets` (int32 [>= n_seqs * n_kv], zero before its first use, left zero): the last split
        to finish merges the partial results in the same kernel; without it a second kernel merges."""
        need = self.lib.sllm_attn_decode_scratch_bytes(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(n_split))
        if scratch.numel() * scratch.element_size() < need:
            raise KernelError(f"attn_decode scratch holds {scratch.numel() * scratch.element_size()} bytes, needs {need}")
        head = (_ptr(q, torch.bfloat16, "q"), c_int(q.shape[1]), _ptr(out, torch.bfloat16, "out"),
                _ptr(seq_pos0, torch.int32, "seq_pos0"), _ptr(block_table, torch.int32, "block_table"),
                c_int(block_table.shape[1]), _ptr(kpages, torch.bfloat16, "kpages"), _ptr(vpages, torch.bfloat16, "vpages"),
                _ptr(scratch, torch.float32, "scratch"))
        tail = (c_int(n_seqs), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(window or 0), c_float(scale),
                c_int(n_split), _stream())
        if tickets is None:
            _check(self.lib.sllm_attn_decode_bf16(*head, *tail), "attn_decode")
        else:
            if tickets.numel() < n_seqs * n_kv:
                raise KernelError(f"attn_decode tickets hold {tickets.numel()} ints, needs {n_seqs * n_kv}")
            _check(self.lib.sllm_attn_decode_merged_bf16(*head, _ptr(tickets, torch.int32, "tickets"), *tail), "attn_decode")


class CastKernels:
    """bfloat16 <-> float32 copies (a matrix stored in 32-bit inside a bfloat16 model)."""

    def __init__(self):
        self.lib = load_library("bf16")

    def to_f32(self, src, dst):
        fn = self.lib.sllm_cast_bf16_to_f32
        fn.restype = c_int
        _check(fn(_ptr(src, torch.bfloat16, "src"), _ptr(dst, torch.float32, "dst"), c_longlong(src.numel()), _stream()),
               "cast_bf16_to_f32")

    def to_bf16(self, src, dst):
        fn = self.lib.sllm_cast_f32_to_bf16
        fn.restype = c_int
        _check(fn(_ptr(src, torch.float32, "src"), _ptr(dst, torch.bfloat16, "dst"), c_longlong(src.numel()), _stream()),
               "cast_f32_to_bf16")


class RandomKernels:
    """Fills tensors with the counter-based generator of random-weights mode (lib_random.cu)."""

    def __init__(self):
        self.lib = load_library("random")
        self.lib.sllm_fill_normal.restype = c_int
        self.lib.sllm_fill_integer.restype = c_int

    def fill_normal(self, out, seed: int, index: int, mean: float, std: float):
        if out.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"fill_normal writes float32 or bfloat16, not {out.dtype}")
        _check(self.lib.sllm_fill_normal(_ptr(out, None, "out"), c_int(0 if out.dtype == torch.float32 else 1),
                                         c_longlong(out.numel()), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                                         ctypes.c_uint(index), ctypes.c_double(mean), ctypes.c_double(std), _stream()),
               "fill_normal")

    def fill_integer(self, out, seed: int, index: int, modulus: int):
        _check(self.lib.sllm_fill_integer(_ptr(out, torch.int32, "out"), c_longlong(out.numel()),
                                          ctypes.c_ulonglong(seed & (2 ** 64 - 1)), ctypes.c_uint(index),
                                          ctypes.c_uint(modulus), _stream()), "fill_integer")


class ProbeKernels:
    """Measuring sticks for benchmarks (lib_probe.cu)."""

    def __init__(self):
        self.lib = load_library("probe")
        self.lib.sllm_fma_loop.restype = c_int

    def fma_tflops(self, device="cuda:0", blocks_per_sm: int = 8, iters: int = 1 << 15, repeats: int = 5) -> float:
        """Best-of-`repeats` rate of float fused multiply-adds (2 operations each) in TFLOP/s."""
        dev = torch.device(device)
        blocks = torch.cuda.get_device_properties(dev).multi_processor_count * blocks_per_sm
        out = torch.empty(blocks * 256, dtype=torch.float32, device=dev)
        best = 0.0
        for i in range(repeats + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _check(self.lib.sllm_fma_loop(_ptr(out, torch.float32, "out"), c_int(blocks), c_int(iters), _stream()), "fma_loop")
            e1.record()
            e1.synchronize()
            if i:
                best = max(best, blocks * 256 * iters * 16 / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        return best


class SamplingKernels:
    STRATEGIES = {"greedy": 0, "temperature": 1, "top_k": 2, "top_p": 3}
    PARAM_WORDS = 8   # int32 words per row: strategy, temperature, top_k, top_p, seed lo/hi, draw lo/hi

    def __init__(self):
        self.lib = load_library("sampling")

    def sample_rows(self, logits, params, out):
        """logits float32 [n, V] (row stride = logits.stride(0)); params int32 [n, 8]; out int32 [n]."""
        if logits.dim() != 2 or logits.stride(1) != 1:
            raise KernelError("logits must be [rows, vocab] with unit column stride")
        n, V = logits.shape
        fn = self.lib.sllm_sample_rows
        fn.restype = c_int
        if not logits.is_cuda or logits.dtype != torch.float32:
            raise KernelError("logits must be float32 on a CUDA device")
        _check(fn(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), c_int(n), c_int(V),
                  _ptr(params, torch.int32, "params"), _ptr(out, torch.int32, "out"), _stream()), "sample_rows")

    STATE_WORDS = 8   # int32 words of a sequence's state record: pos, generated, last token, flags, key x2, counter x2

    def sample_rows_state(self, logits, options, state, slots, pos_after, stop_ids, out):
        """The same, every row's sampling key and draw counter read from (and advanced in) its
        sequence's record state[slots[row]]; options int32 [4] on the device; stop_ids int32 [n] or None."""
        if logits.dim() != 2 or logits.stride(1) != 1 or not logits.is_cuda or logits.dtype != torch.float32:
            raise KernelError("logits must be float32 [rows, vocab] with unit column stride on a CUDA device")
        n, V = logits.shape
        if state.dim() != 2 or state.shape[1] != self.STATE_WORDS or slots.shape[0] < n or out.shape[0] < n:
            raise KernelError("sample_rows_state: state must be [slots, 8] and slots/out must cover every row")
        fn = self.lib.sllm_sample_rows_state
        fn.restype = c_int
        _check(fn(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), c_int(n), c_int(V), _ptr(options, torch.int32, "options"),
                  _ptr(state, torch.int32, "state"), _ptr(slots, torch.int32, "slots"), _ptr(pos_after, torch.int32, "pos_after"),
                  _ptr(stop_ids, torch.int32, "stop_ids"), c_int(0 if stop_ids is None else stop_ids.numel()),
                  _ptr(out, torch.int32, "out"), _stream()), "sample_rows_state")

    def repeat_penalty(self, logits, recent, counts, penalty, last_n):
        n, V = logits.shape
        fn = self.lib.sllm_repeat_penalty
        fn.restype = c_int
        _check(fn(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), c_int(n), c_int(V),
                  _ptr(recent, torch.int32, "recent"), c_int(recent.shape[1]), _ptr(counts, torch.int32, "counts"),
                  _ptr(penalty, torch.float32, "penalty"), c_int(last_n), _stream()), "repeat_penalty")
