"""Each kernel alone against the plain implementation's function for the same op, at sizes other
than any model's (odd widths, head widths in steps of 16, vocabularies that are no power of two)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as plain
from helpers import rel_err

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-6, torch.bfloat16: 6e-3}      # one op deep: float rounding / one bfloat16 rounding


@pytest.fixture(scope="module")
def kernel_sets():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    return {dt: KernelSet(dt) for dt in DTYPES}


def dev(t, dtype=None):
    t = torch.as_tensor(t)
    return (t.to(dtype) if dtype is not None else t).cuda().contiguous()


def f64(t):
    return t.detach().cpu().to(torch.float64)


def rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


# --------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_rows(kernel_sets, dtype):
    ks = kernel_sets[dtype]
    table = dev(rand(37, 24, seed=1), dtype)
    ids = dev([5, 0, 36, 5, 17], torch.int32)
    out = torch.empty(5, 24, dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ks.embed_rows(ids, table, out, err)
    assert torch.equal(out.cpu(), table.float().cpu()[ids.cpu().long()]) and int(err) == 0
    ks.embed_rows(dev([3, 37], torch.int32), table, out[:2], err)       # an id outside the table: flagged, zeros
    assert int(err) == 1 and float(out[1].abs().sum()) == 0.0


# --------------------------------------------------------------------------- norm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, eps, w32", [(40, 1e-5, False), (2048, 1e-6, True), (1000, 1e-3, False), (13000, 1e-5, True)])
def test_add_rmsnorm(kernel_sets, dtype, d, eps, w32):
    ks = kernel_sets[dtype]
    T = 7
    x = dev(rand(T, d, seed=2, scale=3.0))
    delta = dev(rand(T, d, seed=3), dtype)
    w = dev(1.0 + rand(d, seed=4, scale=0.1), torch.float32 if w32 else torch.bfloat16)
    y = torch.empty(T, d, dtype=dtype, device="cuda")
    want_sum = f64(x) + f64(delta)
    want = plain.rms_norm(want_sum, f64(w), eps)
    xs = x.clone()
    ks.add_rmsnorm(xs, delta, None, w, y, eps)
    assert rel_err(y.cpu().float(), want) < TOL[dtype]
    assert rel_err(xs.cpu(), want_sum) < 2e-7                          # the residual sum is kept in 32-bit
    # no addend: x untouched
    xs = x.clone()
    ks.add_rmsnorm(xs, None, None, w, y, eps)
    assert torch.equal(xs, x) and rel_err(y.cpu().float(), plain.rms_norm(f64(x), f64(w), eps)) < TOL[dtype]
    # chosen rows: x untouched, rows of y follow `rows`
    rows = dev([6, 0, 3], torch.int32)
    y3 = torch.empty(3, d, dtype=dtype, device="cuda")
    xs = x.clone()
    ks.add_rmsnorm(xs, delta, rows, w, y3, eps)
    assert torch.equal(xs, x) and rel_err(y3.cpu().float(), want[[6, 0, 3]]) < TOL[dtype]
    # partial sums in float32
    parts = dev(rand(3, T, d, seed=5))
    xs = x.clone()
    ks.add_rmsnorm(xs, parts, None, w, y, eps)
    want_p = f64(x) + f64(parts).sum(0)
    assert rel_err(xs.cpu(), want_p) < 5e-7 and rel_err(y.cpu().float(), plain.rms_norm(want_p, f64(w), eps)) < TOL[dtype]
    ks.add_rmsnorm(x.clone(), parts, rows, w, y3, eps)
    assert rel_err(y3.cpu().float(), plain.rms_norm(want_p, f64(w), eps)[[6, 0, 3]]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, w32", [(128, False), (896, True), (2048, False), (2176, True), (4096, False), (2000, False)])
def test_add_rmsnorm_many_rows(kernel_sets, dtype, d, w32):
    """The many rows of a prompt step (512 or more: small blocks with four accesses in flight per
    thread), with and without an addend, at widths that are and are not multiples of 128."""
    ks = kernel_sets[dtype]
    T, eps = 517, 1e-5
    x = dev(rand(T, d, seed=2, scale=3.0))
    delta = dev(rand(T, d, seed=3), dtype)
    w = dev(1.0 + rand(d, seed=4, scale=0.1), torch.float32 if w32 else torch.bfloat16)
    y = torch.full((T, d), float("nan"), dtype=dtype, device="cuda")
    want_sum = f64(x) + f64(delta)
    xs = x.clone()
    ks.add_rmsnorm(xs, delta, None, w, y, eps)
    assert rel_err(y.cpu().float(), plain.rms_norm(want_sum, f64(w), eps)) < TOL[dtype]
    assert rel_err(xs.cpu(), want_sum) < 2e-7
    xs = x.clone()
    y.fill_(float("nan"))
    ks.add_rmsnorm(xs, None, None, w, y, eps)
    assert torch.equal(xs, x) and rel_err(y.cpu().float(), plain.rms_norm(f64(x), f64(w), eps)) < TOL[dtype]


# --------------------------------------------------------------------------- matrix products
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M, N, K", [(1, 33, 19), (3, 100, 72), (8, 64, 1000), (9, 130, 65), (70, 257, 136), (200, 96, 520),
                                     # K in multiples of 4: the 16-byte kernels (a block per four columns up to 8
                                     # rows, 64- and 128-row register tiles beyond), ragged edges everywhere
                                     (1, 35, 20), (2, 1003, 2048), (4, 6, 4100), (7, 515, 264), (9, 130, 64), (64, 300, 2048),
                                     (65, 129, 136), (300, 515, 264), (130, 1000, 24)])
def test_gemm_nt_generic(kernel_sets, dtype, M, N, K):
    ks = kernel_sets[dtype]
    a, w = dev(rand(M, K, seed=6), dtype), dev(rand(N, K, seed=7, scale=0.1), dtype)
    want = plain.linear(f64(a), f64(w))
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    ks.gemm_nt(a, w, out)
    # float accumulation, float output: one ascending chain of K fused multiply-adds per output, whose
    # rounding error grows like sqrt(K) (2e-6 holds up to about a thousand terms)
    tol32 = 2e-6 * max(1.0, math.sqrt(K / 1024))
    if dtype == torch.float32:
        assert rel_err(out.cpu().float(), want) < tol32
    else:
        assert rel_err(out.cpu().float(), want) < TOL[dtype]
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    ks.gemm_nt(a, w, out32)
    assert rel_err(out32.cpu(), want) < tol32
    if K % 4 == 0:
        for split in (2, 5):                                            # K cut into parts, partial sums for the reader
            parts = torch.full((split, M, N), float("nan"), dtype=torch.float32, device="cuda")
            ks.gemm_nt(a, w, parts)
            assert rel_err(parts.sum(0).cpu(), want) < tol32


def test_gemm_nt_generic_split_choice():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    assert KernelSet.gemm_nt_split(8, 2048, 8192, 148) == 1             # few rows: no cut
    assert KernelSet.gemm_nt_split(64, 2048, 8192, 148) == 16           # 16 tiles on 148 SMs: cut K
    assert KernelSet.gemm_nt_split(64, 2048, 2048, 148) == 8
    assert KernelSet.gemm_nt_split(2048, 8192, 2048, 148) == 1          # enough tiles
    assert KernelSet.gemm_nt_split(20, 96, 200, 148) == 1               # too shallow to cut


def test_attention_split_choice(kernel_sets):
    """About as many blocks as are resident at once (seven per SM for the one-head kernel, two or four
    for the grouped-query one), a tenth more at most, never more splits than pages, none without a page."""
    dk = kernel_sets[torch.bfloat16].decode
    one_head = {b: dk.attention_splits(b, 32, 32, 64, 64, 148) for b in (3, 4, 6, 8, 12, 16, 32, 64)}
    assert one_head == {3: 11, 4: 8, 6: 6, 8: 4, 12: 3, 16: 2, 32: 1, 64: 1}
    for b, n in one_head.items():
        assert n * 32 * b <= 1.12 * 7 * 148 or n == 1
    assert dk.attention_splits(8, 32, 32, 64, 3, 148) == 3                 # never more than pages
    assert dk.attention_splits(4, 32, 32, 64, 64, 148) * -(-64 // 8) == 64  # 9 were wanted: the ninth would be empty
    assert dk.attention_splits(8, 32, 8, 128, 64, 148) == 4                # grouped queries, width 128: two blocks per SM
    assert dk.attention_splits(8, 32, 8, 64, 64, 148) == 8                 # width 64: four (9 wanted, 8 pages each: 8)
    assert dk.attention_splits(8, 32, 8, 128, 8, 148) == 2                 # at least four pages each
    assert dk.attention_splits(1, 32, 32, 64, 64, 148) == 16               # a single sequence: the tensor-core kernel
    assert dk.attention_splits(500, 32, 32, 64, 64, 148) == 1


@pytest.mark.parametrize("M, N, K", [(1, 64, 64), (3, 100, 72), (8, 176, 64), (9, 1003, 144), (16, 2048, 2048),
                                     (33, 96, 200), (64, 640, 4096), (5, 49152 + 16, 256), (12, 16384, 128)])
def test_gemm_small_m(kernel_sets, M, N, K):
    """(The last two sizes, and the K splits of (16, 2048, 2048), have more blocks than are resident at once:
    they take the forms of the kernel with more blocks to an SM.)"""
    dk = kernel_sets[torch.bfloat16].decode
    a, w = dev(rand(M, K, seed=8), torch.bfloat16), dev(rand(N, K, seed=9, scale=0.05), torch.bfloat16)
    assert dk.takes(a, w)
    want = plain.linear(f64(a), f64(w))
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    dk.gemm_small_m(a, w, out)
    assert rel_err(out.cpu().float(), want) < TOL[torch.bfloat16]
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    dk.gemm_small_m(a, w, out32)
    assert rel_err(out32.cpu(), want) < 3e-6
    for split in (2, 5):
        if K // split >= 8:
            parts = torch.full((split, M, N), float("nan"), dtype=torch.float32, device="cuda")
            dk.gemm_small_m(a, w, parts)
            assert rel_err(parts.sum(0).cpu(), want) < 3e-6
    if N % 16 == 0:
        F = N // 2
        tiled = w.view(2, F // 8, 8, K).permute(1, 0, 2, 3).reshape(N, K).contiguous()
        h = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
        dk.gemm_small_m(a, tiled, h, swiglu=True)
        assert rel_err(h.cpu().float(), plain.swiglu(want[:, :F], want[:, F:])) < TOL[torch.bfloat16]


@pytest.mark.parametrize("M, N, K, eps", [(1, 64, 64, 1e-5), (3, 112, 72, 1e-6), (8, 2048, 8192, 1e-5), (13, 1008, 144, 1e-3),
                                          (16, 2048, 2048, 1e-5), (5, 4096, 4104, 1e-5)])
def test_gemm_small_m_takes_over_the_halves_of_a_norm(kernel_sets, M, N, K, eps):
    """A norm folded into the products around it: the product before it adds to the residual stream,
    writes (residual * weight) in bfloat16 and leaves each tile's sums of squares; the product behind
    it scales its output rows by rsqrt(sum / width + eps). Both against the plain formulas, and the
    pair against the plain norm between two plain products."""
    dk = kernel_sets[torch.bfloat16].decode
    a, w = dev(rand(M, K, seed=8), torch.bfloat16), dev(rand(N, K, seed=9, scale=0.05), torch.bfloat16)
    resid0 = rand(M, N, seed=10, scale=2.0).float()
    norm_w = (1.0 + 0.1 * rand(N, seed=11)).float()
    y = plain.linear(f64(a), f64(w))
    # ---- the first half: residual += y, xb, sums of squares
    resid = dev(resid0, torch.float32)
    xb = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    sumsq = torch.full((-(-N // 16), M), float("nan"), dtype=torch.float32, device="cuda")
    dk.gemm_small_m(a, w, resid, fold=(dev(norm_w, torch.float32), xb, sumsq))
    want_resid = resid0.double() + y
    assert rel_err(resid.cpu(), want_resid) < 3e-6
    assert rel_err(xb.cpu().float(), want_resid * norm_w.double()) < TOL[torch.bfloat16]
    assert rel_err(sumsq.sum(0).cpu(), (want_resid ** 2).sum(1)) < 1e-5
    # ---- the second half: a product whose input rows are owed their scale
    w2 = dev(rand(48, N, seed=12, scale=0.05), torch.bfloat16)
    out = torch.empty(M, 48, dtype=torch.bfloat16, device="cuda")
    dk.gemm_small_m(xb, w2, out, owed=(sumsq, N, eps))
    scale = torch.rsqrt((resid.cpu().double() ** 2).mean(1) + eps)
    assert rel_err(out.cpu().float(), plain.linear(f64(xb), f64(w2)) * scale[:, None]) < TOL[torch.bfloat16]
    # ---- the pair is the plain norm between two plain products, up to where bfloat16 rounds
    normed = plain.rms_norm(want_resid, norm_w.double(), eps)
    assert rel_err(out.cpu().float(), plain.linear(normed, f64(w2))) < 2 * TOL[torch.bfloat16]
    # ---- the gated epilogue takes the scale too
    tiled = w2.view(2, 3, 8, N).permute(1, 0, 2, 3).reshape(48, N).contiguous()
    h = torch.empty(M, 24, dtype=torch.bfloat16, device="cuda")
    dk.gemm_small_m(xb, tiled, h, swiglu=True, owed=(sumsq, N, eps))
    full = plain.linear(f64(xb), f64(w2)) * scale[:, None]
    assert rel_err(h.cpu().float(), plain.swiglu(full[:, :24], full[:, 24:])) < TOL[torch.bfloat16]


@pytest.mark.parametrize("M, N, K, eps", [(130, 2048, 2048, 1e-5), (300, 1056, 520, 1e-6), (2048, 2048, 8192, 1e-5), (129, 160, 264, 1e-3),
                                          (700, 4096, 1024, 1e-5)])
def test_gemm_tc_takes_over_the_halves_of_a_norm(kernel_sets, M, N, K, eps):
    """The same two halves in the tensor-core products of a long prompt step: the residual sum,
    residual * weight and the sums of squares per 128 columns in the epilogue of one (staged through
    shared memory so that the float stream is read and written in whole rows); the row scale in the
    plain and the gated epilogue of the other, on the two-SM and the one-SM tiles."""
    tc = kernel_sets[torch.bfloat16].tensor_core
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    a, w = dev(rand(M, K, seed=8), torch.bfloat16), dev(rand(N, K, seed=9, scale=0.05), torch.bfloat16)
    resid0 = rand(M, N, seed=10, scale=2.0).float()
    norm_w = (1.0 + 0.1 * rand(N, seed=11)).float()
    y = plain.linear(f64(a), f64(w))
    resid = dev(resid0, torch.float32)
    xb = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    sumsq = torch.full((-(-N // 128), M), float("nan"), dtype=torch.float32, device="cuda")
    tc.gemm(a, w, resid, err, fold=(dev(norm_w, torch.float32), xb, sumsq))
    want_resid = resid0.double() + y
    assert int(err) == 0
    assert rel_err(resid.cpu(), want_resid) < 3e-5             # tensor-core accumulation over long K, as in the plain product
    assert rel_err(xb.cpu().float(), want_resid * norm_w.double()) < TOL[torch.bfloat16]
    assert rel_err(sumsq.sum(0).cpu(), (want_resid ** 2).sum(1)) < 6e-5
    # the second half: plain and gated epilogues (48 columns: the one-SM tile)
    w2 = dev(rand(48, N, seed=12, scale=0.05), torch.bfloat16)
    scale = torch.rsqrt((resid.cpu().double() ** 2).mean(1) + eps)
    full = plain.linear(f64(xb), f64(w2)) * scale[:, None]
    out = torch.empty(M, 48, dtype=torch.bfloat16, device="cuda")
    tc.gemm(xb, w2, out, err, owed=(sumsq, N, eps))
    assert rel_err(out.cpu().float(), full) < TOL[torch.bfloat16]
    assert rel_err(out.cpu().float(), plain.linear(plain.rms_norm(want_resid, norm_w.double(), eps), f64(w2))) < 2 * TOL[torch.bfloat16]
    tiled = w2.view(2, 3, 8, N).permute(1, 0, 2, 3).reshape(48, N).contiguous()
    h = torch.empty(M, 24, dtype=torch.bfloat16, device="cuda")
    tc.gemm(xb, tiled, h, err, swiglu=True, owed=(sumsq, N, eps))
    assert rel_err(h.cpu().float(), plain.swiglu(full[:, :24], full[:, 24:])) < TOL[torch.bfloat16]
    # a wide product (the two-SM tile): every column tile of a row takes the same scale
    w3 = dev(rand(520, N, seed=13, scale=0.05), torch.bfloat16)
    out3 = torch.empty(M, 520, dtype=torch.float32, device="cuda")
    tc.gemm(xb, w3, out3, err, owed=(sumsq, N, eps))
    assert rel_err(out3.cpu(), plain.linear(f64(xb), f64(w3)) * scale[:, None]) < 3e-5
    assert int(err) == 0


@pytest.mark.parametrize("M, N, K", [(128, 128, 64), (100, 200, 72), (130, 264, 520), (2048, 2048, 2048), (65, 1003 * 8, 136),
                                     (300, 96, 8192), (257, 384, 136), (2304, 6400, 192), (1100, 4104, 2176)])
def test_gemm_tensor_core(kernel_sets, M, N, K):
    """The tcgen05 GEMM: bfloat16 and float outputs, the SiLU-gate epilogue.
    More than 128 rows and columns go to the kernel that pairs two SMs on a 256 x 256 tile: sizes with
    a ragged last tile, with several tiles to a pair (both accumulators, both phases), and with few
    and many k-blocks to a tile (eight or four epilogue warps)."""
    tc = kernel_sets[torch.bfloat16].tensor_core
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    a, w = dev(rand(M, K, seed=14), torch.bfloat16), dev(rand(N, K, seed=15, scale=0.05), torch.bfloat16)
    assert tc.takes(a, w)
    want = plain.linear(f64(a), f64(w))
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    tc.gemm(a, w, out, err)
    assert rel_err(out.cpu().float(), want) < TOL[torch.bfloat16]
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    tc.gemm(a, w, out32, err)
    assert rel_err(out32.cpu(), want) < 3e-5              # tensor-core accumulation over long K
    if N % 16 == 0:
        F = N // 2
        tiled = w.view(2, F // 8, 8, K).permute(1, 0, 2, 3).reshape(N, K).contiguous()
        h = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
        tc.gemm(a, tiled, h, err, swiglu=True)
        assert rel_err(h.cpu().float(), plain.swiglu(want[:, :F], want[:, F:])) < TOL[torch.bfloat16]
    assert int(err) == 0


@pytest.mark.parametrize("M, N, K", [(1, 128, 64), (17, 200, 72), (33, 264, 520), (64, 2048, 2048), (100, 1003 * 8, 136),
                                     (128, 96, 8192), (16, 6144, 2048)])
def test_gemm_tensor_core_few_rows(kernel_sets, M, N, K):
    """The weight-stationary tcgen05 GEMM for at most 128 rows: bfloat16 and float outputs, float partial
    sums of a split K (with more splits than some sizes have k-blocks to give), the SiLU-gate epilogue."""
    tc = kernel_sets[torch.bfloat16].tensor_core
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    a, w = dev(rand(M, K, seed=24), torch.bfloat16), dev(rand(N, K, seed=25, scale=0.05), torch.bfloat16)
    want = plain.linear(f64(a), f64(w))
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    tc.gemm_skinny(a, w, out, err)
    assert rel_err(out.cpu().float(), want) < TOL[torch.bfloat16]
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    tc.gemm_skinny(a, w, out32, err)
    assert rel_err(out32.cpu(), want) < 3e-5
    nkb = -(-K // 64)
    for split in sorted({min(2, nkb), min(4, nkb), min(7, nkb)} - {1}):
        parts = torch.full((split, M, N), float("nan"), dtype=torch.float32, device="cuda")
        tc.gemm_skinny(a, w, parts, err)
        assert rel_err(parts.cpu().double().sum(0), want) < 3e-5
    if N % 16 == 0:
        F = N // 2
        tiled = w.view(2, F // 8, 8, K).permute(1, 0, 2, 3).reshape(N, K).contiguous()
        h = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
        tc.gemm_skinny(a, tiled, h, err, swiglu=True)
        assert rel_err(h.cpu().float(), plain.swiglu(want[:, :F], want[:, F:])) < TOL[torch.bfloat16]
    assert int(err) == 0


@pytest.mark.parametrize("H, G, hd, rot, pairing", [(4, 2, 64, 64, "half"), (3, 1, 128, 128, "half"), (5, 5, 64, 24, "interleaved"),
                                                    (2, 1, 128, 128, "interleaved")])
def test_gemm_qkv_with_rotation_and_cache_write(kernel_sets, H, G, hd, rot, pairing):
    """The q|k|v product whose epilogue rotates queries and keys and puts keys and values into the pages:
    against product, rounding, rotation in plain float64; rows of two sequences at scattered positions."""
    from scriptling_llm_lib_b200.parts.rotary import RotaryEncoding
    tc = kernel_sets[torch.bfloat16].tensor_core
    enc = RotaryEncoding(hd, rot, 54321.0, None, pairing)
    enc.prepare(1024, "cuda")
    table, r, inter = enc.rotation()
    lens, pos0 = [150, 70], [60, 300]
    T, K, N = sum(lens), 136, (H + 2 * G) * hd
    a, w = dev(rand(T, K, seed=41), torch.bfloat16), dev(rand(N, K, seed=42, scale=0.1), torch.bfloat16)
    raw = plain.linear(f64(a), f64(w)).to(torch.bfloat16).to(torch.float64)          # the product, stored in bfloat16
    inv = plain.rope_inv_freq(rot, 54321.0)
    tok_pos = torch.cat([torch.arange(p, p + n) for n, p in zip(lens, pos0)])
    tok_seq = torch.cat([torch.full((n,), b) for b, n in enumerate(lens)])
    q_want = plain.apply_rope(raw[:, :H * hd].view(T, H, hd), tok_pos, inv, pairing).reshape(T, H * hd)
    k_want = plain.apply_rope(raw[:, H * hd:(H + G) * hd].view(T, G, hd), tok_pos, inv, pairing)
    v_want = raw[:, (H + G) * hd:].view(T, G, hd)
    nan = lambda n: torch.full((n, G, hd), float("nan"))
    kp, vp, bt = paged([nan(p + n) for n, p in zip(lens, pos0)], [nan(p + n) for n, p in zip(lens, pos0)],
                       [p + n for n, p in zip(lens, pos0)], dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    qkv = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    tc.gemm_qkv_rope(a, w, qkv, err, dev(tok_pos, torch.int32), dev(tok_seq, torch.int32), bt, table, kp, vp, H, G, hd, r, inter)
    assert int(err) == 0
    assert rel_err(qkv.cpu().float(), q_want) < TOL[torch.bfloat16]
    row = 0
    for b, (n, p) in enumerate(zip(lens, pos0)):
        for t in (0, 1, n // 2, n - 1):
            pos = p + t
            pg = int(bt[b, pos // PAGE])
            assert rel_err(f64(kp[pg, :, pos % PAGE]), k_want[row + t]) < TOL[torch.bfloat16]
            assert rel_err(f64(vp[pg, :, pos % PAGE]), v_want[row + t]) < 1e-6
        assert torch.isnan(kp[int(bt[b, 0]), :, 0].float()).all() if p > 0 else True     # places before the step untouched
        row += n


def test_gemm_small_m_refuses_what_it_cannot_take(kernel_sets):
    from scriptling_llm_lib_b200.csrc.bindings import KernelError
    dk = kernel_sets[torch.bfloat16].decode
    a, w = dev(rand(4, 36), torch.bfloat16), dev(rand(16, 36), torch.bfloat16)     # K no multiple of 8
    assert not dk.takes(a, w)
    with pytest.raises(KernelError):
        dk.gemm_small_m(a, w, torch.empty(4, 16, dtype=torch.bfloat16, device="cuda"))
    assert not dk.takes(dev(rand(65, 64), torch.bfloat16), dev(rand(16, 64), torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("F, tiled", [(176, True), (50, False), (8, True)])
def test_swiglu(kernel_sets, dtype, F, tiled):
    ks = kernel_sets[dtype]
    T = 5
    g, u = rand(T, F, seed=10, scale=2.0), rand(T, F, seed=11)
    gu = torch.cat([g, u], dim=1)
    if tiled:
        gu = torch.stack([g.view(T, F // 8, 8), u.view(T, F // 8, 8)], dim=2).reshape(T, 2 * F)
    gu = dev(gu, dtype)
    h = torch.empty(T, F, dtype=dtype, device="cuda")
    ks.swiglu(gu, h, tiled=tiled)
    gq, uq = f64(dev(g, dtype)), f64(dev(u, dtype))
    assert rel_err(h.cpu().float(), plain.swiglu(gq, uq)) < TOL[dtype]


# --------------------------------------------------------------------------- paged cache helpers
PAGE = 64


def paged(k, v, lengths, n_extra=3, seed=0, dtype=torch.float32):
    """Scatter per-sequence dense K/V [len, G, hd] into pages handed out in a scrambled order.
    Unused cache memory is NaN: a kernel that reads past a sequence's length shows it."""
    G, hd = k[0].shape[1], k[0].shape[2]
    need = [-(-n // PAGE) for n in lengths]
    total = sum(need) + n_extra
    order = np.random.default_rng(seed).permutation(total).tolist()
    kp = torch.full((total, G, PAGE, hd), float("nan"), dtype=torch.float32)
    vp = torch.full((total, G, PAGE, hd), float("nan"), dtype=torch.float32)
    bt = torch.full((len(lengths), max(need)), -1, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for i in range(need[b]):
            pg = order.pop()
            bt[b, i] = pg
            m = min(PAGE, n - i * PAGE)
            kp[pg, :, :m] = k[b][i * PAGE:i * PAGE + m].permute(1, 0, 2)
            vp[pg, :, :m] = v[b][i * PAGE:i * PAGE + m].permute(1, 0, 2)
    return dev(kp, dtype), dev(vp, dtype), dev(bt)


# --------------------------------------------------------------------------- rotary + cache write
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, hd, rot, pairing", [(4, 2, 16, 16, "interleaved"), (3, 1, 32, 16, "half"),
                                                    (6, 3, 48, 48, "half"), (2, 2, 80, 40, "interleaved"),
                                                    (2, 1, 16, 8, "half"), (5, 5, 32, 12, "interleaved")])
def test_rope_kv_write(kernel_sets, dtype, H, G, hd, rot, pairing):
    from scriptling_llm_lib_b200.parts.rotary import RotaryEncoding
    ks = kernel_sets[dtype]
    enc = RotaryEncoding(hd, rot, 12345.0, None, pairing)
    enc.prepare(300, "cuda")
    lens, pos0 = [5, 70, 1], [0, 60, 199]                               # new tokens and tokens already cached
    T = sum(lens)
    qkv = dev(rand(T, (H + 2 * G) * hd, seed=12), dtype)
    tok_seq = np.repeat(np.arange(3), lens)
    tok_pos = np.concatenate([np.arange(p, p + n) for p, n in zip(pos0, lens)])
    n_pages = 9
    kp = torch.zeros(n_pages, G, PAGE, hd, dtype=dtype, device="cuda")
    vp = torch.zeros_like(kp)
    bt = dev([[7, -1, -1, -1], [2, 5, 0, -1], [1, 3, 8, 4]], torch.int32)
    orig = f64(qkv).clone()
    ks.rope_kv_write(qkv, dev(tok_pos, torch.int32), dev(tok_seq, torch.int32), bt, enc.cos_sin, kp, vp, H, G, hd, rot,
                     pairing == "interleaved")
    inv = plain.rope_inv_freq(rot, 12345.0)
    pos_t = torch.as_tensor(tok_pos)
    q_want = plain.apply_rope(orig[:, :H * hd].view(T, H, hd), pos_t, inv, pairing)
    k_want = plain.apply_rope(orig[:, H * hd:(H + G) * hd].view(T, G, hd), pos_t, inv, pairing)
    v_want = orig[:, (H + G) * hd:].view(T, G, hd)
    assert rel_err(f64(qkv)[:, :H * hd], q_want.reshape(T, -1)) < TOL[dtype]
    assert torch.equal(f64(qkv)[:, H * hd:], orig[:, H * hd:])          # k and v columns of the buffer are not rewritten
    for t in range(T):
        pg = int(bt[tok_seq[t], tok_pos[t] // PAGE])
        assert rel_err(f64(kp[pg, :, tok_pos[t] % PAGE]), k_want[t]) < TOL[dtype]
        assert torch.equal(f64(vp[pg, :, tok_pos[t] % PAGE]), v_want[t])
    assert float(kp[6].abs().sum()) == 0.0                               # a page nobody owns stays untouched
    # queries only (a layer that reads another layer's cache)
    q2 = dev(rand(T, H * hd, seed=13), dtype)
    o2 = f64(q2).clone()
    ks.rope_kv_write(q2, dev(tok_pos, torch.int32), dev(tok_seq, torch.int32), bt, enc.cos_sin, None, None, H, 0, hd, rot,
                     pairing == "interleaved")
    assert rel_err(f64(q2), plain.apply_rope(o2.view(T, H, hd), pos_t, inv, pairing).reshape(T, -1)) < TOL[dtype]


# --------------------------------------------------------------------------- attention
def attention_case(H, G, hd, lens, pos0, seed):
    """Per sequence: all keys/values (cached + new) and the new queries."""
    ks_, vs_, qs_ = [], [], []
    for b, (n, p) in enumerate(zip(lens, pos0)):
        ks_.append(rand(p + n, G, hd, seed=seed + 3 * b))
        vs_.append(rand(p + n, G, hd, seed=seed + 3 * b + 1))
        qs_.append(rand(n, H, hd, seed=seed + 3 * b + 2, scale=2.0))
    return qs_, ks_, vs_


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, hd, window", [(4, 2, 16, None), (3, 1, 32, None), (6, 3, 48, 24), (2, 2, 80, None),
                                              (8, 2, 64, 100), (2, 1, 128, None)])
def test_attn_paged(kernel_sets, dtype, H, G, hd, window):
    ks = kernel_sets[dtype]
    lens, pos0 = [37, 1, 130, 16], [0, 250, 70, 64]
    qs, kk, vv = attention_case(H, G, hd, lens, pos0, 20)
    rnd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.bfloat16().float())
    qs, kk, vv = [rnd(t) for t in qs], [rnd(t) for t in kk], [rnd(t) for t in vv]
    kp, vp, bt = paged(kk, vv, [p + n for p, n in zip(pos0, lens)], dtype=dtype)
    T = sum(lens)
    q = dev(torch.cat([t.reshape(t.shape[0], -1) for t in qs]), dtype)
    out = torch.empty(T, H * hd, dtype=dtype, device="cuda")
    seq_start = dev(np.concatenate([[0], np.cumsum(lens)]), torch.int32)
    ks.attn_paged(q, out, seq_start, dev(pos0, torch.int32), bt, kp, vp, len(lens), max(lens), H, G, hd, window,
                  1.0 / math.sqrt(hd))
    want = torch.cat([plain.attention(f64(qs[b]), f64(kk[b]), f64(vv[b]), torch.arange(pos0[b], pos0[b] + lens[b]),
                                      torch.arange(pos0[b] + lens[b]), window).reshape(lens[b], -1) for b in range(len(lens))])
    # a score is a chain of head_dim float multiply-adds: its rounding, and with it the probabilities', grows
    # like sqrt(head_dim) (2e-6 holds up to a width of 64)
    assert rel_err(out.cpu().float(), want) < TOL[dtype] * (max(1.0, math.sqrt(hd / 64)) if dtype == torch.float32 else 1.0)
    # few new rows per sequence: the one-query-at-a-time form of the kernel
    lens2 = [3, 1, 2, 4]
    qs2 = [t[:n] for t, n in zip(qs, lens2)]
    kp2, vp2, bt2 = paged([k[:p + n] for k, p, n in zip(kk, pos0, lens2)], [v[:p + n] for v, p, n in zip(vv, pos0, lens2)],
                          [p + n for p, n in zip(pos0, lens2)], dtype=dtype, seed=5)
    q2 = dev(torch.cat([t.reshape(t.shape[0], -1) for t in qs2]), dtype)
    out2 = torch.empty(sum(lens2), H * hd, dtype=dtype, device="cuda")
    ks.attn_paged(q2, out2, dev(np.concatenate([[0], np.cumsum(lens2)]), torch.int32), dev(pos0, torch.int32), bt2, kp2, vp2,
                  len(lens2), max(lens2), H, G, hd, window, 1.0 / math.sqrt(hd))
    want2 = torch.cat([plain.attention(f64(qs2[b]), f64(kk[b][:pos0[b] + lens2[b]]), f64(vv[b][:pos0[b] + lens2[b]]),
                                       torch.arange(pos0[b], pos0[b] + lens2[b]), torch.arange(pos0[b] + lens2[b]),
                                       window).reshape(lens2[b], -1) for b in range(len(lens2))])
    assert rel_err(out2.cpu().float(), want2) < TOL[dtype] * (max(1.0, math.sqrt(hd / 64)) if dtype == torch.float32 else 1.0)


@pytest.mark.parametrize("lens, pos0", [([37, 1, 130, 64, 200, 128], [0, 250, 70, 64, 0, 300]), ([37], [0]), ([1], [700]),
                                        ([2, 3], [63, 64])])
@pytest.mark.parametrize("H, G, window", [(4, 2, None), (3, 1, None), (6, 3, 24), (8, 2, 100), (5, 5, 1), (2, 2, 64)])
@pytest.mark.parametrize("hd", [64, 128])
def test_attn_prefill_tcgen05(kernel_sets, hd, H, G, window, lens, pos0):
    """The tcgen05 attention (S and P V in tensor memory, TMA-fed pages), heads of 64 and of 128: prompts
    that start at a non-empty cache, a one-token prompt, tiles of exactly 64 and 128 queries, windows;
    unused cache memory is NaN, which the kernel must never let through."""
    fa = kernel_sets[torch.bfloat16].prefill_attention_tc
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    qs, kk, vv = attention_case(H, G, hd, lens, pos0, 30)
    rnd = lambda t: t.bfloat16().float()
    qs, kk, vv = [rnd(t) for t in qs], [rnd(t) for t in kk], [rnd(t) for t in vv]
    kp, vp, bt = paged(kk, vv, [p + n for p, n in zip(pos0, lens)], dtype=torch.bfloat16)
    T = sum(lens)
    q = dev(torch.cat([t.reshape(t.shape[0], -1) for t in qs]), torch.bfloat16)
    out = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    seq_start = dev(np.concatenate([[0], np.cumsum(lens)]), torch.int32)
    fa.attn(q, out, seq_start, dev(pos0, torch.int32), bt, kp, vp, len(lens), max(lens), H, G, hd, window, 1.0 / math.sqrt(hd), err)
    want = torch.cat([plain.attention(f64(qs[b]), f64(kk[b]), f64(vv[b]), torch.arange(pos0[b], pos0[b] + lens[b]),
                                      torch.arange(pos0[b] + lens[b]), window).reshape(lens[b], -1) for b in range(len(lens))])
    assert int(err) == 0
    assert rel_err(out.cpu().float(), want) < 1.2e-2          # probabilities are rounded to bfloat16 before P V


@pytest.mark.parametrize("hd, H, G, window", [(64, 40, 40, None), (64, 24, 6, 700), (128, 24, 6, None), (128, 15, 15, None), (128, 9, 3, 900)])
def test_attn_prefill_tcgen05_long_prompts_many_items(kernel_sets, hd, H, G, window):
    """Prompts of a few thousand tokens and more work items than resident blocks: every block walks several
    items, the key/value ring wraps many times, and at head width 128 both ways of pairing query tiles are
    taken (two heads of a group; two consecutive tiles of one head where the group is odd). Sampled rows
    (the first, the last, the edges of the 64- and 128-row tiles) against the plain implementation, every
    row against the generic kernel."""
    ks = kernel_sets[torch.bfloat16]
    fa = ks.prefill_attention_tc
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    lens, pos0 = [2100, 1500], [0, 64]
    g = torch.Generator().manual_seed(hd + H)
    rnd = lambda t: t.bfloat16().float()
    kk = [rnd(torch.randn(p + n, G, hd, generator=g)) for p, n in zip(pos0, lens)]
    vv = [rnd(torch.randn(p + n, G, hd, generator=g)) for p, n in zip(pos0, lens)]
    qs = [rnd(torch.randn(n, H, hd, generator=g)) for n in lens]
    kp, vp, bt = paged(kk, vv, [p + n for p, n in zip(pos0, lens)], dtype=torch.bfloat16)
    T = sum(lens)
    q = dev(torch.cat([t.reshape(t.shape[0], -1) for t in qs]), torch.bfloat16)
    seq_start = dev(np.concatenate([[0], np.cumsum(lens)]), torch.int32)
    out = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    fa.attn(q, out, seq_start, dev(pos0, torch.int32), bt, kp, vp, len(lens), max(lens), H, G, hd, window, 1.0 / math.sqrt(hd), err)
    assert int(err) == 0
    got = out.cpu().float()
    assert torch.isfinite(got).all()
    row0 = 0
    for b, n in enumerate(lens):
        rows = sorted({0, 1, 62, 63, 64, 65, 126, 127, 128, 129, 191, 192, 255, 256, 1023, 1024, n - 129, n - 128, n - 65, n - 64, n - 2, n - 1}
                      | {int(x) for x in torch.randint(0, n, (24,), generator=g)})
        idx = torch.tensor(rows)
        want = plain.attention(f64(qs[b][idx]), f64(kk[b]), f64(vv[b]), pos0[b] + idx, torch.arange(pos0[b] + n), window).reshape(len(rows), -1)
        assert rel_err(got[row0 + idx], want) < 1.2e-2, (b, hd, H, G)
        row0 += n
    other = torch.empty_like(out)
    ks.attn_paged(q, other, seq_start, dev(pos0, torch.int32), bt, kp, vp, len(lens), max(lens), H, G, hd, window, 1.0 / math.sqrt(hd))
    assert rel_err(got, other.cpu().float()) < 1.5e-2


@pytest.mark.parametrize("hd, H, G", [(64, 32, 32), (128, 32, 8), (128, 5, 5)])
def test_attn_prefill_tcgen05_same_bits_every_launch(kernel_sets, hd, H, G):
    """The hand-overs between the kernel's roles must not let timing into the result: twenty launches on
    the same input, unequal prompts, give the same bits (a buffer reused a phase too early shows here)."""
    fa = kernel_sets[torch.bfloat16].prefill_attention_tc
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    lens = [1943, 560, 700, 65, 1, 1024]
    g = torch.Generator().manual_seed(hd + H)
    kk = [torch.randn(n, G, hd, generator=g) for n in lens]
    vv = [torch.randn(n, G, hd, generator=g) for n in lens]
    kp, vp, bt = paged(kk, vv, lens, dtype=torch.bfloat16)
    T = sum(lens)
    q = dev(torch.randn(T, H * hd, generator=g), torch.bfloat16)
    seq_start = dev(np.concatenate([[0], np.cumsum(lens)]), torch.int32)
    pos0 = dev([0] * len(lens), torch.int32)
    first = None
    for _ in range(20):
        out = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        fa.attn(q, out, seq_start, pos0, bt, kp, vp, len(lens), max(lens), H, G, hd, None, 1.0 / math.sqrt(hd), err)
        if first is None:
            first = out
            assert torch.isfinite(first.float()).all()
        else:
            assert torch.equal(out, first)
    assert int(err) == 0


@pytest.mark.parametrize("H, G, hd, window", [(4, 2, 16, None), (3, 1, 32, None), (32, 32, 64, None), (8, 2, 128, 300),
                                              (4, 1, 64, 65), (2, 2, 256, None),
                                              # two or more query heads per key/value head at widths 64 and 128: the
                                              # tensor-core variant; 12 and 40 heads per group use its upper rows and loop
                                              (32, 8, 64, None), (9, 3, 64, 100), (6, 3, 128, None), (24, 2, 64, 17),
                                              (40, 1, 128, 500),
                                              # one head per group, few (sequence, head) pairs: the same variant
                                              (4, 4, 64, None), (8, 8, 128, 70)])
@pytest.mark.parametrize("n_split", [1, 3, 16, 40, 70])      # 70: more than the merging block weighs in one pass
def test_attn_decode(kernel_sets, H, G, hd, window, n_split):
    dk = kernel_sets[torch.bfloat16].decode
    lens, pos0 = [1, 1, 1, 1, 1], [0, 63, 64, 700, 257]
    qs, kk, vv = attention_case(H, G, hd, lens, pos0, 40)
    rnd = lambda t: t.bfloat16().float()
    qs, kk, vv = [rnd(t) for t in qs], [rnd(t) for t in kk], [rnd(t) for t in vv]
    kp, vp, bt = paged(kk, vv, [p + 1 for p in pos0], dtype=torch.bfloat16)
    q = dev(torch.cat([t.reshape(1, -1) for t in qs]), torch.bfloat16)
    B = len(lens)
    out = torch.empty(B, H * hd, dtype=torch.bfloat16, device="cuda")
    scratch = torch.full((B * H * n_split * (hd + 2),), float("nan"), dtype=torch.float32, device="cuda")
    dk.attn_decode(q, out, dev(pos0, torch.int32), bt, kp, vp, scratch, B, H, G, hd, window, 1.0 / math.sqrt(hd), n_split)
    want = torch.cat([plain.attention(f64(qs[b]), f64(kk[b]), f64(vv[b]), torch.tensor([pos0[b]]),
                                      torch.arange(pos0[b] + 1), window).reshape(1, -1) for b in range(B)])
    assert rel_err(out.cpu().float(), want) < TOL[torch.bfloat16]
    # one kernel: the last split to finish merges; twice, the tickets must come back to zero
    tickets = torch.zeros(B * G, dtype=torch.int32, device="cuda")
    for _ in range(2):
        out.fill_(float("nan"))
        scratch.fill_(float("nan"))
        dk.attn_decode(q, out, dev(pos0, torch.int32), bt, kp, vp, scratch, B, H, G, hd, window, 1.0 / math.sqrt(hd), n_split,
                       tickets=tickets)
        assert rel_err(out.cpu().float(), want) < TOL[torch.bfloat16]
        assert int(tickets.abs().sum()) == 0


@pytest.mark.parametrize("H, G, hd, rot, pairing, window", [(4, 2, 16, 16, "half", None), (3, 1, 32, 16, "interleaved", None),
                                                            (32, 32, 64, 64, "half", None), (8, 2, 128, 64, "half", 300),
                                                            (4, 4, 64, 8, "interleaved", 65),
                                                            (9, 3, 64, 64, "half", 70), (12, 1, 64, 32, "interleaved", None),
                                                            (32, 8, 128, 128, "half", None)])
@pytest.mark.parametrize("n_split", [1, 5])
def test_attn_decode_with_rotation_and_cache_write_fused(kernel_sets, H, G, hd, rot, pairing, window, n_split):
    """One kernel does what rope_kv_write + attn_decode do: rotate q, rotate and store the new key,
    store the new value, attend. Checked against the plain functions, and the cache afterwards."""
    from scriptling_llm_lib_b200.parts.rotary import RotaryEncoding
    dk = kernel_sets[torch.bfloat16].decode
    enc = RotaryEncoding(hd, rot, 54321.0, None, pairing)
    enc.prepare(1024, "cuda")
    assert dk.rotation_fusable(rot, pairing == "interleaved")
    pos0 = [0, 63, 64, 700, 257]
    B = len(pos0)
    rnd = lambda t: t.bfloat16().float()
    old_k = [rnd(rand(p, G, hd, seed=90 + b)) for b, p in enumerate(pos0)]           # cached (already rotated) keys
    old_v = [rnd(rand(p, G, hd, seed=95 + b)) for b, p in enumerate(pos0)]
    raw = rnd(rand(B, (H + 2 * G) * hd, seed=99, scale=1.5))                         # this step's unrotated q | k | v
    inv = plain.rope_inv_freq(rot, 54321.0)
    q_rot, k_new, v_new = [], [], []
    for b, p in enumerate(pos0):
        pos = torch.tensor([p])
        q_rot.append(rnd(plain.apply_rope(f64(raw[b:b + 1, :H * hd]).view(1, H, hd), pos, inv, pairing).float()))
        k_new.append(rnd(plain.apply_rope(f64(raw[b:b + 1, H * hd:(H + G) * hd]).view(1, G, hd), pos, inv, pairing).float()))
        v_new.append(raw[b:b + 1, (H + G) * hd:].view(1, G, hd))
    want = torch.cat([plain.attention(f64(q_rot[b]), f64(torch.cat([old_k[b], k_new[b]])), f64(torch.cat([old_v[b], v_new[b]])),
                                      torch.tensor([pos0[b]]), torch.arange(pos0[b] + 1), window).reshape(1, -1) for b in range(B)])
    # pages sized for pos0 + 1 keys; the new key's place holds NaN until the kernel writes it
    nan_row = torch.full((1, G, hd), float("nan"))
    kp, vp, bt = paged([torch.cat([old_k[b], nan_row]) for b in range(B)], [torch.cat([old_v[b], nan_row]) for b in range(B)],
                       [p + 1 for p in pos0], dtype=torch.bfloat16)
    out = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    scratch = torch.full((B * H * n_split * (hd + 2),), float("nan"), dtype=torch.float32, device="cuda")
    tickets = torch.zeros(B * G, dtype=torch.int32, device="cuda")
    dk.attn_decode_rope(dev(raw, torch.bfloat16), out, dev(pos0, torch.int32), bt, kp, vp, scratch, tickets, enc.cos_sin, rot,
                        pairing == "interleaved", True, B, H, G, hd, window, 1.0 / math.sqrt(hd), n_split)
    assert rel_err(out.cpu().float(), want) < TOL[torch.bfloat16]
    assert int(tickets.abs().sum()) == 0
    for b, p in enumerate(pos0):
        pg = int(bt[b, p // PAGE])
        assert rel_err(f64(kp[pg, :, p % PAGE]), f64(k_new[b][0])) < TOL[torch.bfloat16]
        assert torch.equal(f64(vp[pg, :, p % PAGE]), f64(v_new[b][0]))
    # a layer that reads another layer's cache: queries only, the key at the query's position is read, not written
    out2 = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    dk.attn_decode_rope(dev(raw[:, :H * hd], torch.bfloat16), out2, dev(pos0, torch.int32), bt, kp, vp, scratch, tickets,
                        enc.cos_sin, rot, pairing == "interleaved", False, B, H, G, hd, window, 1.0 / math.sqrt(hd), n_split)
    assert rel_err(out2.cpu().float(), want) < TOL[torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, hd, window", [(4, 2, 16, None), (3, 1, 32, 40), (6, 3, 48, None), (32, 32, 64, None),
                                              (2, 2, 80, 100), (8, 2, 128, 300), (2, 1, 256, None), (2, 2, 320, 65)])
@pytest.mark.parametrize("n_split", [1, 3, 16])
def test_attn_decode_split_generic(kernel_sets, dtype, H, G, hd, window, n_split):
    """The decode attention of the generic path (all of the 32-bit decode step): head widths in
    steps of 4 elements up to 512, any grouping, windows, one or many splits (also more splits than
    a short sequence has pages)."""
    ks = kernel_sets[dtype]
    pos0 = [0, 63, 64, 700, 257]
    B = len(pos0)
    qs, kk, vv = attention_case(H, G, hd, [1] * B, pos0, 44)
    rnd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.bfloat16().float())
    qs, kk, vv = [rnd(t) for t in qs], [rnd(t) for t in kk], [rnd(t) for t in vv]
    kp, vp, bt = paged(kk, vv, [p + 1 for p in pos0], dtype=dtype)
    q = dev(torch.cat([t.reshape(1, -1) for t in qs]), dtype)
    assert ks.attn_decode_split_takes(hd, q.stride(0))
    out = torch.full((B, H * hd), float("nan"), dtype=dtype, device="cuda")
    part = torch.full((B * H * n_split * (hd + 2),), float("nan"), dtype=torch.float32, device="cuda") if n_split > 1 else None
    ks.attn_decode_split(q, out, dev(pos0, torch.int32), bt, kp, vp, part, B, H, G, hd, window, 1.0 / math.sqrt(hd), n_split)
    want = torch.cat([plain.attention(f64(qs[b]), f64(kk[b]), f64(vv[b]), torch.tensor([pos0[b]]),
                                      torch.arange(pos0[b] + 1), window).reshape(1, -1) for b in range(B)])
    assert rel_err(out.cpu().float(), want) < TOL[dtype]


FAR_CASES = [(3, None, True), (517, None, True), (899 - 199, 200, True), (899 - 200, 200, False),
             (640, 260, True), (639, 260, False)]     # the last two: the window's edge (key 640) on a page and tile boundary


def far_key_case(H, G, hd, n, far, dtype, n_new=1):
    """`n` keys; the queries at the last `n_new` positions all point at key `far`, whose score towers
    over the others: the output must be that key's value if and only if the key is seen."""
    k = rand(n, G, hd, seed=60, scale=0.1)
    v = rand(n, G, hd, seed=61)
    base = rand(G, hd, seed=62, scale=0.1)                               # one query direction per key/value head
    nrep = H // G
    q = base.repeat_interleave(nrep, dim=0)[None].repeat(n_new, 1, 1).contiguous()    # every head of a group, every row
    k[far] = base * (2260.0 / math.sqrt(hd))                            # score about 22 above the others
    rnd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.bfloat16().float())
    return rnd(q), rnd(k), rnd(v)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_and_respects_the_windows_edge(kernel_sets, dtype):
    """Random keys would hide a key read from the wrong place: one key among 900 gets a score far
    above the rest, so the output must be that key's value; with a window, the key at distance
    window-1 is seen and the key at distance window is not. Through the generic kernels of both
    element types: the one-query form, the register-tiled form (several new rows on a non-empty
    cache) and the split-key decode form."""
    ks = kernel_sets[dtype]
    H = G = 2
    hd, n = 32, 900
    scale = 1.0 / math.sqrt(hd)
    for far, window, seen in FAR_CASES:
        q, k, v = far_key_case(H, G, hd, n, far, dtype)
        kp, vp, bt = paged([k], [v], [n], dtype=dtype, seed=far)
        out = torch.empty(1, H * hd, dtype=dtype, device="cuda")
        qd = dev(q.reshape(1, -1), dtype)
        ks.attn_paged(qd, out, dev([0, 1], torch.int32), dev([n - 1], torch.int32), bt, kp, vp, 1, 1, H, G, hd, window, scale)
        want = plain.attention(f64(q), f64(k), f64(v), torch.tensor([n - 1]), torch.arange(n), window).reshape(1, -1)
        assert rel_err(out.cpu().float(), want) < TOL[dtype]
        hit = rel_err(out.cpu().float(), f64(v[far]).reshape(1, -1)) < 1e-2
        assert hit == seen
        for n_split in (1, 5):
            part = torch.empty(H * n_split * (hd + 2), dtype=torch.float32, device="cuda")
            out.fill_(float("nan"))
            ks.attn_decode_split(qd, out, dev([n - 1], torch.int32), bt, kp, vp, part, 1, H, G, hd, window, scale, n_split)
            assert rel_err(out.cpu().float(), want) < TOL[dtype]
            assert (rel_err(out.cpu().float(), f64(v[far]).reshape(1, -1)) < 1e-2) == seen
        if dtype == torch.bfloat16:
            for n_split in (1, 5):
                scratch = torch.empty(H * n_split * (hd + 2), dtype=torch.float32, device="cuda")
                ks.decode.attn_decode(qd, out, dev([n - 1], torch.int32), bt, kp, vp, scratch, 1, H, G, hd, window, scale, n_split)
                assert rel_err(out.cpu().float(), want) < TOL[dtype]
                assert (rel_err(out.cpu().float(), f64(v[far]).reshape(1, -1)) < 1e-2) == seen
        # the register-tiled form: the last 7 rows are new, the far key lies in an earlier page of the cache
        n_new = 7
        q7, k7, v7 = far_key_case(H, G, hd, n, far, dtype, n_new)
        out7 = torch.empty(n_new, H * hd, dtype=dtype, device="cuda")
        ks.attn_paged(dev(q7.reshape(n_new, -1), dtype), out7, dev([0, n_new], torch.int32), dev([n - n_new], torch.int32), bt,
                      kp, vp, 1, n_new, H, G, hd, window, scale)
        want7 = plain.attention(f64(q7), f64(k7), f64(v7), torch.arange(n - n_new, n), torch.arange(n), window).reshape(n_new, -1)
        assert rel_err(out7.cpu().float(), want7) < TOL[dtype]
        assert (rel_err(out7[-1:].cpu().float(), f64(v[far]).reshape(1, -1)) < 1e-2) == seen


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("H, G", [(4, 2), (24, 2), (3, 3)])
def test_fast_bfloat16_attention_finds_one_far_key_and_respects_the_windows_edge(kernel_sets, hd, H, G):
    """The same through the kernels that generation uses at real head widths: the tcgen05 prompt
    attention with new rows on a non-empty cache (the far key in an earlier page, the window's edge
    inside a 64-key tile and on a tile boundary), the decode attention on mma.sync with grouped
    queries (4 and 24 heads on 2 key/value heads: its lower rows only, and its upper rows too) and
    its one-head form, with one and five splits, and the decode form that rotates and writes the
    cache itself (identity rotation: position table of angle 0)."""
    ks = kernel_sets[torch.bfloat16]
    n = 900
    scale = 1.0 / math.sqrt(hd)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ident = torch.zeros(n, hd // 2, 2, dtype=torch.float32, device="cuda")
    ident[..., 0] = 1.0                                                  # cos 1, sin 0 at every position
    for far, window, seen in FAR_CASES:
        q, k, v = far_key_case(H, G, hd, n, far, torch.bfloat16)
        kp, vp, bt = paged([k], [v], [n], dtype=torch.bfloat16, seed=far)
        qd = dev(q.reshape(1, -1), torch.bfloat16)
        want = plain.attention(f64(q), f64(k), f64(v), torch.tensor([n - 1]), torch.arange(n), window).reshape(1, -1)
        vfar = torch.cat([f64(v[far, h // (H // G)]) for h in range(H)]).reshape(1, -1)
        tickets = torch.zeros(G, dtype=torch.int32, device="cuda")
        for n_split in (1, 5):
            scratch = torch.empty(H * n_split * (hd + 2), dtype=torch.float32, device="cuda")
            out = torch.full((1, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
            ks.decode.attn_decode(qd, out, dev([n - 1], torch.int32), bt, kp, vp, scratch, 1, H, G, hd, window, scale, n_split,
                                  tickets=tickets)
            assert rel_err(out.cpu().float(), want) < 1.2e-2
            assert (rel_err(out.cpu().float(), vfar) < 1e-2) == seen
            # rotation and cache write fused: raw row [q | k | v] of the last position, the cache holds the rest
            raw = torch.cat([q.reshape(1, -1), k[n - 1].reshape(1, -1), v[n - 1].reshape(1, -1)], dim=1)
            kp2, vp2 = kp.clone(), vp.clone()
            pg = int(bt[0, (n - 1) // PAGE])
            kp2[pg, :, (n - 1) % PAGE] = float("nan")
            vp2[pg, :, (n - 1) % PAGE] = float("nan")
            out.fill_(float("nan"))
            ks.decode.attn_decode_rope(dev(raw, torch.bfloat16), out, dev([n - 1], torch.int32), bt, kp2, vp2, scratch, tickets,
                                       ident, hd, False, True, 1, H, G, hd, window, scale, n_split)
            assert rel_err(out.cpu().float(), want) < 1.2e-2
            assert (rel_err(out.cpu().float(), vfar) < 1e-2) == seen
            assert torch.equal(kp2[pg, :, (n - 1) % PAGE], kp[pg, :, (n - 1) % PAGE])
        # prompt attention: 70 new rows on 830 cached keys; the last row's far key lies pages back
        n_new = 70
        q7, k7, v7 = far_key_case(H, G, hd, n, far, torch.bfloat16, n_new)
        out7 = torch.full((n_new, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        ks.prefill_attention_tc.attn(dev(q7.reshape(n_new, -1), torch.bfloat16), out7, dev([0, n_new], torch.int32),
                                     dev([n - n_new], torch.int32), bt, kp, vp, 1, n_new, H, G, hd, window, scale, err)
        want7 = plain.attention(f64(q7), f64(k7), f64(v7), torch.arange(n - n_new, n), torch.arange(n), window).reshape(n_new, -1)
        assert int(err) == 0
        assert rel_err(out7.cpu().float(), want7) < 1.2e-2
        assert (rel_err(out7[-1:].cpu().float(), vfar) < 1e-2) == seen


# --------------------------------------------------------------------------- sampling
def params_for(options, seeds, draws):
    from scriptling_llm_lib_b200.sampling.sampler import pack_params
    return dev(pack_params(options, seeds, draws))


@pytest.mark.parametrize("V", [5, 384, 1003, 49152])
def test_sampling_kernel_follows_the_plain_samplers(V):
    from scriptling_llm_lib_b200.csrc.bindings import SamplingKernels
    from scriptling_llm_lib_b200.sampling.sampler import SamplingOptions
    sk = SamplingKernels()
    n = 12
    logits = rand(n, V, seed=70, scale=2.5)
    logits[0, 3] = logits[0].max() + 1.0
    if V > 4:
        logits[0, 1] = logits[0, 3]                                     # equal maxima: the first wins
        logits[1, :] = 0.25                                             # all equal but one: ties everywhere
        logits[1, 0] = 0.5
    lg = dev(logits)
    seeds = [1000 + 7 * i for i in range(n)]
    draws = [i % 5 for i in range(n)]
    for opts in [SamplingOptions("greedy"), SamplingOptions("temperature", 0.8), SamplingOptions("temperature", 2.5),
                 SamplingOptions("top_k", 0.9, top_k=7), SamplingOptions("top_k", 1.0, top_k=1),
                 SamplingOptions("top_k", 1.3, top_k=10 ** 6), SamplingOptions("top_p", 1.0, top_p=0.5),
                 SamplingOptions("top_p", 0.7, top_p=0.9), SamplingOptions("top_p", 1.0, top_p=1.0),
                 SamplingOptions("temperature", 0.0)]:
        out = torch.empty(n, dtype=torch.int32, device="cuda")
        sk.sample_rows(lg, params_for(opts, seeds, draws), out)
        got = out.cpu().tolist()
        for i in range(n):
            u = plain.uniform_for(seeds[i], draws[i])
            strategy = "greedy" if opts.is_greedy else opts.strategy
            want = plain.sample(logits[i].numpy(), strategy, opts.temperature or 1.0, opts.top_k, opts.top_p, u)
            assert got[i] == want, f"{opts} row {i}: kernel {got[i]}, plain {want}"
    # a strided view of a wider buffer (the padded logits of a replayed step)
    wide = torch.zeros(n, V + 13, device="cuda")
    wide[:, :V] = lg
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    sk.sample_rows(wide[:, :V], params_for(SamplingOptions("greedy"), seeds, draws), out)
    assert out.cpu().tolist() == [plain.argmax_first(logits[i].numpy()) for i in range(n)]


def test_temperature_sampling_has_the_right_distribution():
    from scriptling_llm_lib_b200.csrc.bindings import SamplingKernels
    from scriptling_llm_lib_b200.sampling.sampler import SamplingOptions
    sk = SamplingKernels()
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5]])
    n = 4000
    lg = dev(logits.repeat(n, 1))
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    sk.sample_rows(lg, params_for(SamplingOptions("temperature", 0.7), [5] * n, list(range(n))), out)
    freq = np.bincount(out.cpu().numpy(), minlength=5) / n
    assert np.abs(freq - plain.softmax_t(logits[0].numpy(), 0.7)).max() < 0.03


def test_repeat_penalty_kernel():
    from scriptling_llm_lib_b200.csrc.bindings import SamplingKernels
    sk = SamplingKernels()
    logits = rand(3, 50, seed=80)
    lg = dev(logits.clone())
    recent = [[4, 9, 4, 49, 60, -1, 9], list(range(30)), [7]]
    last_n = 6
    win = np.full((3, last_n), -1, dtype=np.int32)
    counts = np.zeros(3, dtype=np.int32)
    for i, r in enumerate(recent):
        tail = r[-last_n:]
        win[i, :len(tail)], counts[i] = tail, len(tail)
    pen = dev([1.3, 2.0, 0.0])
    sk.repeat_penalty(lg, dev(win), dev(counts), pen, last_n)
    for i, p in enumerate([1.3, 2.0]):
        want = plain.apply_repeat_penalty(logits[i].numpy(), recent[i], p, last_n)
        assert rel_err(lg[i].cpu(), want) < 1e-6
    assert torch.equal(lg[2].cpu(), logits[2])                           # penalty 0: off
