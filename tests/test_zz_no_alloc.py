"""The decode-attention entry point that allocates nothing, called through its exported C symbol
and compared with the ordinary entry point (which takes the caller's scratch) and with the plain
implementation's attention.

Some callers cannot allocate device memory while they run (a callback inside another library, a
loop that must not hit cudaMalloc's synchronisation, a program whose own arena owns all device
memory); for them the per-split scratch sits in a fixed array inside the library. Here both entry
points get the same inputs, twice in a row with different data, so that anything the shared array
kept from the first call would show in the second. This file sorts last on purpose: a run that
stops at the first failure has run every other test before it.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu


def _lib():
    from scriptling_llm_lib_b200.csrc.build import compile_library
    lib = ctypes.CDLL(str(compile_library("decode_bf16")))
    lib.sllm_attn_decode_bf16_noalloc.restype = c_int
    lib.sllm_attn_decode_bf16.restype = c_int
    lib.sllm_attn_decode_noalloc_strerror.restype = ctypes.c_char_p
    lib.sllm_attn_decode_noalloc_capacity_floats.restype = ctypes.c_longlong
    return lib


def _case(seed, B, H, G, hd, lengths):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // 64) for n in lengths) + 2
    kp = torch.randn(n_pages, G, 64, hd, generator=g).bfloat16().cuda()
    vp = torch.randn(n_pages, G, 64, hd, generator=g).bfloat16().cuda()
    order = np.random.default_rng(seed).permutation(n_pages).tolist()
    width = max(-(-n // 64) for n in lengths)
    bt = torch.full((B, width), -1, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for i in range(-(-n // 64)):
            bt[b, i] = order.pop()
    q = (torch.randn(B, H * hd, generator=g) * 2).bfloat16().cuda()
    pos0 = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    return q, kp, vp, bt.cuda(), pos0


def _plain(q, kp, vp, bt, lengths, H, G, hd):
    """The plain implementation's attention for the one query of each sequence over its pages."""
    rows = []
    for b, n in enumerate(lengths):
        pages = [int(p) for p in bt[b, :-(-n // 64)]]
        k = torch.cat([kp[p].permute(1, 0, 2) for p in pages])[:n].double().cpu()       # [n, G, hd]
        v = torch.cat([vp[p].permute(1, 0, 2) for p in pages])[:n].double().cpu()
        rows.append(plain.attention(q[b].double().cpu().view(1, H, hd), k, v, torch.tensor([n - 1]), torch.arange(n)).reshape(1, -1))
    return torch.cat(rows)


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = _lib()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    B, H, G, hd, n_split = 5, 8, 2, 64, 6
    assert lib.sllm_attn_decode_noalloc_capacity_floats() == 1 << 20
    for seed, lengths in [(1, [700, 1, 64, 65, 333]), (2, [3, 512, 129, 900, 64])]:
        q, kp, vp, bt, pos0 = _case(seed, B, H, G, hd, lengths)
        args = (c_void_p(q.data_ptr()), c_int(H * hd))
        tail = (c_void_p(pos0.data_ptr()), c_void_p(bt.data_ptr()), c_int(bt.shape[1]), c_void_p(kp.data_ptr()),
                c_void_p(vp.data_ptr()))
        dims = (c_int(B), c_int(H), c_int(G), c_int(hd), c_int(0), c_float(1.0 / math.sqrt(hd)), c_int(n_split), stream)
        want = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(B * H * n_split * (hd + 2), dtype=torch.float32, device="cuda")
        rc = lib.sllm_attn_decode_bf16(*args, c_void_p(want.data_ptr()), *tail, c_void_p(scratch.data_ptr()), *dims)
        assert rc == 0
        got = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.sllm_attn_decode_bf16_noalloc(*args, c_void_p(got.data_ptr()), *tail, *dims)
        assert rc == 0, lib.sllm_attn_decode_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        scale = float(want.float().abs().max())
        assert float((got.float() - want.float()).abs().max()) <= 6e-3 * scale      # the kernels tests' bfloat16 tolerance
        ref = _plain(q, kp, vp, bt, lengths, H, G, hd)
        assert float((got.double().cpu() - ref).abs().max()) <= 6e-3 * float(ref.abs().max())
        # a warm call takes nothing from the device: the driver's count of free bytes (which sees any
        # cudaMalloc, not only torch's allocator) is the same before and after
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.sllm_attn_decode_bf16_noalloc(*args, c_void_p(got.data_ptr()), *tail, *dims)
        torch.cuda.synchronize()
        assert rc == 0 and torch.cuda.mem_get_info()[0] == free_before


def test_no_alloc_entry_point_refuses_what_its_scratch_cannot_hold():
    lib = _lib()
    q, kp, vp, bt, pos0 = _case(3, 2, 8, 2, 64, [10, 20])
    out = torch.zeros(2, 8 * 64, dtype=torch.bfloat16, device="cuda")
    rc = lib.sllm_attn_decode_bf16_noalloc(
        c_void_p(q.data_ptr()), c_int(8 * 64), c_void_p(out.data_ptr()), c_void_p(pos0.data_ptr()), c_void_p(bt.data_ptr()),
        c_int(bt.shape[1]), c_void_p(kp.data_ptr()), c_void_p(vp.data_ptr()), c_int(2), c_int(8), c_int(2), c_int(64), c_int(0),
        c_float(0.125), c_int(1 << 14), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -10 and b"exceed the built-in scratch" in lib.sllm_attn_decode_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0                          # nothing ran
    assert b"head width" in lib.sllm_attn_decode_noalloc_strerror(-1)
