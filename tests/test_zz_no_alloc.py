"""Allocation-free decode attention (``fb_attn_decode_static``).

Some hosts of the kernel library cannot allocate device memory around a call -- a server that has frozen
device allocation after start-up, a plug-in that only borrows tensors from another runtime -- so the
library offers one entry point that keeps its scratch in a fixed device array of its own.  This test calls
that entry point through its exported C symbol, twice in a row with different inputs (the array is shared
and keeps the previous call's contents), and checks each result against the regular entry point that takes
caller-allocated scratch and against the plain PyTorch evaluation of the same attention.  It also checks that an over-sized request is refused before anything is launched.
"""
import ctypes
import math
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = Path(__file__).resolve().parent.parent / "fastllm_b200" / "lib" / "libfb_kernels.so"
TOO_LARGE = -3


def _sym():
    lib = ctypes.CDLL(str(LIB))
    fn = lib.fb_attn_decode_static
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn.argtypes = [P, P, P, P, I, P, P, I, I, I, I, LL, I, F, I, P]
    fn.restype = I
    return fn


def _case(seed, lens, Hq, Hkv, dev):
    from tests.test_kernels_gpu import _make_cache

    torch.manual_seed(seed)
    D, dt = 128, torch.bfloat16
    k_pool, v_pool, pt = _make_cache(len(lens), lens, Hkv, D, dt)
    q = torch.randn(len(lens), Hq * D).to(dt)
    seq = torch.tensor(lens, dtype=torch.int32)
    return [t.to(dev) for t in (q, k_pool, v_pool, pt, seq)]


def test_static_scratch_entry_matches_regular_entry():
    from fastllm_b200.ops import _lib, attention as A

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    fn = _sym()
    Hq, Hkv, D = 32, 8, 128
    scale = 1 / math.sqrt(D)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for seed, lens in ((11, [1, 130, 700, 64, 257]), (12, [900, 3, 128])):      # two calls in a row, different shapes
        q, k_pool, v_pool, pt, seq = _case(seed, lens, Hq, Hkv, dev)
        ref = A.attn_decode(q, k_pool, v_pool, pt, seq, scale, Hq, Hkv, D)
        out = torch.empty_like(q)
        rc = fn(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), out.stride(0), pt.data_ptr(), seq.data_ptr(),
                len(lens), Hq, Hkv, D, k_pool.shape[0] * k_pool.shape[1], pt.stride(0), scale, 1, stream)
        assert rc == 0, f"fb_attn_decode_static returned {rc}"
        torch.cuda.synchronize()
        _lib.check_device_errors()
        err = (out.float() - ref.float()).abs()
        tol = 2e-2 + 2e-2 * ref.float().abs()
        assert bool((err <= tol).all()), f"max err {err.max().item()}"
        # and against the plain PyTorch evaluation of paged attention (what attn_decode computes for CPU tensors)
        ref32 = A.attn_decode(q.cpu(), k_pool.cpu(), v_pool.cpu(), pt.cpu(), seq.cpu(), scale, Hq, Hkv, D).float()
        err = (out.float().cpu() - ref32).abs()
        assert bool((err <= 2e-2 + 2e-2 * ref32.abs()).all()), f"max err vs PyTorch {err.max().item()}"


def test_static_scratch_entry_rejects_oversize():
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    fn = _sym()
    dummy = torch.zeros(16, device=dev, dtype=torch.int32)
    # 1024 requests x 64 pages = 65536 work items > 16384: must be refused without launching anything
    rc = fn(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 4096, dummy.data_ptr(), dummy.data_ptr(),
            1024, 32, 8, 128, 1 << 20, 64, 0.1, 1, ctypes.c_void_p(0))
    assert rc == TOO_LARGE
    torch.cuda.synchronize()
