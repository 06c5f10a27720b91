"""Dense operators: Linear (+bias, +residual, +SwiGLU), RMSNorm, SiLU-mul, embedding, arg-max.

On CUDA tensors every function launches the hand-written sm_100a kernels from ``libfb_kernels.so``; on
CPU tensors it evaluates the plain PyTorch definition, which is also the numerical oracle of the tests.
Operator semantics follow the reference's op API (include/fastllm.h:874-1318): ``Linear(x[n,m], W[k,m],
b[k]) -> y[n,k]`` with weights stored ``[out, in]`` row-major.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.nn.functional as F

from . import _lib, cpu

GEMM_BIAS, GEMM_RESIDUAL, GEMM_SWIGLU, GEMM_OUT_F32 = 1, 2, 4, 8


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return 1
    if dt == torch.float16:
        return 0
    raise TypeError(f"16-bit kernels need fp16/bf16, got {dt}")


# ---------------------------------------------------------------------------------------------------
# gate/up weight interleave used by the fused SwiGLU epilogue
# ---------------------------------------------------------------------------------------------------
def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Stack gate and up rows so that every 128-row tile holds 64 gate rows followed by their 64 up rows.

    Works for weights ``[I, H]`` and for per-row vectors ``[I]`` (biases, scales).  ``I`` must be a
    multiple of 64.
    """
    inter = w_gate.shape[0]
    if inter % 64 != 0:
        raise ValueError("intermediate size must be a multiple of 64 for the fused SwiGLU layout")
    rest = w_gate.shape[1:]
    g = w_gate.reshape(inter // 64, 64, *rest)
    u = w_up.reshape(inter // 64, 64, *rest)
    return torch.cat([g, u], dim=1).reshape(2 * inter, *rest).contiguous()


def deinterleave_gate_up(w: torch.Tensor):
    inter = w.shape[0] // 2
    rest = w.shape[1:]
    t = w.reshape(inter // 64, 2, 64, *rest)
    return t[:, 0].reshape(inter, *rest), t[:, 1].reshape(inter, *rest)


# ---------------------------------------------------------------------------------------------------
# Linear
# ---------------------------------------------------------------------------------------------------
def linear_ref(x, w, bias=None, residual=None, swiglu=False, interleaved=True, out_dtype=None):
    """fp32 reference of ``linear``; mirrors the fused epilogue order (bias -> swiglu -> residual)."""
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if swiglu:
        if interleaved:
            n = y.shape[-1]
            t = y.reshape(*y.shape[:-1], n // 128, 2, 64)
            g, u = t[..., 0, :], t[..., 1, :]
            y = (F.silu(g) * u).reshape(*y.shape[:-1], n // 2)
        else:
            g, u = y.chunk(2, dim=-1)
            y = F.silu(g) * u
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def cpu_native(x: torch.Tensor) -> bool:
    """True when ``x`` should run on the C++ CPU backend (fp32 CPU tensor and the library is built)."""
    return (not x.is_cuda) and x.dtype == torch.float32 and cpu.available()


def cpu_linear_epilogue(y, residual, swiglu, interleaved, out_dtype=None):
    """SwiGLU / residual after a native CPU linear, in the same order as the fused CUDA epilogue."""
    if swiglu:
        if interleaved:
            n = y.shape[-1]
            t = y.reshape(*y.shape[:-1], n // 128, 2, 64)
            y = (F.silu(t[..., 0, :]) * t[..., 1, :]).reshape(*y.shape[:-1], n // 2)
        else:
            y = cpu.swiglu(y)
    if residual is not None:
        y = y + residual.float()
    return y if out_dtype is None else y.to(out_dtype)


# A fused tensor-parallel collective that ended without waiting for its peers' rows leaves a pending wait here:
# (address of the arrival counter, address of its expected value, fallback that launches a stand-alone wait kernel).
# The next ``linear`` hands the two addresses to its GEMM, whose producer thread waits after it has requested its first
# weight tiles; any other path calls ``flush_pending_wait`` first.
_pending_wait = None


def set_pending_wait(cnt_ptr: int, expect_ptr: int, flush_fn) -> None:
    global _pending_wait
    flush_pending_wait()
    _pending_wait = (cnt_ptr, expect_ptr, flush_fn)


def flush_pending_wait() -> None:
    """Resolve an outstanding deferred wait with a stand-alone kernel (consumers that cannot wait themselves)."""
    global _pending_wait
    if _pending_wait is not None:
        fn = _pending_wait[2]
        _pending_wait = None
        fn()


def _take_pending_wait():
    global _pending_wait
    w = _pending_wait
    _pending_wait = None
    return w


F32_SPLIT = os.environ.get("FB_F32_SPLIT", "1") != "0"
_F32_PARTS: dict = {}


def _f32_split(w: torch.Tensor):
    """(bf16 head, bf16 remainder) of an fp32 weight, built once per weight tensor."""
    key = (w.data_ptr(), tuple(w.shape), w._version)
    p = _F32_PARTS.get(key)
    if p is None:
        if len(_F32_PARTS) > 4096:
            _F32_PARTS.clear()
        wh = w.to(torch.bfloat16)
        p = _F32_PARTS[key] = (wh, (w - wh.float()).to(torch.bfloat16))
    return p


def linear(x: torch.Tensor, w: torch.Tensor, bias=None, residual=None, swiglu: bool = False, interleaved: bool = True,
           out_f32: bool = False, out: torch.Tensor | None = None, nsplit: int = 0) -> torch.Tensor:
    """``y = x @ w.T`` with optional fused bias, SwiGLU (``w`` = gate/up stacked) and residual add.

    x: ``[M, K]`` (row stride may exceed K), w: ``[N, K]``.  16-bit CUDA tensors run the tcgen05 GEMM.
    """
    if not x.is_cuda:
        flush_pending_wait()
        # native kernels for decode-sized batches and for 16-bit weights (used in place); large fp32 GEMMs go to the BLAS
        # behind torch.matmul
        if cpu_native(x) and (x.numel() // x.shape[-1] <= 32 or w.dtype != torch.float32):
            return cpu_linear_epilogue(cpu.linear(x, w, bias), residual, swiglu, interleaved)
        return linear_ref(x, w, bias, residual, swiglu, interleaved, torch.float32 if out_f32 else None)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M, K = x2.shape
    N = w.shape[0]
    if (x.dtype == torch.float32 and w.dtype == torch.float32 and K % 64 == 0 and N % 8 == 0 and F32_SPLIT and out is None
            and w.is_contiguous()):
        # fp32 activations and weights on the tensor core: both operands are split into a bf16 head and a bf16 remainder
        # (x = xh + xl with 16 mantissa bits between them) and y = xh wh' + xh wl' + xl wh' runs as three bf16 GEMMs with fp32
        # accumulation; the dropped xl wl' term is 2^-16 relative, far below TF32's 2^-11 operand rounding
        # (reference: a CUDA-core fp32 GEMV / cuBLAS SGEMM, src/devices/cuda/linear/fastllm-linear-fp32.cu:11)
        flush_pending_wait()
        wh, wl = _f32_split(w)
        xh = x2.to(torch.bfloat16)
        xl = (x2 - xh.float()).to(torch.bfloat16)
        y = linear(xh, wh, out_f32=True)
        y += linear(xh, wl, out_f32=True)
        y += linear(xl, wh, out_f32=True)
        if bias is not None:
            y += bias.float()
        if swiglu:
            y = glu_act_ref(y, "silu", interleaved)
        if residual is not None:
            y += residual.reshape(-1, residual.shape[-1]).float()
        return y.reshape(*lead, y.shape[-1])
    if K % 64 != 0 or N % 8 != 0 or x.dtype not in (torch.float16, torch.bfloat16) or (x2.data_ptr() & 15) or (x2.stride(0) * 2) % 16:
        # shapes outside the tensor-core kernels' tiling (rare: odd projection widths): plain PyTorch definition
        flush_pending_wait()
        return linear_ref(x, w, bias, residual, swiglu, interleaved, torch.float32 if out_f32 else None)
    if swiglu and not interleaved:
        raise ValueError("CUDA SwiGLU epilogue needs tile-interleaved gate/up weights (interleave_gate_up)")
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((M, n_out), device=x.device, dtype=torch.float32 if out_f32 else x.dtype)
    flags = (GEMM_BIAS if bias is not None else 0) | (GEMM_RESIDUAL if residual is not None else 0) | \
            (GEMM_SWIGLU if swiglu else 0) | (GEMM_OUT_F32 if out_f32 else 0)
    res2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
    lib = _lib.kernels()
    dt = dtype_code(x.dtype)
    if M <= 256 or N % 32 != 0:
        step = 256
        pend = _take_pending_wait()
        for m0 in range(0, M, step):
            m1 = min(M, m0 + step)
            if pend is not None:
                rc = lib.fb_gemm_16bit_wait(_ptr(x2[m0:m1]), _ptr(w), _ptr(out[m0:m1]), _ptr(bias),
                                            _ptr(res2[m0:m1]) if res2 is not None else _ptr(None), m1 - m0, N, K, x2.stride(0),
                                            w.stride(0), out.stride(0), res2.stride(0) if res2 is not None else 0, dt, flags, nsplit,
                                            ctypes.c_void_p(pend[0]), ctypes.c_void_p(pend[1]), _stream())
                pend = None
                _lib.check(rc, "fb_gemm_16bit_wait")
                continue
            rc = lib.fb_gemm_16bit(_ptr(x2[m0:m1]), _ptr(w), _ptr(out[m0:m1]), _ptr(bias),
                                   _ptr(res2[m0:m1]) if res2 is not None else _ptr(None), m1 - m0, N, K, x2.stride(0),
                                   w.stride(0), out.stride(0), res2.stride(0) if res2 is not None else 0, dt, flags, nsplit,
                                   _stream())
            _lib.check(rc, "fb_gemm_16bit")
    else:
        flush_pending_wait()
        rc = lib.fb_gemm_16bit(_ptr(x2), _ptr(w), _ptr(out), _ptr(bias), _ptr(res2), M, N, K, x2.stride(0), w.stride(0),
                               out.stride(0), res2.stride(0) if res2 is not None else 0, dt, flags, nsplit, _stream())
        _lib.check(rc, "fb_gemm_16bit")
    return out.reshape(*lead, n_out)


def linear_batched(x: torch.Tensor, w: torch.Tensor, batch: int, x_cols: int, out: torch.Tensor, out_cols: int) -> torch.Tensor:
    """``out[m, z * out_cols + n] = sum_k x[m, z * x_cols + k] * w[z, n, k]`` for ``z < batch``: one small GEMM per attention head
    in one launch (the absorbed multi-head-latent-attention projections).  x ``[M, >= batch * x_cols]``, w ``[batch, N, K]``
    contiguous, out ``[M, >= batch * out_cols]`` (written in place and returned)."""
    M = x.shape[0]
    _, N, K = w.shape
    ok = (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and w.dtype == x.dtype and out.dtype == x.dtype and K % 64 == 0
          and N % 8 == 0 and x_cols % 8 == 0 and out_cols % 4 == 0 and x.stride(-1) == 1 and out.stride(-1) == 1
          and not (x.data_ptr() & 15) and not ((x.stride(0) * 2) & 15) and w.is_contiguous())
    if not ok:
        flush_pending_wait()
        xs = x.as_strided((M, batch, K), (x.stride(0), x_cols, 1))
        ov = out.as_strided((M, batch, N), (out.stride(0), out_cols, 1))
        ov.copy_(torch.einsum("mzk,znk->mzn", xs.float(), w.float()).to(out.dtype))
        return out
    flush_pending_wait()
    lib = _lib.kernels()
    for m0 in range(0, M, 256):
        m1 = min(M, m0 + 256)
        rc = lib.fb_gemm_16bit_batched(_ptr(x[m0:m1]), _ptr(w), _ptr(out[m0:m1]), m1 - m0, N, K, batch, x.stride(0), K, out.stride(0),
                                       x_cols, out_cols, dtype_code(x.dtype), _stream())
        _lib.check(rc, "fb_gemm_16bit_batched")
    return out


# ---------------------------------------------------------------------------------------------------
# RMSNorm
# ---------------------------------------------------------------------------------------------------
def rmsnorm_ref(x, w, eps, residual=None, unit_offset=0.0):
    h = x.float()
    if residual is not None:
        h = (h + residual.float()).to(x.dtype).float()
    y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + unit_offset)
    return y.to(x.dtype), (h.to(x.dtype) if residual is not None else None)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: torch.Tensor | None = None, unit_offset: float = 0.0,
            out: torch.Tensor | None = None, quant_mode: int = 0) -> torch.Tensor:
    """RMSNorm over the last dim.  With ``residual`` given: ``residual += x`` in place, then normalise it.

    ``quant_mode`` 3 / 4: ``y`` itself is rounded to the int8 / e4m3 grid per 128-wide block (``y.fb_quant = (mode, ...)`` marks it).
    ``quant_mode`` 1 (int8) / 2 (e4m3): the kernel also writes the row quantised per 128-wide block for the 8-bit-activation
    GEMM that consumes it; the result carries it as ``y.fb_quant = (mode, xq, scales, sums, ld_a)`` and the quantised linear
    layers pick it up instead of launching their own quantiser."""
    if not x.is_cuda:
        if cpu_native(x) and (residual is None or residual.dtype == torch.float32):
            if residual is not None:
                residual.add_(x)
                x = residual
            return cpu.rmsnorm(x, w, eps, unit_offset)
        y, new_res = rmsnorm_ref(x, w, eps, residual, unit_offset)
        if residual is not None:
            residual.copy_(new_res)
        return y
    x2 = x.reshape(-1, x.shape[-1])
    M, H = x2.shape
    if out is None:
        out = torch.empty((M, H), device=x.device, dtype=x.dtype)
    if residual is not None and not residual.is_contiguous():
        raise ValueError("residual must be contiguous")
    if quant_mode in (3, 4) and H % 128 == 0 and x.dtype in (torch.float16, torch.bfloat16):
        # y rounded to the 8-bit grid its consumer's small-batch kernels use (large batches run on 16-bit activations)
        rc = _lib.kernels().fb_rmsnorm_quant(_ptr(x2), _ptr(w), _ptr(out), _ptr(residual), M, H, x2.stride(0), out.stride(0), float(eps),
                                             float(unit_offset), dtype_code(x.dtype), quant_mode, _ptr(None), 0, _ptr(None), _ptr(None), 0,
                                             _stream())
        _lib.check(rc, "fb_rmsnorm_quant")
        y = out.reshape(x.shape)
        y.fb_quant = (quant_mode, None, None, None, 0)
        return y
    if quant_mode in (1, 2) and H % 128 == 0 and M <= 128 and x.dtype in (torch.float16, torch.bfloat16):
        ld_a = (M + 128 + 3) // 4 * 4
        xq = torch.empty((M, H), device=x.device, dtype=torch.int8 if quant_mode == 1 else torch.uint8)
        sa = torch.empty((H // 128, ld_a), device=x.device, dtype=torch.float32)
        xs = torch.empty((H // 128, ld_a), device=x.device, dtype=torch.float32) if quant_mode == 1 else None
        rc = _lib.kernels().fb_rmsnorm_quant(_ptr(x2), _ptr(w), _ptr(out), _ptr(residual), M, H, x2.stride(0), out.stride(0), float(eps),
                                             float(unit_offset), dtype_code(x.dtype), quant_mode, _ptr(xq), H, _ptr(sa), _ptr(xs), ld_a,
                                             _stream())
        _lib.check(rc, "fb_rmsnorm_quant")
        y = out.reshape(x.shape)
        y.fb_quant = (quant_mode, xq, sa, xs, ld_a)
        return y
    rc = _lib.kernels().fb_rmsnorm(_ptr(x2), _ptr(w), _ptr(out), _ptr(residual), M, H, x2.stride(0), out.stride(0), float(eps),
                                   float(unit_offset), dtype_code(x.dtype), _stream())
    _lib.check(rc, "fb_rmsnorm")
    return out.reshape(x.shape)


# ---------------------------------------------------------------------------------------------------
# SiLU-mul, embedding, arg-max
# ---------------------------------------------------------------------------------------------------
def silu_mul(x: torch.Tensor) -> torch.Tensor:
    """``silu(x[..., :I]) * x[..., I:]``"""
    inter = x.shape[-1] // 2
    if not x.is_cuda:
        if cpu_native(x):
            return cpu.swiglu(x)
        g, u = x.float().chunk(2, dim=-1)
        return (F.silu(g) * u).to(x.dtype)
    x2 = x.reshape(-1, x.shape[-1])
    out = torch.empty((x2.shape[0], inter), device=x.device, dtype=x.dtype)
    rc = _lib.kernels().fb_silu_mul(_ptr(x2), _ptr(out), x2.shape[0], inter, x2.stride(0), out.stride(0), dtype_code(x.dtype),
                                    _stream())
    _lib.check(rc, "fb_silu_mul")
    return out.reshape(*x.shape[:-1], inter)


GLU_ACTS = {"silu": 0, "swiglu": 0, "gelu_pytorch_tanh": 1, "gelu_new": 1, "gelu_fast": 1, "gelu_tanh": 1, "gelu": 2, "relu": 3}


def glu_act_ref(x: torch.Tensor, act: str, interleaved: bool = False) -> torch.Tensor:
    """PyTorch fp32 statement of ``act(gate) * up`` (both layouts)."""
    if interleaved:
        n = x.shape[-1]
        t = x.reshape(*x.shape[:-1], n // 128, 2, 64)
        g, u = t[..., 0, :].reshape(*x.shape[:-1], n // 2), t[..., 1, :].reshape(*x.shape[:-1], n // 2)
    else:
        g, u = x.chunk(2, dim=-1)
    gf = g.float()
    code = GLU_ACTS[act]
    a = F.silu(gf) if code == 0 else F.gelu(gf, approximate="tanh") if code == 1 else F.gelu(gf) if code == 2 else torch.relu(gf)
    return (a * u.float()).to(x.dtype)


def glu_act(x: torch.Tensor, act: str, interleaved: bool = False) -> torch.Tensor:
    """``act(gate) * up`` of a fused gate/up projection output ``[..., 2I]`` -> ``[..., I]``.  ``interleaved``: gate and up
    alternate in blocks of 64 columns (the layout of the fused gate/up weights); else the gate half comes first."""
    if act not in GLU_ACTS:
        raise ValueError(f"unsupported MLP activation '{act}'")
    inter = x.shape[-1] // 2
    if not x.is_cuda or x.dtype not in (torch.float16, torch.bfloat16) or inter % 8 != 0 or (interleaved and inter % 64 != 0):
        return glu_act_ref(x, act, interleaved)
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], inter), device=x.device, dtype=x.dtype)
    rc = _lib.kernels().fb_glu_act(_ptr(x2), _ptr(out), x2.shape[0], inter, x2.stride(0), out.stride(0), GLU_ACTS[act],
                                   1 if interleaved else 0, dtype_code(x.dtype), _stream())
    _lib.check(rc, "fb_glu_act")
    return out.reshape(*x.shape[:-1], inter)


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if not table.is_cuda or table.dtype not in (torch.float16, torch.bfloat16):
        return F.embedding(ids.long(), table)
    ids32 = ids.reshape(-1).to(torch.int32)
    M, H = ids32.numel(), table.shape[1]
    if out is None:
        out = torch.empty((M, H), device=table.device, dtype=table.dtype)
    rc = _lib.kernels().fb_embedding(_ptr(ids32), _ptr(table), _ptr(out), M, H, table.shape[0], _stream())
    _lib.check(rc, "fb_embedding")
    return out.reshape(*ids.shape, H)


def argmax(logits: torch.Tensor, id_offset: int = 0, want_values: bool = False, out: torch.Tensor | None = None):
    """Row-wise arg-max (ties -> lowest index) as int32; optionally also the max values (fp32)."""
    if not logits.is_cuda:
        v, i = logits.float().max(dim=-1)
        i = (i + id_offset).to(torch.int32)
        if out is not None:
            out.copy_(i)
            i = out
        return (i, v) if want_values else i
    l2 = logits.reshape(-1, logits.shape[-1])
    M, V = l2.shape
    ids = out if out is not None else torch.empty((M,), device=logits.device, dtype=torch.int32)
    vals = torch.empty((M,), device=logits.device, dtype=torch.float32) if want_values else None
    kind = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[logits.dtype]
    rc = _lib.kernels().fb_argmax(_ptr(l2), _ptr(ids), _ptr(vals), M, V, l2.stride(0), id_offset, kind, _stream())
    _lib.check(rc, "fb_argmax")
    return (ids, vals) if want_values else ids
