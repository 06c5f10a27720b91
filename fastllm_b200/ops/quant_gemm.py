"""Weight-only-quantised and block-scaled FP8 GEMM dispatch (CUDA).

``linear_quant`` runs ``csrc/gemm_quant.cu`` (packed weights stream through TMA, dequant in shared memory, tcgen05
MMA) for up to 256 tokens per launch; larger token counts are processed in 256-row chunks up to a limit, beyond which
the caller de-quantises once and uses the dense prefill GEMM (``None`` is returned).
"""
from __future__ import annotations

import ctypes

import os

import torch

from . import _lib
from .basic import GEMM_BIAS, GEMM_OUT_F32, GEMM_RESIDUAL, GEMM_SWIGLU, _ptr, _stream, dtype_code

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_lib.register_sigs({"fb_gemm_quant": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P]}, ["gemm_quant"])

_lib.register_sigs({
    "fb_quant_act_fp8": [P, I, P, I, P, I, I, I, I, P, P],
    "fb_round_act": [P, I, P, I, I, I, I, I, P],
    "fb_gemm_fp8": [P, I, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, P],
    "fb_moe_grouped_gemm_fp8": [P, I, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P],
    "fb_moe_gather_quant_fp8": [P, P, P, P, I, I, I, I, I, P],
    "fb_quant_act_i8": [P, I, P, I, P, P, I, I, I, I, P, P, I, P],
    "fb_gemm_i8": [P, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P, I, I, I, P],
    "fb_gemv_i4": [P, I, P, P, I, P, P, P, I, I, I, I, I, I, P, P, I, P],
}, ["gemm_fp8", "gemm_i8"])

_QMODE = {"int8": 1, "int4g": 2, "fp8": 3, "fp4": 4}
# FP8 weights run as W8A8 (activations quantised per token and 128-wide k block, e4m3 x e4m3 on the tensor core) for decode-sized
# batches; FB_FP8_W8A16=1 keeps 16-bit activations (weights de-quantised in shared memory), which is also the path for M > 128.
FP8_NATIVE = __import__("os").environ.get("FB_FP8_W8A16", "0") != "1"
# fp4 weights with fp16 activations: half2 de-quantiser (one multiply per value pair) while the scale table fits fp16's range
FP4_F16W = __import__("os").environ.get("FB_FP4_F16W", "1") != "0"
GEMM_FP4_F16W = 256


# int8 / int4-group(128) weights run with int8 activations on the integer tensor-core path (FB_INT_A16=1 keeps 16-bit activations)
INT_A8 = __import__("os").environ.get("FB_INT_A16", "0") != "1"


# rows up to which the integer path is the faster one (measured on B200); above it the 16-bit-activation kernels run
INT_A8_MAX_M = {"int8": 128, "int4g": 64}


def uses_int_a8(lw) -> bool:
    return INT_A8 and ((lw.kind == "int8") or (lw.kind == "int4g" and lw.group == 128)) and lw.k % 128 == 0


def quant_act_i8(x2: torch.Tensor, rows_used=None, pos=None, topk: int = 1, rows_cap: int | None = None):
    """x ``[M, K]`` 16-bit -> (int8 ``[rows, K]``, scales, block sums ``[K / 128, ld_a]``).  With ``pos`` the rows are
    scattered to ``pos[pair]`` of an expert-sorted buffer of ``rows_cap`` rows (gather fused with the quantisation)."""
    M, K = x2.shape
    rows = rows_cap if rows_cap is not None else M
    ld_a = (rows + 128 + 3) // 4 * 4
    xq = torch.empty((rows, K), device=x2.device, dtype=torch.int8)
    sa = torch.empty((K // 128, ld_a), device=x2.device, dtype=torch.float32)
    xs = torch.empty((K // 128, ld_a), device=x2.device, dtype=torch.float32)
    n = M * topk if pos is not None else M
    rc = _lib.kernels().fb_quant_act_i8(_ptr(x2), x2.stride(0), _ptr(xq), K, _ptr(sa), _ptr(xs), ld_a, n, K, dtype_code(x2.dtype),
                                        _ptr(rows_used), _ptr(pos), topk, _stream())
    _lib.check(rc, "fb_quant_act_i8")
    return xq, sa, xs, ld_a


def round_act(x: torch.Tensor, mode: int) -> torch.Tensor:
    """``x`` rounded to the int8 (mode 0) or e4m3 (mode 1) grid of its (token, 128-wide k block), in its own 16-bit dtype."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 4 != 0:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], x2.shape[1]), device=x.device, dtype=x.dtype)
    rc = _lib.kernels().fb_round_act(_ptr(x2), x2.stride(0), _ptr(out), out.stride(0), x2.shape[0], x2.shape[1], dtype_code(x.dtype), mode,
                                     _stream())
    _lib.check(rc, "fb_round_act")
    return out.reshape(x.shape)


def act_quant_mode(lw, M: int) -> int:
    """Which form of its input ``lw`` consumes for ``M`` rows: 1 int8 bytes, 2 e4m3 bytes, 3 / 4 16-bit values rounded to the
    int8 / e4m3 grid (batches above the 8-bit kernels' row limit), 0 plain 16-bit activations."""
    if lw is None or lw.k % 128 != 0 or lw.adapters:
        return 0
    if uses_int_a8(lw):
        return 1 if M <= INT_A8_MAX_M[lw.kind] else 3
    if lw.kind == "fp8" and FP8_NATIVE:
        return 2 if M <= 128 else 4
    return 0


def prepare(lw) -> None:
    """Bring a freshly built weight into the form its kernels read (int8: q - 128 bytes for the integer path)."""
    if uses_int_a8(lw) and lw.w.is_cuda:
        _a8_tensors(lw)


I4_GEMV = os.environ.get("FB_I4_GEMV", "1") != "0"      # int4-group weights at one to four rows: dp4a kernel (csrc/gemv_i4.cu)
I4_GEMV_MAX_M = 4


def _a8_tensors(lw):
    """Weight-side tensors of the integer path: (bytes, scale, zero-or-min, kind code).  int8 storage is switched to q - 128 once."""
    if lw.kind == "int8":
        if not lw.signed:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("int8 weight reaches the integer path for the first time inside a CUDA graph capture; "
                                   "call quant_gemm.prepare(weight) when the weight is built")
            lw.w.view(torch.uint8).bitwise_xor_(0x80)          # in place: views of stacked expert storage stay views
            lw.signed = True
        if lw._a8 is None:
            lw._a8 = (lw.scale.float().contiguous(), (lw.zero.float() - 128.0).contiguous())
        return lw.w, lw._a8[0], lw._a8[1], 1
    return lw.w, _kernel_tensors(lw)[0], None, 2          # (scale, min) pairs [groups, N, 2], shared with the 16-bit route


def _linear_i8(x2, lw, out, bias, res2, flags, pre=None):
    M, K = x2.shape
    w, sc, zr, kind = _a8_tensors(lw)
    if pre is not None and pre[0] == 1 and pre[1].shape == (M, K):
        _, xq, sa, xs, ld_a = pre              # quantised by the kernel that produced x (fused RMSNorm)
    else:
        xq, sa, xs, ld_a = quant_act_i8(x2)
    if (kind == 2 and M <= I4_GEMV_MAX_M and I4_GEMV and bias is None and res2 is None and (flags & ~GEMM_SWIGLU) == 0
            and lw.n % 128 == 0 and K <= 16384 and lw.group == 128 and out.dtype == x2.dtype):
        # one to four rows: the CUDA-core dp4a kernel streams the packed rows directly (no unpack / MMA / promotion pipeline)
        rc = _lib.kernels().fb_gemv_i4(_ptr(xq), K, _ptr(sa), _ptr(xs), ld_a, _ptr(w), _ptr(sc), _ptr(out), M, lw.n, K, out.stride(0),
                                       dtype_code(x2.dtype), flags, _ptr(None), _ptr(None), 1, _stream())
        _lib.check(rc, "fb_gemv_i4")
        return
    for m0 in range(0, M, 128):           # the kernel takes up to 128 rows; the weights of later chunks come from L2
        m1 = min(M, m0 + 128)
        rc = _lib.kernels().fb_gemm_i8(_ptr(xq[m0:m1]), K, _ptr(sa[:, m0:]), _ptr(xs[:, m0:]), ld_a, _ptr(w), _ptr(sc), _ptr(zr),
                                       _ptr(out[m0:m1]), _ptr(bias), _ptr(res2[m0:m1]) if res2 is not None else _ptr(None),
                                       m1 - m0, lw.n, K, out.stride(0), res2.stride(0) if res2 is not None else 0,
                                       dtype_code(x2.dtype), flags, kind, 0, _ptr(None), _ptr(None), 0, 0, 0, _stream())
        _lib.check(rc, "fb_gemm_i8")


def quant_act_fp8(x2: torch.Tensor, rows_used: torch.Tensor | None = None):
    """x ``[M, K]`` 16-bit -> (e4m3 ``[M, K]``, scales fp32 ``[K / 128, ld_a]`` with ``ld_a >= M + 128``, multiple of 4)."""
    M, K = x2.shape
    ld_a = (M + 128 + 3) // 4 * 4
    xq = torch.empty((M, K), device=x2.device, dtype=torch.uint8)
    sa = torch.empty((K // 128, ld_a), device=x2.device, dtype=torch.float32)
    rc = _lib.kernels().fb_quant_act_fp8(_ptr(x2), x2.stride(0), _ptr(xq), K, _ptr(sa), ld_a, M, K, dtype_code(x2.dtype), _ptr(rows_used),
                                         _stream())
    _lib.check(rc, "fb_quant_act_fp8")
    return xq, sa, ld_a


def _linear_fp8_native(x2, lw, out, bias, res2, flags, pre=None):
    M, K = x2.shape
    if pre is not None and pre[0] == 2 and pre[1].shape == (M, K):
        _, xq, sa, _xs, ld_a = pre             # quantised by the kernel that produced x (fused RMSNorm)
    else:
        xq, sa, ld_a = quant_act_fp8(x2)
    rc = _lib.kernels().fb_gemm_fp8(_ptr(xq), K, _ptr(sa), ld_a, _ptr(lw.w), _ptr(_kernel_tensors(lw)[0]), _ptr(out), _ptr(bias), _ptr(res2),
                                    M, lw.n, K, out.stride(0), res2.stride(0) if res2 is not None else 0, dtype_code(x2.dtype), flags, 0,
                                    _stream())
    _lib.check(rc, "fb_gemm_fp8")
MAX_CHUNKED_TOKENS = 1024


def _kernel_tensors(lw):
    """Scale tensors in the layout the kernel reads (built once per weight)."""
    if lw._dq is None:
        if lw.kind == "int8":
            lw._dq = (lw.scale.float().contiguous(), lw.zero.float().contiguous())
        elif lw.kind == "int4g":
            sm = torch.stack([lw.scale.float(), lw.zero.float()], dim=-1)          # [N, groups, 2]
            lw._dq = (sm.permute(1, 0, 2).contiguous(), None)                      # [groups, N, 2]
        elif lw.kind == "fp4":
            # bf16 block scales [N, K / group] read as they are; the per-tensor factor (NVFP4) rides in the zero slot; the third
            # entry says whether every scale x 6 stays a normal fp16 number (fp16 activations then take the half2 de-quantiser)
            sf = lw.scale.float()
            nz = sf[sf > 0]
            ok = bool(FP4_F16W and (nz.numel() == 0 or (float(nz.max()) * 6.0 < 60000.0 and float(nz.min()) * 0.5 >= 2.0 ** -14)))
            lw._dq = (lw.scale.to(torch.bfloat16).contiguous(), lw.zero.float().contiguous() if lw.zero is not None else None, ok)
        else:
            lw._dq = (lw.scale.float().contiguous(), None)
    return lw._dq


def linear_quant(x, lw, residual=None, swiglu=False, out_f32=False):
    if lw.kind not in _QMODE or x.dtype not in (torch.float16, torch.bfloat16):
        return None
    lead = x.shape[:-1]
    pre = getattr(x, "fb_quant", None)
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M, K = x2.shape
    N = lw.n
    if M > MAX_CHUNKED_TOKENS or K % 64 != 0 or N % 8 != 0:
        return None
    if lw.kind == "int4g" and (lw.group % 64 != 0 or K % lw.group != 0):
        return None
    if lw.kind == "fp8" and K % 128 != 0:
        return None
    if lw.kind == "fp4" and (lw.group not in (16, 32) or (N * (K // lw.group)) % 2 != 0):
        return None
    if swiglu and (not lw.interleaved or N % 128 != 0):
        return None
    a8 = uses_int_a8(lw) and M <= INT_A8_MAX_M[lw.kind] and x2.stride(0) % 4 == 0
    scale, zero = (None, None) if a8 else _kernel_tensors(lw)[:2]
    n_out = N // 2 if swiglu else N
    out = torch.empty((M, n_out), device=x.device, dtype=torch.float32 if out_f32 else x.dtype)
    res2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
    flags = (GEMM_BIAS if lw.bias is not None else 0) | (GEMM_RESIDUAL if residual is not None else 0) | \
            (GEMM_SWIGLU if swiglu else 0) | (GEMM_OUT_F32 if out_f32 else 0)
    if lw.kind == "fp4" and _kernel_tensors(lw)[2]:
        flags |= GEMM_FP4_F16W
    bias = lw.bias
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    if a8:
        _linear_i8(x2, lw, out, bias, res2, flags, pre)
        return out.reshape(*lead, n_out)
    if lw.kind == "fp8" and FP8_NATIVE and M <= 128 and x2.stride(0) % 4 == 0:
        _linear_fp8_native(x2, lw, out, bias, res2, flags, pre)
        return out.reshape(*lead, n_out)
    if lw.kind == "fp8" and FP8_NATIVE:
        from .quant import fake_quant_act_fp8

        if not (pre is not None and pre[0] == 4):
            x2 = fake_quant_act_fp8(x2)      # same activation rounding as the e4m3 x e4m3 path used for small batches
    elif uses_int_a8(lw):
        if not (pre is not None and pre[0] == 3):
            x2 = round_act(x2, 0)            # same activation rounding as the int8 x int8 path used for small batches
    lib = _lib.kernels()
    group = -1 if (lw.kind == "int8" and lw.signed) else (lw.group or 0)      # -1: int8 bytes hold q - 128
    for m0 in range(0, M, 256):
        m1 = min(M, m0 + 256)
        rc = lib.fb_gemm_quant(_ptr(x2[m0:m1]), _ptr(lw.w), _ptr(scale), _ptr(zero), _ptr(out[m0:m1]), _ptr(bias),
                               _ptr(res2[m0:m1]) if res2 is not None else _ptr(None), m1 - m0, N, K, x2.stride(0), out.stride(0),
                               res2.stride(0) if res2 is not None else 0, dtype_code(x.dtype), _QMODE[lw.kind], group, flags, 0,
                               _stream())
        _lib.check(rc, "fb_gemm_quant")
    return out.reshape(*lead, n_out)
