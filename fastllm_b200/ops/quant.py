"""Weight quantisation formats and the ``LinearWeight`` holder that dispatches a linear layer by format.

Formats (numerics follow the reference quantiser, include/fastllm.h:239-306 and
src/fastllm.cpp:1033-1145, 1311-1577):

* ``int8``   per-output-channel asymmetric: ``scale = (max-min)/255``, ``zero = round(-min/scale)``,
             ``w ~ scale * (q - zero)``, q stored as uint8.
* ``int4g``  group-wise asymmetric 4 bit (group 128 by default): per (row, group) ``min`` and
             ``scale = (max-min)/15``, ``w ~ min + scale * q``; two values per byte, FIRST value in the
             HIGH nibble.
* ``fp8``    FP8-E4M3 with one fp32 scale per 128x128 weight block (``weight_scale_inv`` convention of
             block-scaled checkpoints): ``w ~ fp8 * scale``.
* ``dense``  fp16 / bf16.
"""
from __future__ import annotations

import torch

from . import basic as B

FP8_MAX = 448.0


# ---------------------------------------------------------------------------------------------------
# quantisers (pure torch; run on whatever device the weight lives on)
# ---------------------------------------------------------------------------------------------------
def quantize_int8(w: torch.Tensor):
    wf = w.float()
    mn = wf.amin(dim=1, keepdim=True).clamp(max=0.0)
    mx = wf.amax(dim=1, keepdim=True).clamp(min=0.0)
    scale = ((mx - mn) / 255.0).clamp(min=1e-12)
    zero = torch.round(-mn / scale).clamp(0, 255)
    q = torch.round(wf / scale + zero).clamp(0, 255).to(torch.uint8)
    return q, scale.squeeze(1), zero.squeeze(1)


def dequantize_int8(q, scale, zero, dtype):
    return ((q.float() - zero[:, None]) * scale[:, None]).to(dtype)


def quantize_int4g(w: torch.Tensor, group: int = 128):
    """Group-wise asymmetric 4-bit: ``w = min + scale * q``, q in 0..15.  Groups whose values already lie on a 16-point grid
    (weights that come out of a 4-bit checkpoint, e.g. AWQ ``(q - zero) * scale`` kept in fp32) get that grid back exactly --
    its step is found from the smallest gap between the group's distinct values -- instead of a new min / max grid."""
    n, k = w.shape
    if k % group != 0:
        raise ValueError(f"in-features {k} not divisible by group {group}")
    wf = w.float().reshape(n, k // group, group)
    mn = wf.amin(dim=2, keepdim=True)
    mx = wf.amax(dim=2, keepdim=True)
    scale = ((mx - mn) / 15.0).clamp(min=1e-12)
    if w.dtype == torch.float32:
        rng = (mx - mn).clamp(min=1e-30)
        srt = wf.sort(dim=2).values
        gap = srt[..., 1:] - srt[..., :-1]
        gmin = torch.where(gap > rng * 1e-4, gap, torch.full_like(gap, float("inf"))).amin(dim=2, keepdim=True)
        k0 = (wf - mn) / scale
        found = (k0 - k0.round()).abs().amax(dim=2, keepdim=True) < 2e-3          # the min / max grid is already exact
        for m_ in (1, 2, 3, 4, 5, 6, 7):        # the smallest gap is m steps when neighbouring codes are unused
            s_ = gmin / m_
            kk = (wf - mn) / s_
            ok = torch.isfinite(s_) & ((kk - kk.round()).abs().amax(dim=2, keepdim=True) < 2e-3) & (kk.amax(dim=2, keepdim=True) < 15.5) & ~found
            scale = torch.where(ok, s_, scale)
            found |= ok
    q = torch.round((wf - mn) / scale).clamp(0, 15).to(torch.uint8).reshape(n, k)
    packed = (q[:, 0::2] << 4) | q[:, 1::2]
    return packed.contiguous(), scale.squeeze(2).contiguous(), mn.squeeze(2).contiguous()


def dequantize_int4g(packed, scale, mn, dtype, group: int = 128):
    n, kh = packed.shape
    q = torch.stack([(packed >> 4) & 0xF, packed & 0xF], dim=2).reshape(n, kh * 2).float()
    q = q.reshape(n, -1, group)
    return (q * scale[:, :, None] + mn[:, :, None]).reshape(n, kh * 2).to(dtype)


def quantize_fp8_block(w: torch.Tensor, block: int = 128):
    n, k = w.shape
    nb, kb = (n + block - 1) // block, (k + block - 1) // block
    wf = torch.zeros((nb * block, kb * block), dtype=torch.float32, device=w.device)
    wf[:n, :k] = w.float()
    t = wf.reshape(nb, block, kb, block)
    amax = t.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale = amax / FP8_MAX
    q = (t / scale[:, None, :, None]).reshape(nb * block, kb * block)[:n, :k].to(torch.float8_e4m3fn)
    return q.contiguous(), scale.contiguous()


def dequantize_fp8_block(q, scale, dtype, block: int = 128):
    n, k = q.shape
    s = scale.repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return (q.float() * s).to(dtype)


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _fp4_codes(v: torch.Tensor) -> torch.Tensor:
    """Round fp32 values (already divided by their block scale) to e2m1 codes 0..15 (sign in bit 3), nearest value, ties to
    the even code."""
    grid = torch.tensor(_E2M1, dtype=torch.float32, device=v.device)
    a = v.abs().clamp(max=6.0)
    d = (a[..., None] - grid).abs()
    code = d.argmin(dim=-1)
    # ties: argmin takes the lower code; move to the upper one when that one is even
    up = (code + 1).clamp(max=7)
    tie = (d.gather(-1, up[..., None])[..., 0] == d.gather(-1, code[..., None])[..., 0]) & (up != code) & (up % 2 == 0)
    code = torch.where(tie, up, code)
    return (code | ((v < 0).long() << 3)).to(torch.uint8)


def quantize_fp4(w: torch.Tensor, block: int = 16):
    """Dense ``[N, K]`` -> (packed uint8 ``[N, K/2]``, low nibble = even element; bf16 block scales ``[N, K/block]``; fp32
    per-tensor factor ``[1]`` or None).  ``block`` 16: NVFP4 -- e4m3-valued block scales under one per-tensor factor
    (amax / (448 * 6)); ``block`` 32: MXFP4 -- power-of-two block scales (the reference's NVFP4_BLOCK_16 / MXFP4 types,
    include/fastllm.h:308-339)."""
    N, K = w.shape
    wf = w.float().reshape(N, K // block, block)
    amax = wf.abs().amax(-1)
    if block == 16:
        g = (wf.abs().max() / (448.0 * 6.0)).clamp(min=1e-30)
        sc = (amax / 6.0 / g).to(torch.float8_e4m3fn).float().clamp(min=2.0 ** -9)
        eff = sc * g
        gl = g.reshape(1).float()
    else:
        sc = torch.exp2(torch.ceil(torch.log2((amax / 6.0).clamp(min=2.0 ** -126))))
        eff, gl = sc, None
    codes = _fp4_codes(wf / eff[..., None]).reshape(N, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, sc.to(torch.bfloat16).contiguous(), gl


def dequantize_fp4(packed, scale, glob, dtype, block: int = 16):
    lut = torch.tensor(_E2M1 + tuple(-x for x in _E2M1), dtype=torch.float32, device=packed.device)
    vals = torch.stack([lut[(packed & 0x0F).long()], lut[(packed >> 4).long()]], dim=-1).reshape(packed.shape[0], -1)
    out = vals.reshape(packed.shape[0], -1, block) * scale.float()[..., None]
    if glob is not None:
        out = out * glob.float().reshape(-1)[0]
    return out.reshape(packed.shape[0], -1).to(dtype)


DEQUANT_KERNEL = __import__("os").environ.get("FB_DEQUANT_KERNEL", "1") != "0"


def fake_quant_act_fp8(x: torch.Tensor) -> torch.Tensor:
    """Round activations to e4m3 per (token, 128-wide k block) and return them in their own dtype.  FP8 layers use the
    tensor core's e4m3 x e4m3 path for decode-sized batches; larger batches go through 16-bit GEMMs and apply this rounding
    first, so a request sees the same activation numerics whatever batch it is scheduled in."""
    K = x.shape[-1]
    if K % 128 != 0:
        return x
    if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16):
        from . import quant_gemm

        return quant_gemm.round_act(x, 1)
    xb = x.float().reshape(-1, K // 128, 128)
    sc = xb.abs().amax(-1, keepdim=True).clamp(min=1e-12) / FP8_MAX
    return ((xb / sc).to(torch.float8_e4m3fn).float() * sc).reshape(x.shape).to(x.dtype)


def fake_quant_act_i8(x: torch.Tensor) -> torch.Tensor:
    """Round activations to int8 per (token, 128-wide k block); see ``fake_quant_act_fp8``."""
    K = x.shape[-1]
    if K % 128 != 0:
        return x
    if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16):
        from . import quant_gemm

        return quant_gemm.round_act(x, 0)
    xb = x.float().reshape(-1, K // 128, 128)
    sc = xb.abs().amax(-1, keepdim=True).clamp(min=1e-12) / 127.0
    return (torch.round(xb / sc).clamp(-127, 127) * sc).reshape(x.shape).to(x.dtype)


def normalize_wdtype(name: str | None) -> tuple[str, int]:
    """Map CLI dtype names (``--dtype`` / ``--moe_dtype``) to (kind, group)."""
    if name is None:
        return "dense", 0
    n = str(name).lower()
    if n in ("auto", "float16", "fp16", "half", "bfloat16", "bf16", "float32", "fp32", "dense"):
        return "dense", 0
    if n in ("int8",):
        return "int8", 0
    if n.startswith("int4g"):
        g = n[5:]
        return "int4g", int(g) if g else 128
    if n in ("int4", "int4_nozero", "int4nozero", "int4_channel"):
        return "int4g", -1              # one (scale, minimum) pair per output channel: the group is the whole row
    if n in ("fp8", "fp8_e4m3", "float8", "fp8_block128"):
        return "fp8", 128
    if n in ("nvfp4", "fp4", "fp4_e2m1", "nvfp4_block16"):
        return "fp4", 16
    if n in ("mxfp4", "nvfp4_block32_e8m0", "fp4_block32"):
        return "fp4", 32
    raise ValueError(f"unsupported weight dtype '{name}'")


# ---------------------------------------------------------------------------------------------------
class LinearWeight:
    """Weight (+ optional bias) of one linear layer in one of the storage formats above."""

    __slots__ = ("kind", "w", "scale", "zero", "bias", "group", "n", "k", "interleaved", "dtype", "_dq", "signed", "_a8", "adapters")
    active_adapter: str | None = None       # name of the run-time low-rank adapter applied by every weight that carries it

    def __init__(self, kind, w, scale=None, zero=None, bias=None, group=0, dtype=torch.bfloat16, interleaved=False):
        self.kind, self.w, self.scale, self.zero, self.bias, self.group = kind, w, scale, zero, bias, group
        self.n = w.shape[0]
        self.k = w.shape[1] * (2 if kind in ("int4g", "fp4") else 1)
        self.dtype = dtype
        self.interleaved = interleaved      # gate/up rows interleaved per 128-row tile for the SwiGLU epilogue
        self._dq = None
        self._a8 = None
        self.adapters = None                # name -> (A [r, K], B [N, r]) run-time low-rank deltas (fastllm_b200/lora.py)
        self.signed = False                 # int8 only: bytes hold q - 128 (the integer tensor-core path's operand form)

    @staticmethod
    def from_dense(w: torch.Tensor, wdtype: str = "dense", bias=None, interleaved=False, act_dtype=None) -> "LinearWeight":
        kind, group = normalize_wdtype(wdtype)
        act_dtype = act_dtype or (w.dtype if w.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16)
        if kind == "dense":
            return LinearWeight("dense", w.contiguous(), bias=bias, dtype=w.dtype, interleaved=interleaved)
        if kind == "int8":
            q, s, z = quantize_int8(w)
            lw = LinearWeight("int8", q, s, z, bias, dtype=act_dtype, interleaved=interleaved)
            if q.is_cuda:
                from . import quant_gemm

                quant_gemm.prepare(lw)          # operand form of the integer path, before any CUDA graph is captured
            return lw
        if kind == "int4g":
            if group < 0:                # per-channel: the reference's INT4_NOZERO (src/fastllm.cpp, PerChannelQuantizationMultiThread)
                group = w.shape[1]
            if w.shape[1] % group != 0:
                return LinearWeight("dense", w.contiguous(), bias=bias, dtype=w.dtype, interleaved=interleaved)
            q, s, mn = quantize_int4g(w, group)
            return LinearWeight("int4g", q, s, mn, bias, group, act_dtype, interleaved)
        if kind == "fp4":
            if w.shape[1] % 64 != 0:
                return LinearWeight("dense", w.contiguous(), bias=bias, dtype=w.dtype, interleaved=interleaved)
            q, s, gl = quantize_fp4(w, group)
            return LinearWeight("fp4", q, s, gl, bias, group, act_dtype, interleaved)
        q, s = quantize_fp8_block(w, 128)
        return LinearWeight("fp8", q, s, None, bias, 128, act_dtype, interleaved)

    def dequant(self, dtype=None) -> torch.Tensor:
        dtype = dtype or self.dtype
        if self.kind == "dense":
            return self.w if self.w.dtype == dtype else self.w.to(dtype)
        if self.w.is_cuda and dtype in (torch.float16, torch.bfloat16) and DEQUANT_KERNEL and self.k % 8 == 0:
            # one pass over the packed weight (prefill-sized batches run the dense GEMM on the result)
            from . import _lib
            from .basic import _ptr, _stream, dtype_code

            mode = {"int8": 1, "int4g": 2, "fp8": 3, "fp4": 4}[self.kind]
            ok = not ((mode in (2, 4)) and (self.group % 8 != 0 or self.k % self.group != 0))
            if ok:
                out = torch.empty((self.n, self.k), device=self.w.device, dtype=dtype)
                sc = self.scale.to(torch.bfloat16) if mode == 4 else self.scale.float()
                ze = self.zero.float() if self.zero is not None else None
                rc = _lib.kernels().fb_dequant_weight(_ptr(self.w), _ptr(sc.contiguous()), _ptr(ze.contiguous() if ze is not None else None),
                                                      _ptr(out), self.n, self.k, self.k, mode, int(self.group or 0),
                                                      1 if (mode == 1 and self.signed) else 0, dtype_code(dtype), _stream())
                _lib.check(rc, "fb_dequant_weight")
                return out
        if self.kind == "int8":
            if self.signed:
                return ((self.w.view(torch.int8).float() + 128.0 - self.zero[:, None]) * self.scale[:, None]).to(dtype)
            return dequantize_int8(self.w, self.scale, self.zero, dtype)
        if self.kind == "int4g":
            return dequantize_int4g(self.w, self.scale, self.zero, dtype, self.group)
        if self.kind == "fp4":
            return dequantize_fp4(self.w, self.scale, self.zero, dtype, self.group)
        return dequantize_fp8_block(self.w, self.scale, dtype, self.group)

    def nbytes(self) -> int:
        n = self.w.numel() * self.w.element_size()
        for t in (self.scale, self.zero, self.bias):
            if t is not None:
                n += t.numel() * t.element_size()
        return n

    def __call__(self, x, residual=None, swiglu=False, out_f32=False):
        if LinearWeight.active_adapter is not None and self.adapters and LinearWeight.active_adapter in self.adapters:
            # y = W x + B (A x): the delta goes in before the activation, so the fused epilogues are applied afterwards
            a, b = self.adapters[LinearWeight.active_adapter]
            y = self._base(x, None, False, False)
            y = y + B.linear(B.linear(x, a.to(x.dtype)), b.to(x.dtype))
            if swiglu:
                t = y.float()
                if self.interleaved:
                    t = t.reshape(*t.shape[:-1], t.shape[-1] // 128, 2, 64)
                    g, u = t[..., 0, :], t[..., 1, :]
                else:
                    g, u = t.chunk(2, dim=-1)
                y = (torch.nn.functional.silu(g) * u).reshape(*y.shape[:-1], y.shape[-1] // 2).to(y.dtype)
            if residual is not None:
                y = y + residual
            return y.float() if out_f32 else y
        return self._base(x, residual, swiglu, out_f32)

    def _base(self, x, residual=None, swiglu=False, out_f32=False):
        if self.kind == "dense":
            w = self.w
            if w.dtype != x.dtype:
                w = w.to(x.dtype)
            return B.linear(x, w, self.bias, residual, swiglu, self.interleaved, out_f32)
        if B.cpu_native(x) and self.kind in ("int8", "int4g"):
            y = B.cpu.linear(x, self.w, self.bias, self.kind, self.scale, self.zero, self.group)
            return B.cpu_linear_epilogue(y, residual, swiglu, self.interleaved)
        if x.is_cuda:
            from . import quant_gemm

            y = quant_gemm.linear_quant(x, self, residual, swiglu, out_f32)
            if y is not None:
                return y
            pre = getattr(x, "fb_quant", None)
            if self.kind == "fp8" and quant_gemm.FP8_NATIVE:
                if not (pre is not None and pre[0] == 4):
                    x = fake_quant_act_fp8(x)
            elif quant_gemm.uses_int_a8(self):
                if not (pre is not None and pre[0] == 3):
                    x = fake_quant_act_i8(x)
        return B.linear(x, self.dequant(x.dtype), self.bias, residual, swiglu, self.interleaved, out_f32)
