"""Weight-only-quantised and block-scaled FP8 GEMM dispatch (CUDA).

``linear_quant`` returns ``None`` when no fused kernel covers the (format, shape) pair; the caller then
dequantises and runs the dense tcgen05 GEMM.
"""
from __future__ import annotations


def linear_quant(x, lw, residual=None, swiglu=False, out_f32=False):
    return None
