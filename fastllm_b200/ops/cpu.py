"""Native CPU backend (``lib/libfb_cpu.so``): C++ AVX2 / AVX-512 kernels behind a persistent thread pool.

This is the executor for ``--device cpu`` (fp32 activations; fp32 / bf16 / fp16 / int8 / int4-group weights used in place,
without de-quantising to a scratch copy) and the oracle the CUDA kernels are compared with.  It plays the role of the
reference's ``cpu`` device (src/devices/cpu/cpudevice.cpp:284-394, Linear kernels src/devices/cpu/linear.cpp:412-1278).
``FB_CPU_NATIVE=0`` makes every operator fall back to its plain PyTorch definition.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

_LIB = None
_PATH = Path(__file__).resolve().parent.parent / "lib" / "libfb_cpu.so"
P, I, F = c_void_p, c_int, c_float

_SIGS = {
    "fbcpu_get_threads": ([], I), "fbcpu_set_threads": ([I], None), "fbcpu_isa": ([], I),
    "fbcpu_set_accel": ([I], I), "fbcpu_get_accel": ([], I), "fbcpu_accel_caps": ([], I),
    "fbcpu_linear": ([P, I, P, I, P, P, I, P, P, I, I, I, I], I),
    "fbcpu_rmsnorm": ([P, I, P, P, I, I, I, F, F], None),
    "fbcpu_layernorm": ([P, I, P, P, P, I, I, I, F], None),
    "fbcpu_swiglu": ([P, I, P, I, I, I], None),
    "fbcpu_activation": ([P, c_longlong, I], None),
    "fbcpu_softmax": ([P, I, I, I], None),
    "fbcpu_rope": ([P, I, P, P, P, I, I, I, I, I], None),
    "fbcpu_kv_append": ([P, I, P, I, P, P, P, I, I], None),
    "fbcpu_attention_paged": ([P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, P], I),
    "fbcpu_embedding": ([P, P, P, I, I, F], None),
    "fbcpu_select_expert": ([P, P, I, I, I, I, I, F, P, P], None),
}


def available() -> bool:
    return os.environ.get("FB_CPU_NATIVE", "1") != "0" and _PATH.exists()


def lib():
    global _LIB
    if _LIB is None:
        if not _PATH.exists():
            raise RuntimeError(f"{_PATH} is missing: run `python -m fastllm_b200.build`")
        L = ctypes.CDLL(str(_PATH))
        for name, (args, res) in _SIGS.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = res
        n = os.environ.get("FB_CPU_THREADS")
        if n:
            L.fbcpu_set_threads(int(n))
        acc = os.environ.get("FB_CPU_ACCEL")
        if acc:
            L.fbcpu_set_accel(int(acc))
        _LIB = L
    return _LIB


ACCEL_VNNI, ACCEL_BF16, ACCEL_AMX = 1, 2, 4


def accel_caps() -> int:
    """Which reduced-precision-activation instruction sets this CPU offers (bits ``ACCEL_VNNI | ACCEL_BF16 | ACCEL_AMX``)."""
    return int(lib().fbcpu_accel_caps())


def set_accel(flags: int) -> int:
    """Switch the VNNI (int8 / int4-group weights x int8 activations), AVX-512 BF16 and AMX kernels on or off; they round the
    activations (int8 per token and 128-wide block, or bf16) where the default kernels keep them fp32.  Returns the bits in
    effect (requested AND available).  ``FB_CPU_ACCEL=7`` in the environment does the same at load."""
    return int(lib().fbcpu_set_accel(int(flags)))


def get_accel() -> int:
    return int(lib().fbcpu_get_accel())


def set_threads(n: int) -> None:
    lib().fbcpu_set_threads(int(n))


def get_threads() -> int:
    return lib().fbcpu_get_threads()


def isa() -> str:
    """Instruction set the dispatcher picked on this machine."""
    return {256: "avx2", 512: "avx512"}.get(int(lib().fbcpu_isa()), "unknown")


def _p(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _f32c(t):
    if t is None:
        return None
    if t.dtype != torch.float32:
        t = t.float()
    return t if t.is_contiguous() else t.contiguous()


ACT = {"silu": 0, "gelu": 1, "gelu_new": 2, "gelu_pytorch_tanh": 2, "relu": 3, "sigmoid": 4, "tanh": 5, "exp": 6}
_WTYPE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def linear(x: torch.Tensor, w: torch.Tensor, bias=None, kind: str = "dense", scale=None, zero=None, group: int = 0) -> torch.Tensor:
    """``x @ W.T + bias`` in fp32.  ``kind``: dense (w fp32/bf16/fp16), int8 (uint8 + per-row scale/zero),
    int4g (packed nibbles + per-(row, group) scale/min)."""
    lead = x.shape[:-1]
    x2 = _f32c(x.reshape(-1, x.shape[-1]))
    M, K = x2.shape
    if kind == "dense":
        if w.dtype not in _WTYPE:
            w = w.float()
        wt = _WTYPE[w.dtype]
    elif kind == "int8":
        wt = 3
    elif kind == "int4g":
        wt = 4
    else:
        raise ValueError(f"unsupported CPU weight kind {kind}")
    w = w if w.is_contiguous() else w.contiguous()
    N = w.shape[0]
    y = torch.empty((M, N), dtype=torch.float32)
    sc, zr, b = _f32c(scale), _f32c(zero), _f32c(bias)
    rc = lib().fbcpu_linear(_p(x2), x2.stride(0), _p(w), wt, _p(sc), _p(zr), int(group), _p(b), _p(y), N, M, N, K)
    if rc != 0:
        raise RuntimeError(f"fbcpu_linear: unsupported shape (K={K}, group={group})")
    return y.reshape(*lead, N)


def rmsnorm(x, w, eps, unit_offset=0.0):
    x2 = _f32c(x.reshape(-1, x.shape[-1]))
    y = torch.empty_like(x2)
    lib().fbcpu_rmsnorm(_p(x2), x2.stride(0), _p(_f32c(w)), _p(y), y.stride(0), x2.shape[0], x2.shape[1], float(eps), float(unit_offset))
    return y.reshape(x.shape)


def layernorm(x, w, b, eps):
    x2 = _f32c(x.reshape(-1, x.shape[-1]))
    y = torch.empty_like(x2)
    lib().fbcpu_layernorm(_p(x2), x2.stride(0), _p(_f32c(w)), _p(_f32c(b)), _p(y), y.stride(0), x2.shape[0], x2.shape[1], float(eps))
    return y.reshape(x.shape)


def swiglu(gu):
    """``silu(gu[..., :I]) * gu[..., I:]``."""
    g2 = _f32c(gu.reshape(-1, gu.shape[-1]))
    inter = g2.shape[1] // 2
    out = torch.empty((g2.shape[0], inter), dtype=torch.float32)
    lib().fbcpu_swiglu(_p(g2), g2.stride(0), _p(out), inter, g2.shape[0], inter)
    return out.reshape(*gu.shape[:-1], inter)


def activation(x, name: str):
    y = _f32c(x).clone()
    lib().fbcpu_activation(_p(y), y.numel(), ACT[name])
    return y


def softmax(x):
    y = _f32c(x.reshape(-1, x.shape[-1])).clone()
    lib().fbcpu_softmax(_p(y), y.stride(0), y.shape[0], y.shape[1])
    return y.reshape(x.shape)


def rope_(x, positions, cos, sin, heads, head_dim, rot, mode):
    """In-place rotary embedding of ``x [T, heads*head_dim]`` (fp32, contiguous).  mode: 1 neox, 2 interleaved."""
    assert x.dtype == torch.float32 and x.stride(-1) == 1
    pos = positions.to(torch.int32).contiguous()
    lib().fbcpu_rope(_p(x), x.stride(0), _p(pos), _p(_f32c(cos)), _p(_f32c(sin)), x.shape[0], heads, head_dim, rot, mode)
    return x


def kv_append(k, v, slots, k_pool, v_pool):
    """k, v: ``[T, Hkv*D]`` fp32 (unit inner stride); pools ``[pages, page_len, Hkv, D]`` fp32."""
    assert k.stride(-1) == 1 and v.stride(-1) == 1 and k_pool.dtype == torch.float32 and k.dtype == v.dtype == torch.float32
    s = slots.to(torch.int32).contiguous()
    lib().fbcpu_kv_append(_p(k), k.stride(0), _p(v), v.stride(0), _p(s), _p(k_pool), _p(v_pool), k.shape[0], k.shape[1])


def attention_paged(q, k_pool, v_pool, page_table, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim, window=0, sinks=None):
    q2 = _f32c(q)
    out = torch.empty_like(q2)
    pt = page_table.to(torch.int32).contiguous()
    kl = kv_lens.to(torch.int32).contiguous()
    cq = cu_q.to(torch.int32).contiguous()
    rc = lib().fbcpu_attention_paged(_p(q2), q2.stride(0), _p(k_pool), _p(v_pool), _p(pt), pt.shape[1], _p(kl), _p(cq), _p(out),
                                     out.stride(0), kl.numel(), num_q_heads, num_kv_heads, head_dim, k_pool.shape[1], float(scale),
                                     int(window or 0), _p(_f32c(sinks)))
    if rc != 0:
        raise RuntimeError("fbcpu_attention_paged: unsupported head configuration")
    return out


def embedding(table, ids, scale=1.0):
    t = _f32c(table)
    i = ids.to(torch.int32).contiguous().reshape(-1)
    out = torch.empty((i.numel(), t.shape[1]), dtype=torch.float32)
    lib().fbcpu_embedding(_p(t), _p(i), _p(out), i.numel(), t.shape[1], float(scale))
    return out


def select_expert(logits, bias, topk, mode="softmax", renorm=True, route_scale=1.0):
    """Returns (indices int32 ``[T, topk]``, weights fp32 ``[T, topk]``); reference: src/devices/cpu/cpudevice.cpp:8885-8955."""
    lg = _f32c(logits.reshape(-1, logits.shape[-1]))
    T, E = lg.shape
    idx = torch.empty((T, topk), dtype=torch.int32)
    w = torch.empty((T, topk), dtype=torch.float32)
    lib().fbcpu_select_expert(_p(lg), _p(_f32c(bias)), T, E, topk, {"softmax": 0, "sigmoid": 1, "none": 2}[mode], int(bool(renorm)),
                              float(route_scale), _p(idx), _p(w))
    return idx, w
