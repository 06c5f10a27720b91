"""RoPE tables, fused QKV post-processing and paged attention.

KV cache layout is ``[num_pages, page_len, kv_heads, head_dim]`` per layer for K and for V (the
reference's page pool shape, include/fastllm.h:643-698, page_len 128); a token's ``slot`` is
``page * page_len + offset``.

CUDA tensors run the sm_100a kernels (``attn_decode.cu``, ``attn_prefill.cu``, ``elementwise.cu``);
CPU tensors run the PyTorch definitions below, which double as the test oracle.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _lib, cpu
from .basic import _ptr, _stream, cpu_native, dtype_code

PAGE_LEN = 128
ROPE_NONE, ROPE_NEOX, ROPE_INTERLEAVED = 0, 1, 2
# Merging the split-KV partials inside the attention kernel (last-arriving CTA) was measured slower than the separate combine
# kernel (107 us vs 61 us per layer at 64 x 1150 tokens: the arrival atomic sits on every work item's critical path), so it
# stays off unless requested.
_FUSED_COMBINE = __import__("os").environ.get("FB_ATTN_FUSED_COMBINE", "0") == "1"


# ---------------------------------------------------------------------------------------------------
# RoPE tables: all frequency-scaling variants reduce to a (cos, sin) table indexed by position.
# Reference kernels: RopeEncoding / Llama3RopeEncoding / YarnRopeEncoding
# (src/devices/cuda/fastllm-cuda.cu:2340, 2510, 2417) and the linear / dynamic-NTK handling in
# src/models/llama.cpp:82-93.
# ---------------------------------------------------------------------------------------------------
def _yarn_find_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def rope_inv_freq(rot_dim: int, base: float, scaling: dict | None = None, max_pos: int = 0):
    """Return (inv_freq [rot_dim/2] float64 tensor, attention scale factor)."""
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    mscale = 1.0
    if not scaling:
        return inv, mscale
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    factor = float(scaling.get("factor", 1.0))
    if kind == "linear":
        inv = inv / factor
    elif kind == "dynamic":
        orig = int(scaling.get("original_max_position_embeddings", max_pos or 2048))
        if max_pos > orig:
            nb = base * ((factor * max_pos / orig) - (factor - 1)) ** (rot_dim / (rot_dim - 2))
            inv = 1.0 / (nb ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    elif kind == "llama3":
        lo = float(scaling.get("low_freq_factor", 1.0))
        hi = float(scaling.get("high_freq_factor", 4.0))
        orig = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        smooth = (orig / wavelen - lo) / (hi - lo)
        scaled = torch.where(wavelen > orig / lo, inv / factor, inv)
        mid = (wavelen <= orig / lo) & (wavelen >= orig / hi)
        inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
    elif kind == "yarn":
        orig = int(scaling.get("original_max_position_embeddings", 4096))
        beta_fast = float(scaling.get("beta_fast", 32))
        beta_slow = float(scaling.get("beta_slow", 1))
        low, high = _yarn_find_dim(beta_fast, rot_dim, base, orig), _yarn_find_dim(beta_slow, rot_dim, base, orig)
        if scaling.get("truncate", True):          # gpt-oss keeps the fractional correction range
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, rot_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rot_dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        inv_mask = 1 - ramp
        inv = inv / factor * (1 - inv_mask) + inv * inv_mask
        ms = float(scaling.get("mscale", 1.0))
        ms_all = float(scaling.get("mscale_all_dim", 0.0))

        def get_mscale(scale, m):
            return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

        if "attention_factor" in scaling and scaling["attention_factor"] is not None:
            mscale = float(scaling["attention_factor"])
        elif ms_all:
            mscale = get_mscale(factor, ms) / get_mscale(factor, ms_all)
        else:
            mscale = get_mscale(factor, 1.0)
    return inv, mscale


def build_rope_tables(rot_dim: int, max_pos: int, base: float, scaling: dict | None = None, device="cpu"):
    """(cos, sin) fp32 tables ``[max_pos, rot_dim/2]``; the yarn magnitude factor is folded in."""
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type", "default"))
    if kind in ("longrope", "su") and scaling.get("short_factor") is not None:
        # Phi-3 / MiniCPM3 long-context tables: per-dimension divisors, the short set for positions inside the original window
        # and the long set beyond it; rows scaled by sqrt(1 + ln(extension) / ln(original window))
        orig = int(scaling.get("original_max_position_embeddings", max_pos) or max_pos)
        inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
        short = torch.tensor(scaling["short_factor"], dtype=torch.float64)[: rot_dim // 2]
        long = torch.tensor(scaling.get("long_factor", scaling["short_factor"]), dtype=torch.float64)[: rot_dim // 2]
        ext = float(scaling.get("factor") or (max_pos / orig if orig else 1.0))
        ms = scaling.get("attention_factor")
        ms = float(ms) if ms is not None else (1.0 if ext <= 1.0 else math.sqrt(1.0 + math.log(ext) / math.log(orig)))
        pos = torch.arange(max_pos, dtype=torch.float64)[:, None]
        ang = torch.where(pos < orig, pos * (inv / short)[None, :], pos * (inv / long)[None, :])
        return (ang.cos() * ms).float().to(device).contiguous(), (ang.sin() * ms).float().to(device).contiguous()
    inv, mscale = rope_inv_freq(rot_dim, base, scaling, max_pos)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return (ang.cos() * mscale).float().to(device).contiguous(), (ang.sin() * mscale).float().to(device).contiguous()


def apply_rope_ref(x, positions, cos, sin, mode, rot):
    """x: [T, H, D]; rotates the first ``rot`` dims. fp32 math, returns x.dtype."""
    if mode == ROPE_NONE:
        return x
    xf = x.float()
    c = cos[positions.long()][:, None, :]
    s = sin[positions.long()][:, None, :]
    xr, rest = xf[..., :rot], xf[..., rot:]
    if mode == ROPE_NEOX:
        a, b = xr[..., : rot // 2], xr[..., rot // 2:]
        out = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    else:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * c - b * s, a * s + b * c], dim=-1).flatten(-2)
    return torch.cat([out, rest], dim=-1).to(x.dtype)


def _head_norm_ref(x, w, eps, unit_offset):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + unit_offset)).to(x.dtype)


def qkv_post(qkv, positions, slots, k_pool, v_pool, num_q_heads, num_kv_heads, head_dim, cos, sin, rope_mode=ROPE_NEOX,
             rot_dim=None, q_norm_w=None, k_norm_w=None, eps=1e-6, norm_unit_offset=0.0, q_out=None, q8=None):
    """Split packed QKV, per-head RMSNorm on Q/K (optional), RoPE, append K/V to the page pools, return Q.

    e4m3 page pools (CUDA): the rows are appended as e4m3 bytes by the same launch; ``q8`` = two ``[T, Hq * D]`` byte buffers
    that receive the queries as two e4m3 terms (the operand form of the fp8 tensor-core decode attention).

    qkv: ``[T, (Hq + 2 Hkv) * D]``; positions, slots: int32 ``[T]``; pools ``[pages, page_len, Hkv, D]``.
    One launch on CUDA (reference: QKVRMSNormRopeSplitAppendPagedCache, src/devices/cuda/fastllm-cuda.cu:12190).
    """
    T = qkv.shape[0]
    Hq, Hkv, D = num_q_heads, num_kv_heads, head_dim
    rot = rot_dim or D
    if cpu_native(qkv) and k_pool.dtype == torch.float32 and qkv.stride(-1) == 1:
        q = qkv[:, :Hq * D].contiguous()
        k = qkv[:, Hq * D:(Hq + Hkv) * D].contiguous()
        v = qkv[:, (Hq + Hkv) * D:]
        if q_norm_w is not None:
            q = cpu.rmsnorm(q.view(T * Hq, D), q_norm_w, eps, norm_unit_offset).view(T, Hq * D)
        if k_norm_w is not None:
            k = cpu.rmsnorm(k.view(T * Hkv, D), k_norm_w, eps, norm_unit_offset).view(T, Hkv * D)
        if rope_mode != ROPE_NONE:
            cpu.rope_(q, positions, cos, sin, Hq, D, rot, rope_mode)
            cpu.rope_(k, positions, cos, sin, Hkv, D, rot, rope_mode)
        cpu.kv_append(k, v, slots, k_pool, v_pool)
        return q
    if not qkv.is_cuda:
        q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
        q, k, v = q.reshape(T, Hq, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D)
        if q_norm_w is not None:
            q = _head_norm_ref(q, q_norm_w, eps, norm_unit_offset)
        if k_norm_w is not None:
            k = _head_norm_ref(k, k_norm_w, eps, norm_unit_offset)
        q = apply_rope_ref(q, positions, cos, sin, rope_mode, rot)
        k = apply_rope_ref(k, positions, cos, sin, rope_mode, rot)
        valid = slots >= 0
        kp = k_pool.view(-1, Hkv, D)
        vp = v_pool.view(-1, Hkv, D)
        kp[slots[valid].long()] = k[valid].to(kp.dtype)
        vp[slots[valid].long()] = v[valid].to(vp.dtype)
        return q.reshape(T, Hq * D)
    if q_out is None:
        q_out = torch.empty((T, Hq * D), device=qkv.device, dtype=qkv.dtype)
    if k_pool.dtype == torch.float8_e4m3fn:
        rc = _lib.kernels().fb_qkv_post_kv8(_ptr(qkv), qkv.stride(0), _ptr(q_out), q_out.stride(0), _ptr(k_pool), _ptr(v_pool),
                                            _ptr(positions), _ptr(slots), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos), _ptr(sin), T, Hq,
                                            Hkv, D, rot, rope_mode, float(eps), float(norm_unit_offset), dtype_code(qkv.dtype),
                                            _ptr(q8[0] if q8 is not None else None), _ptr(q8[1] if q8 is not None else None), _stream())
        _lib.check(rc, "fb_qkv_post_kv8")
        return q_out
    rc = _lib.kernels().fb_qkv_post(_ptr(qkv), qkv.stride(0), _ptr(q_out), q_out.stride(0), _ptr(k_pool), _ptr(v_pool),
                                    _ptr(positions), _ptr(slots), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos), _ptr(sin), T, Hq,
                                    Hkv, D, rot, rope_mode, float(eps), float(norm_unit_offset), dtype_code(qkv.dtype),
                                    _stream())
    _lib.check(rc, "fb_qkv_post")
    return q_out


_FUSED_QKV = __import__("os").environ.get("FB_FUSED_QKV_POST", "1") == "1"


def mla_post(ckv, q, q_full, lat_pool, positions, slots, norm_w, cos, sin, H, nope, rope, lora, rope_mode, eps):
    """Multi-head latent attention, everything between the projections and the attention in one launch: RMSNorm of the
    latent row and RoPE of the shared key into the cache entry (``slots`` < 0 go to the pool's spare last slot), RoPE of every
    head's rotary query part into ``q_full[..., lora:]``.  ckv ``[T, lora + rope]``, q ``[T, H * (nope + rope)]``,
    q_full ``[T, H, lora + rope]``, lat_pool ``[pages, page_len, 1, lora + rope]``."""
    T = ckv.shape[0]
    flat = lat_pool.view(-1, lora + rope)
    spare = flat.shape[0] - 1
    if ckv.is_cuda and ckv.dtype in (torch.float16, torch.bfloat16) and lat_pool.dtype == ckv.dtype and q.dtype == ckv.dtype \
            and rope_mode in (ROPE_NEOX, ROPE_INTERLEAVED) and ckv.stride(-1) == 1 and q.stride(-1) == 1:
        rc = _lib.kernels().fb_mla_post(_ptr(ckv), ckv.stride(0), _ptr(q), q.stride(0), _ptr(q_full), q_full.stride(0), _ptr(lat_pool),
                                        _ptr(positions), _ptr(slots), _ptr(norm_w), _ptr(cos), _ptr(sin), T, H, nope, rope, lora, rope_mode,
                                        spare, float(eps), dtype_code(ckv.dtype), _stream())
        _lib.check(rc, "fb_mla_post")
        return
    from .basic import rmsnorm

    c_lat = rmsnorm(ckv[:, :lora].contiguous(), norm_w, eps)
    k_pe = apply_rope_ref(ckv[:, lora:].reshape(T, 1, rope), positions, cos, sin, rope_mode, rope)
    qv = q.view(T, H, nope + rope)
    q_full[..., lora:] = apply_rope_ref(qv[..., nope:], positions, cos, sin, rope_mode, rope).to(q_full.dtype)
    entry = torch.cat([c_lat, k_pe.reshape(T, rope)], dim=-1).to(flat.dtype)
    flat.index_copy_(0, torch.where(slots >= 0, slots, spare).long(), entry)


def qkv_proj_post(x, w, positions, slots, k_pool, v_pool, num_q_heads, num_kv_heads, head_dim, cos, sin, rope_mode=ROPE_NEOX,
                  rot_dim=None, q_norm_w=None, k_norm_w=None, eps=1e-6, norm_unit_offset=0.0):
    """QKV projection + ``qkv_post`` in one launch for decode-sized batches: ``w`` is a dense ``LinearWeight`` with
    ``(Hq + 2 Hkv) * 128`` output rows; the per-head norm / RoPE / cache append run as the GEMM's epilogue.  Returns Q
    ``[T, Hq * 128]``, or None when the shape is outside the fused kernel (the caller then runs the two steps)."""
    from .basic import _take_pending_wait
    from .quant import LinearWeight

    Hq, Hkv, D = num_q_heads, num_kv_heads, head_dim
    rot = rot_dim or D
    T = x.shape[0]
    if (not _FUSED_QKV or not x.is_cuda or D != 128 or T > 256 or w.kind != "dense" or LinearWeight.active_adapter is not None
            or x.dtype not in (torch.float16, torch.bfloat16) or w.w.dtype != x.dtype or w.n != (Hq + 2 * Hkv) * D or w.k % 64 != 0
            or rot % 8 != 0 or rot > D or w.n // 128 > 148 or k_pool.dtype != x.dtype or x.stride(-1) != 1
            or (x.data_ptr() & 15) or (x.stride(0) * 2) % 16):
        return None
    q_out = torch.empty((T, Hq * D), device=x.device, dtype=x.dtype)
    pend = _take_pending_wait()
    P = ctypes.c_void_p
    rc = _lib.kernels().fb_gemm_qkv_post(_ptr(x), _ptr(w.w), _ptr(w.bias), T, w.n, w.k, x.stride(0), w.w.stride(0), dtype_code(x.dtype),
                                         P(pend[0]) if pend else P(0), P(pend[1]) if pend else P(0), _ptr(q_out), q_out.stride(0),
                                         _ptr(k_pool), _ptr(v_pool), _ptr(positions), _ptr(slots), _ptr(q_norm_w), _ptr(k_norm_w),
                                         _ptr(cos), _ptr(sin), Hq, Hkv, rot, rope_mode, float(eps), float(norm_unit_offset), _stream())
    if rc == -1:
        if pend is not None:
            pend[2]()
        return None
    _lib.check(rc, "fb_gemm_qkv_post")
    return q_out


# ---------------------------------------------------------------------------------------------------
# paged attention
# ---------------------------------------------------------------------------------------------------
def paged_attention_ref(q, k_pool, v_pool, page_table, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim):
    """Causal attention of packed new tokens against the paged cache (fp32 math).

    q: ``[T, Hq*D]``; request b owns rows ``cu_q[b]:cu_q[b+1]`` whose absolute positions are the last
    ``q_len`` positions of its ``kv_lens[b]`` cached tokens.  Decode is the case q_len == 1.
    """
    Hq, Hkv, D = num_q_heads, num_kv_heads, head_dim
    G = Hq // Hkv
    out = torch.zeros_like(q)
    page_len = k_pool.shape[1]
    cu = cu_q.tolist()
    for b in range(len(cu) - 1):
        q0, q1 = cu[b], cu[b + 1]
        if q1 == q0:
            continue
        L = int(kv_lens[b])
        npg = (L + page_len - 1) // page_len
        pages = page_table[b, :npg].long()
        k = k_pool[pages].reshape(-1, Hkv, D)[:L].float()
        v = v_pool[pages].reshape(-1, Hkv, D)[:L].float()
        qq = q[q0:q1].reshape(q1 - q0, Hkv, G, D).float()
        s = torch.einsum("qhgd,khd->hgqk", qq, k) * scale
        qpos = torch.arange(L - (q1 - q0), L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        s = s.masked_fill(kpos > qpos, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgqk,khd->qhgd", p, v)
        out[q0:q1] = o.reshape(q1 - q0, Hq * D).to(q.dtype)
    return out


def paged_attention_general(q, k_pool, v_pool, page_table, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim,
                            window: int = 0, sinks=None, softcap: float = 0.0):
    """Causal paged attention with the less common options, evaluated with PyTorch ops on any device:
    sliding window (each query sees its last ``window`` positions), a per-head sink logit that only enters the softmax
    denominator, and tanh soft-capping of the logits.  Used by the model families outside the tensor-core kernels' coverage
    (reference: those families run on the old engine's generic Attention op, src/models/gpt_oss.cpp, src/models/gemma4.cpp)."""
    Hq, Hkv, D = num_q_heads, num_kv_heads, head_dim
    G = Hq // Hkv
    out = torch.zeros_like(q)
    page_len = k_pool.shape[1]
    cu = cu_q.tolist()
    lens = kv_lens.tolist()
    for b in range(len(cu) - 1):
        q0, q1 = cu[b], cu[b + 1]
        if q1 == q0:
            continue
        L = int(lens[b])
        npg = (L + page_len - 1) // page_len
        pages = page_table[b, :npg].long()
        k = k_pool[pages].reshape(-1, Hkv, D)[:L].float()
        v = v_pool[pages].reshape(-1, Hkv, D)[:L].float()
        qq = q[q0:q1].reshape(q1 - q0, Hkv, G, D).float()
        s = torch.einsum("qhgd,khd->hgqk", qq, k) * scale
        if softcap:
            s = torch.tanh(s / softcap) * softcap
        qpos = torch.arange(L - (q1 - q0), L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        mask = kpos > qpos
        if window:
            mask = mask | (kpos <= qpos - window)
        s = s.masked_fill(mask, float("-inf"))
        if sinks is not None:
            sk = sinks.float().reshape(Hkv, G, 1, 1).expand(Hkv, G, q1 - q0, 1)
            p = torch.softmax(torch.cat([s, sk], dim=-1), dim=-1)[..., :-1]
        else:
            p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgqk,khd->qhgd", p, v)
        out[q0:q1] = o.reshape(q1 - q0, Hq * D).to(q.dtype)
    return out


class DecodeWorkspace:
    """Device scratch for split-KV decode attention, sized once for (max_batch, max_pages_per_seq)."""

    def __init__(self, max_batch, num_kv_heads, group, max_pages, device, head_dim=128, window: int = 0):
        self.max_batch, self.max_pages = max_batch, max_pages
        self.work = torch.zeros((max_batch * max_pages, 2), device=device, dtype=torch.int32)
        self.n_work = torch.zeros((1,), device=device, dtype=torch.int32)
        # sliding-window layers get their own work list: pages that lie wholly before the window are not visited
        self.window = int(window)
        self.work_w = torch.zeros((max_batch * max_pages, 2), device=device, dtype=torch.int32) if window else None
        self.n_work_w = torch.zeros((1,), device=device, dtype=torch.int32) if window else None
        self.part_o = torch.empty((max_batch * num_kv_heads * max_pages * group * head_dim,), device=device,
                                  dtype=torch.float32)
        self.part_ml = torch.empty((max_batch * num_kv_heads * max_pages * group * 2,), device=device, dtype=torch.float32)
        # arrival counters of the fused combine: zero here, and left at zero by every launch
        self.counters = torch.zeros((max_batch * num_kv_heads,), device=device, dtype=torch.int32)
        self._q8 = None

    def q8_terms(self, width: int):
        """Two ``[max_batch, width]`` byte buffers for the e4m3 terms of the queries (fp8 tensor-core mode of the decode kernel)."""
        if self._q8 is None or self._q8[0].shape[1] != width:
            dev = self.work.device
            self._q8 = (torch.empty((self.max_batch, width), device=dev, dtype=torch.uint8),
                        torch.empty((self.max_batch, width), device=dev, dtype=torch.uint8))
        return self._q8

    def plan(self, seq_lens: torch.Tensor):
        """Flatten (request, page) work items for the current sequence lengths (one tiny launch per step)."""
        B = seq_lens.numel()
        rc = _lib.kernels().fb_attn_decode_plan(_ptr(seq_lens), B, _ptr(self.work), _ptr(self.n_work),
                                                self.work.shape[0], _stream())
        _lib.check(rc, "fb_attn_decode_plan")
        if self.window:
            rc = _lib.kernels().fb_attn_decode_plan_window(_ptr(seq_lens), B, _ptr(self.work_w), _ptr(self.n_work_w),
                                                           self.work_w.shape[0], self.window, _stream())
            _lib.check(rc, "fb_attn_decode_plan_window")


def kv_append_fp8(k, v, k_pool, v_pool, slots):
    """New 16-bit K / V rows ``[T, Hkv * D]`` -> unscaled e4m3 at pool rows ``slots`` (negative: skipped).  One launch."""
    T = k.shape[0]
    if not k.is_cuda:
        ok = slots >= 0
        sl = slots[ok].long()
        k_pool.view(-1, k.shape[-1])[sl] = k[ok].to(k_pool.dtype)
        v_pool.view(-1, v.shape[-1])[sl] = v[ok].to(v_pool.dtype)
        return
    rc = _lib.kernels().fb_kv_append_fp8(_ptr(k.contiguous()), _ptr(v.contiguous()), _ptr(k_pool), _ptr(v_pool), _ptr(slots), T, k.shape[-1],
                                         dtype_code(k.dtype), _stream())
    _lib.check(rc, "fb_kv_append_fp8")


KV8_KERNEL = True          # e4m3 page pools run the decode kernel's KV8 mode (tests switch it off to compare with the PyTorch path)
# e4m3 pages straight into the fp8 tensor core (queries and probabilities as two e4m3 terms each) instead of converting every
# page to an fp16 operand tile in shared memory
KV8_MMA = os.environ.get("FB_KV8_MMA", "1") != "0"


def attn_decode(q, k_pool, v_pool, page_table, seq_lens, scale, num_q_heads, num_kv_heads, head_dim,
                ws: DecodeWorkspace | None = None, out=None, planned=False, grid_ctas=0, quant_mode: int = 0,
                window: int = 0, softcap: float = 0.0, sinks=None, q8_ready: bool = False):
    """One new token per request. q: ``[B, Hq*D]`` -> ``[B, Hq*D]``.

    ``window`` > 0: sliding-window attention; ``softcap`` > 0: tanh soft-capping of the logits; ``sinks``: fp32 ``[Hq]`` per-head
    sink logits in the softmax denominator.  All three run inside the same kernels.

    ``quant_mode`` 1 (int8) / 2 (e4m3): the combine kernel also writes the output quantised per (request, head) -- one 128-wide
    k block of the output projection -- and the result carries it as ``out.fb_quant`` (see ``ops.basic.rmsnorm``)."""
    B = q.shape[0]
    variant = bool(window or softcap or sinks is not None)
    if not q.is_cuda:
        cu = torch.arange(B + 1, dtype=torch.int32)
        if variant:
            return paged_attention_general(q, k_pool, v_pool, page_table, seq_lens, cu, scale, num_q_heads, num_kv_heads, head_dim,
                                           window=window, sinks=sinks, softcap=softcap)
        if cpu_native(q) and k_pool.dtype == torch.float32:
            return cpu.attention_paged(q, k_pool, v_pool, page_table, seq_lens, cu, scale, num_q_heads, num_kv_heads, head_dim)
        return paged_attention_ref(q, k_pool, v_pool, page_table, seq_lens, cu, scale, num_q_heads, num_kv_heads, head_dim)
    G = num_q_heads // num_kv_heads
    kv8 = (k_pool.dtype == torch.float8_e4m3fn and v_pool.dtype == torch.float8_e4m3fn and KV8_KERNEL
           and q.dtype in (torch.float16, torch.bfloat16))
    if head_dim != 128 or G > 16 or k_pool.shape[1] != PAGE_LEN or (k_pool.dtype != q.dtype and not kv8):
        cu = torch.arange(B + 1, dtype=torch.int32, device=q.device)
        if variant or k_pool.dtype != q.dtype:
            return paged_attention_general(q, k_pool, v_pool, page_table, seq_lens, cu, scale, num_q_heads, num_kv_heads, head_dim,
                                           window=window, sinks=sinks, softcap=softcap)
        return paged_attention_ref(q, k_pool, v_pool, page_table, seq_lens.cpu(), cu.cpu(), scale, num_q_heads, num_kv_heads,
                                   head_dim)
    if ws is None or (window and ws.window != window):
        ws = DecodeWorkspace(B, num_kv_heads, G, page_table.shape[1], q.device, window=window)
        planned = False
    if B > ws.max_batch or page_table.shape[1] > ws.max_pages:
        raise ValueError("decode workspace too small for this batch / page table")
    if not planned:
        ws.plan(seq_lens)
    if out is None:
        out = torch.empty_like(q)
    num_slots = k_pool.shape[0] * k_pool.shape[1]
    if kv8:
        # e4m3 pages: the kernel turns every raw page into an fp16 operand tile in shared memory (exact conversion) and computes in
        # fp16, so queries go in and the output comes back as fp16
        work, n_work = (ws.work_w, ws.n_work_w) if window else (ws.work, ws.n_work)
        if KV8_MMA:
            qa, qb = ws.q8_terms(num_q_heads * head_dim)
            if not q8_ready:               # (the QKV post-processing kernel can write the two terms itself)
                qc = q if q.is_contiguous() else q.contiguous()
                rc = _lib.kernels().fb_quant_q_e4m3x2(_ptr(qc), _ptr(qa), _ptr(qb), B * num_q_heads * head_dim, dtype_code(q.dtype),
                                                      _stream())
                _lib.check(rc, "fb_quant_q_e4m3x2")
            rc = _lib.kernels().fb_attn_decode_opts(_ptr(qa), _ptr(k_pool), _ptr(v_pool), _ptr(out), out.stride(0), _ptr(work),
                                                    _ptr(n_work), _ptr(page_table), _ptr(seq_lens), _ptr(ws.part_o), _ptr(ws.part_ml), B,
                                                    num_q_heads, num_kv_heads, head_dim, num_slots, page_table.stride(0), ws.max_pages,
                                                    ws.work.shape[0], float(scale), 5 if out.dtype == torch.bfloat16 else 4, grid_ctas,
                                                    _ptr(None), 0, _ptr(qb), num_q_heads * head_dim, _ptr(None), _ptr(None), 0,
                                                    int(window), float(softcap), _ptr(sinks), _stream())
            _lib.check(rc, "fb_attn_decode_opts(kv8 mma)")
            return out
        q16 = q if q.dtype == torch.float16 else q.to(torch.float16)
        o16 = out                       # the combine kernel writes the caller's 16-bit type
        rc = _lib.kernels().fb_attn_decode_opts(_ptr(q16), _ptr(k_pool), _ptr(v_pool), _ptr(o16), o16.stride(0), _ptr(work),
                                                _ptr(n_work), _ptr(page_table), _ptr(seq_lens), _ptr(ws.part_o), _ptr(ws.part_ml), B,
                                                num_q_heads, num_kv_heads, head_dim, num_slots, page_table.stride(0), ws.max_pages,
                                                ws.work.shape[0], float(scale), 3 if out.dtype == torch.bfloat16 else 2, grid_ctas, _ptr(None), 0, _ptr(None),
                                                num_q_heads * head_dim, _ptr(None), _ptr(None), 0, int(window), float(softcap),
                                                _ptr(sinks), _stream())
        _lib.check(rc, "fb_attn_decode_opts(kv8)")
        return out
    xq = sa = xs = None
    ld_a = 0
    if quant_mode in (1, 2) and not _FUSED_COMBINE and B <= 128:
        K = num_q_heads * head_dim
        ld_a = (B + 128 + 3) // 4 * 4
        xq = torch.empty((B, K), device=q.device, dtype=torch.int8 if quant_mode == 1 else torch.uint8)
        sa = torch.empty((num_q_heads, ld_a), device=q.device, dtype=torch.float32)
        xs = torch.empty((num_q_heads, ld_a), device=q.device, dtype=torch.float32) if quant_mode == 1 else None
    else:
        quant_mode = 0
    if variant:
        work, n_work = (ws.work_w, ws.n_work_w) if window else (ws.work, ws.n_work)
        rc = _lib.kernels().fb_attn_decode_opts(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), out.stride(0), _ptr(work),
                                                _ptr(n_work), _ptr(page_table), _ptr(seq_lens), _ptr(ws.part_o), _ptr(ws.part_ml), B,
                                                num_q_heads, num_kv_heads, head_dim, num_slots, page_table.stride(0), ws.max_pages,
                                                ws.work.shape[0], float(scale), dtype_code(q.dtype), grid_ctas, _ptr(None), quant_mode,
                                                _ptr(xq), num_q_heads * head_dim, _ptr(sa), _ptr(xs), ld_a, int(window), float(softcap),
                                                _ptr(sinks), _stream())
        _lib.check(rc, "fb_attn_decode_opts")
        if quant_mode:
            out.fb_quant = (quant_mode, xq, sa, xs, ld_a)
        return out
    rc = _lib.kernels().fb_attn_decode(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), out.stride(0), _ptr(ws.work),
                                       _ptr(ws.n_work), _ptr(page_table), _ptr(seq_lens), _ptr(ws.part_o), _ptr(ws.part_ml), B,
                                       num_q_heads, num_kv_heads, head_dim, num_slots, page_table.stride(0), ws.max_pages,
                                       ws.work.shape[0], float(scale), dtype_code(q.dtype), grid_ctas,
                                       _ptr(ws.counters if _FUSED_COMBINE else None), quant_mode, _ptr(xq),
                                       num_q_heads * head_dim, _ptr(sa), _ptr(xs), ld_a, _stream())
    _lib.check(rc, "fb_attn_decode")
    if quant_mode:
        out.fb_quant = (quant_mode, xq, sa, xs, ld_a)
    return out


def attn_prefill(q, k_pool, v_pool, page_table, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim, out=None,
                 cu_q_host=None):
    """Packed causal prefill (also chunked prefill / prefix-cache continuation). q: ``[T, Hq*D]``."""
    if cpu_native(q) and k_pool.dtype == torch.float32:
        return cpu.attention_paged(q, k_pool, v_pool, page_table, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim)
    if (q.is_cuda and k_pool.dtype == torch.float8_e4m3fn and head_dim == 128 and k_pool.shape[1] == PAGE_LEN
            and q.dtype in (torch.float16, torch.bfloat16)):
        # e4m3 pages: the pages this batch reads are brought into a scratch pool in the activations' type (exact conversion)
        # and the tensor-core prefill kernel runs on that pool through a re-indexed page table.  Prefill is bound by its
        # MMAs, the conversion reads every context byte once.
        P = page_table.shape[1]
        npg = ((kv_lens.to(torch.long) + PAGE_LEN - 1) // PAGE_LEN).clamp(max=P)
        mask = torch.arange(P, device=q.device)[None, :] < npg[:, None]
        used = page_table[mask].long()
        pt = torch.zeros_like(page_table)
        pt[mask] = torch.arange(used.numel(), device=q.device, dtype=page_table.dtype)
        kt = k_pool.index_select(0, used).to(q.dtype)
        vt = v_pool.index_select(0, used).to(q.dtype)
        return attn_prefill(q, kt, vt, pt, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim, out, cu_q_host)
    if not q.is_cuda or head_dim != 128 or k_pool.shape[1] != PAGE_LEN:
        o = paged_attention_ref(q, k_pool, v_pool, page_table, kv_lens.cpu(), cu_q.cpu(), scale, num_q_heads, num_kv_heads,
                                head_dim)
        return o
    cu = cu_q_host if cu_q_host is not None else cu_q.tolist()
    blocks = []
    for b in range(len(cu) - 1):
        for q0 in range(0, cu[b + 1] - cu[b], 128):
            blocks.append((b, q0))
    blocks.sort(key=lambda t: -t[1])        # causal work grows with the block's start: longest blocks are scheduled first
    if out is None:
        out = torch.empty_like(q)
    if not blocks:
        return out
    blk = torch.tensor(blocks, dtype=torch.int32).to(q.device, non_blocking=True)
    num_slots = k_pool.shape[0] * k_pool.shape[1]
    rc = _lib.kernels().fb_attn_prefill(_ptr(q), q.stride(0), q.shape[0], _ptr(k_pool), _ptr(v_pool), _ptr(out), out.stride(0),
                                        _ptr(blk), len(blocks), _ptr(cu_q), _ptr(kv_lens), _ptr(page_table), num_q_heads,
                                        num_kv_heads, head_dim, num_slots, page_table.stride(0), float(scale),
                                        dtype_code(q.dtype), _stream())
    _lib.check(rc, "fb_attn_prefill")
    return out


# ---------------------------------------------------------------------------------------------------
# MLA decode (absorbed latent attention, kv_lora 512 + rope 64)
# ---------------------------------------------------------------------------------------------------
_lib.register_sigs({"fb_mla_decode": [ctypes.c_void_p] * 10 + [ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_float, ctypes.c_int, ctypes.c_void_p]}, ["attn_mla"])
_MLA_WS: dict = {}


class MlaWorkspace:
    """Device scratch of the MLA decode kernel for up to (max_batch, max_pages, heads)."""

    def __init__(self, max_batch, max_pages, heads, device):
        groups = (heads + 31) // 32
        self.max_items = max_batch * max_pages * groups
        self.work = torch.zeros((self.max_items, 4), device=device, dtype=torch.int32)
        self.n_work = torch.zeros((1,), device=device, dtype=torch.int32)
        self.item_range = torch.zeros((max_batch, 2), device=device, dtype=torch.int32)
        self.part_o = torch.empty((self.max_items * 32 * 512,), device=device, dtype=torch.float32)
        self.part_ml = torch.empty((self.max_items * 32 * 2,), device=device, dtype=torch.float32)


def mla_decode(q_full, lat_pool, page_table, seq_lens, scale, ws: MlaWorkspace | None = None):
    """q_full ``[B, H, 576]`` (absorbed q_nope | rotated q_pe), lat_pool ``[pages, 128, 1, 576]`` -> ``[B, H, 512]``."""
    B, H, _ = q_full.shape
    P = page_table.shape[1]
    if ws is None:
        key = (q_full.device, B, P, H)
        ws = _MLA_WS.get(key)
        if ws is None:
            ws = _MLA_WS[key] = MlaWorkspace(B, P, H, q_full.device)
    q_full = q_full.contiguous()
    out = torch.empty((B, H, 512), device=q_full.device, dtype=q_full.dtype)
    num_slots = lat_pool.shape[0] * lat_pool.shape[1]
    rc = _lib.kernels().fb_mla_decode(_ptr(q_full), _ptr(lat_pool), _ptr(out), _ptr(page_table), _ptr(seq_lens), _ptr(ws.work),
                                      _ptr(ws.n_work), _ptr(ws.item_range), _ptr(ws.part_o), _ptr(ws.part_ml), B, H, num_slots,
                                      page_table.stride(0), ws.max_items, float(scale), dtype_code(q_full.dtype), _stream())
    _lib.check(rc, "fb_mla_decode")
    return out
