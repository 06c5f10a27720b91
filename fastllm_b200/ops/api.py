"""Operator-level API under the reference's operator names.

The reference registers about 130 named operators per device (src/devices/cuda/cudadevice.cpp:4019-4139,
src/devices/cpu/cpudevice.cpp:284-394) and tests every device against the CPU one (test/ops/cppOps.cpp).  This module is that
surface for PyTorch tensors: each function runs the hand-written sm_100a kernel when the tensor is on the GPU and the kernel
covers the case, the native C++ CPU backend for fp32 CPU tensors, and the plain PyTorch definition otherwise -- so the same
call is both the product path and, on the CPU, the oracle.  Functions return their result (the reference writes into an output
argument); the ``*To`` forms update their first argument in place like the reference.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import attention as A
from . import basic as B
from . import cpu as C
from . import moe as M

# ---- dtype conversion ---------------------------------------------------------------------------
def ToFloat16(x): return x.to(torch.float16)
def ToFloat32(x): return x.to(torch.float32)
def ToBFloat16(x): return x.to(torch.bfloat16)
ConvertToFloat16, ConvertToFloat32, ConvertToBFloat16 = ToFloat16, ToFloat32, ToBFloat16


# ---- embedding / norms ----------------------------------------------------------------------------
def Embedding(ids, weight):
    if B.cpu_native(weight):
        return C.embedding(weight, ids).reshape(*ids.shape, weight.shape[1])
    return B.embedding(ids, weight)


def RMSNorm(x, weight, eps):
    return B.rmsnorm(x, weight, eps)


def LayerNorm(x, gamma, beta, eps=1e-5):
    if B.cpu_native(x):
        return C.layernorm(x, gamma, beta, eps)
    return F.layer_norm(x.float(), (x.shape[-1],), gamma.float(), beta.float() if beta is not None else None, eps).to(x.dtype)


# ---- linear family --------------------------------------------------------------------------------
def Linear(x, weight, bias=None):
    """``y[n, k] = x[n, m] W[k, m]^T + b[k]``; ``weight`` may be a tensor or a quantised ``LinearWeight``."""
    from .quant import LinearWeight

    if isinstance(weight, LinearWeight):
        return weight(x)
    return B.linear(x, weight, bias)


def LinearAdd(x, weight, bias, out):
    """``out += Linear(x)`` (residual fused into the GEMM epilogue on the GPU)."""
    y = B.linear(x, weight, bias, residual=out)
    out.copy_(y)
    return out


def LinearSwiglu(x, weight_gate_up, bias=None, interleaved=False):
    """``silu(x Wg^T) * (x Wu^T)`` with ``weight_gate_up = [Wg; Wu]`` (tile-interleaved rows when ``interleaved``)."""
    return B.linear(x, weight_gate_up, bias, swiglu=True, interleaved=interleaved)


def SwigluLinearAdd(gate_up, weight_down, out):
    return LinearAdd(Swiglu(gate_up), weight_down, None, out)


def MatMul(a, b, alpha=1.0):
    return torch.matmul(a, b) * alpha if alpha != 1.0 else torch.matmul(a, b)


def MatMulTransB(a, b, alpha=1.0):
    return torch.matmul(a, b.transpose(-1, -2)) * alpha if alpha != 1.0 else torch.matmul(a, b.transpose(-1, -2))


# ---- activations ----------------------------------------------------------------------------------
def _act(x, name, fn):
    if B.cpu_native(x):
        return C.activation(x, name)
    return fn(x.float()).to(x.dtype)


def Silu(x): return _act(x, "silu", F.silu)
def Gelu(x): return _act(x, "gelu", F.gelu)
def GeluNew(x): return _act(x, "gelu_new", lambda t: F.gelu(t, approximate="tanh"))
def Relu(x): return _act(x, "relu", torch.relu)
def Sigmoid(x): return _act(x, "sigmoid", torch.sigmoid)
def TanH(x): return _act(x, "tanh", torch.tanh)
def Exp(x): return _act(x, "exp", torch.exp)
def Swiglu(x): return B.silu_mul(x)


def Geglu(x):
    g, u = x.float().chunk(2, dim=-1)
    return (F.gelu(g) * u).to(x.dtype)


def SoftMax(x, axis=-1):
    if B.cpu_native(x) and axis in (-1, x.dim() - 1):
        return C.softmax(x)
    return torch.softmax(x.float(), dim=axis).to(x.dtype)


# ---- arithmetic / layout ----------------------------------------------------------------------------
def Add(x, v): return x + v
def Mul(x, v): return x * v
def AddTo(x, y, alpha=1.0): return x.add_(y, alpha=alpha)
def MulTo(x, y): return x.mul_(y)
def Cat(a, b, axis): return torch.cat([a, b], dim=axis)
def Split(x, axis, start, end): return x.narrow(axis, start, end - start)
def Repeat(x, axis, times): return torch.cat([x] * times, dim=axis)
def Permute(x, axes): return x.permute(*axes).contiguous()
PermuteSelf = Permute


def TopK(x, k):
    """Returns ``[..., k, 2]`` pairs (index, value) like the reference's TopK."""
    v, i = torch.topk(x.float(), k, dim=-1)
    return torch.stack([i.float(), v], dim=-1)


# ---- masks / penalties ------------------------------------------------------------------------------
def AttentionMask(scores, mask, value):
    return scores.masked_fill(mask.bool(), value)


def CausalMask(scores, base=0, value=-1e4):
    q, k = scores.shape[-2], scores.shape[-1]
    m = torch.arange(k, device=scores.device)[None, :] > (torch.arange(q, device=scores.device)[:, None] + base)
    return scores.masked_fill(m, value)


def AlibiMask(scores, slopes, value=-1e4):
    """``scores[h, i, j] += slopes[h] * (j - i)`` on the causal part, ``value`` above the diagonal (key length - query length offset)."""
    q, k = scores.shape[-2], scores.shape[-1]
    i = torch.arange(q, device=scores.device)[:, None] + (k - q)
    j = torch.arange(k, device=scores.device)[None, :]
    out = scores + slopes.reshape(-1, 1, 1).to(scores.dtype) * (j - i).to(scores.dtype)
    return out.masked_fill(j > i, value)


def RepeatPenalty(logits, recent_ids, penalty):
    """Divide positive / multiply negative logits of the recently generated tokens (one row per request)."""
    from ..engine.sampling import apply_repeat_penalty

    return apply_repeat_penalty(logits, recent_ids, penalty)


# ---- rotary embeddings ------------------------------------------------------------------------------
def LlamaRotatePosition2D(x, position_ids, sin, cos, rotary_dim):
    """Half-split (neox) rotation with precomputed tables; x ``[T, H, D]``, rotates the first ``2 * rotary_dim`` dims."""
    return A.apply_rope_ref(x, position_ids, cos, sin, A.ROPE_NEOX, 2 * rotary_dim)


def NearlyRotatePosition2D(x, position_ids, sin, cos, rotary_dim):
    """Interleaved-pair rotation (DeepSeek MLA, GLM)."""
    return A.apply_rope_ref(x, position_ids, cos, sin, A.ROPE_INTERLEAVED, 2 * rotary_dim)


def RopeEncoding(x, position_ids, rotary_dim, rope_theta, rope_scale=1.0):
    """Rotation with frequencies computed from ``rope_theta`` (linear position scaling by ``rope_scale``)."""
    scaling = {"type": "linear", "factor": rope_scale} if rope_scale != 1.0 else None
    cos, sin = A.build_rope_tables(rotary_dim, int(position_ids.max()) + 1, rope_theta, scaling, x.device)
    return A.apply_rope_ref(x, position_ids, cos, sin, A.ROPE_NEOX, rotary_dim)


def Llama3RopeEncoding(x, position_ids, rotary_dim, rope_theta, scaling: dict):
    cos, sin = A.build_rope_tables(rotary_dim, int(position_ids.max()) + 1, rope_theta, dict(scaling, rope_type="llama3"), x.device)
    return A.apply_rope_ref(x, position_ids, cos, sin, A.ROPE_NEOX, rotary_dim)


def YarnRopeEncoding(x, position_ids, rotary_dim, rope_theta, scaling: dict):
    cos, sin = A.build_rope_tables(rotary_dim, int(position_ids.max()) + 1, rope_theta, dict(scaling, rope_type="yarn"), x.device)
    return A.apply_rope_ref(x, position_ids, cos, sin, A.ROPE_NEOX, rotary_dim)


# ---- attention --------------------------------------------------------------------------------------
def Attention(q, k, v, mask=None, group=1, scale=None, causal=False):
    """Dense (non-paged) attention; q ``[Hq, Tq, D]``, k / v ``[Hkv, Tk, D]`` with ``Hq = group * Hkv``."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    kk = k.repeat_interleave(group, dim=0) if group > 1 else k
    vv = v.repeat_interleave(group, dim=0) if group > 1 else v
    s = torch.matmul(q.float(), kk.float().transpose(-1, -2)) * scale
    if causal:
        s = CausalMask(s, base=k.shape[-2] - q.shape[-2], value=float("-inf"))
    if mask is not None:
        s = s.masked_fill(mask.bool(), float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vv.float()).to(q.dtype)


def AppendPagedCache(k, v, slots, k_pool, v_pool):
    """Write new K / V rows ``[T, Hkv * D]`` into the page pools at ``slots`` (negative slots are skipped)."""
    if B.cpu_native(k) and k_pool.dtype == torch.float32:
        C.kv_append(k, v, slots, k_pool, v_pool)
        return
    ok = slots >= 0
    sl = slots[ok].long()
    k_pool.view(-1, k.shape[-1])[sl] = k[ok].to(k_pool.dtype)
    v_pool.view(-1, v.shape[-1])[sl] = v[ok].to(v_pool.dtype)


def AttentionPaged(q, k_pool, v_pool, page_table, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim, is_decode=False):
    """Causal attention of packed new tokens over the paged cache (decode when every request has one new token)."""
    if is_decode:
        return A.attn_decode(q, k_pool, v_pool, page_table, kv_lens, scale, num_q_heads, num_kv_heads, head_dim)
    return A.attn_prefill(q, k_pool, v_pool, page_table, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim)


AttentionPagedBatch = AttentionPaged
QKVRMSNormRopeSplitAppendPagedCache = A.qkv_post


def MergeMLAPaged(q_full, lat_pool, fb, scale, kv_lora_rank):
    return M.mla_paged_attention(q_full, lat_pool, fb, scale, kv_lora_rank)


# ---- mixture of experts -----------------------------------------------------------------------------
def SelectExpert(logits, bias, topk, need_norm, route_scale=1.0, mode="none"):
    """Top-k on ``score(logits) + bias`` with the weights taken from the un-biased scores (optional renorm, times scale)."""
    if B.cpu_native(logits):
        return C.select_expert(logits, bias, topk, mode, need_norm, route_scale)
    return M.route_topk(logits, bias, topk, {"softmax": 0, "sigmoid": 1, "none": 2}[mode], need_norm, 1, 1, route_scale)


def FusedSoftmaxSelectExpert(logits, topk, need_norm, route_scale=1.0):
    return SelectExpert(logits, None, topk, need_norm, route_scale, "softmax")


def FusedSigmoidSelectExpert(logits, bias, topk, need_norm, route_scale=1.0):
    return SelectExpert(logits, bias, topk, need_norm, route_scale, "sigmoid")


def MergeMOE(x, index, score, experts, shared=None, shared_scale=1.0):
    """``y = sum_k score_k * expert_k(x) (+ shared_scale * shared(x))``; ``experts`` is an ``ExpertWeights`` set."""
    y = M.moe_forward(x, index, score, experts)
    if shared is not None:
        y = y + shared(x) * shared_scale
    return y


FusedMOE = MergeMOE
