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


# ---- the rest of the reference's operator list (src/devices/cuda/cudadevice.cpp:4019-4139, cpudevice.cpp:284-394) ----------
def EmbeddingDirect(ids, weight, out):
    out.copy_(Embedding(ids, weight))
    return out


def RMSNormPart(x, weight, eps, start, end):
    """RMSNorm of the column range ``[start, end)`` of every row, other columns untouched (tensor-parallel sharded norms)."""
    out = x.clone()
    out[..., start:end] = B.rmsnorm(x[..., start:end].contiguous(), weight, eps)
    return out


def Normalize(x, axis=-1, eps=1e-12):
    return (x.float() / x.float().norm(dim=axis, keepdim=True).clamp_min(eps)).to(x.dtype)


def Copy(dst, src):
    dst.copy_(src)
    return dst


def CatDirect(dst, x, axis):
    """Append ``x`` to ``dst`` along ``axis`` (the reference grows a pre-expanded buffer in place; here a new tensor is returned)."""
    return x.clone() if dst is None or dst.numel() == 0 else torch.cat([dst, x], dim=axis)


def Pad(x, axis, before, after, value=0.0):
    pads = [0, 0] * x.dim()
    ax = axis % x.dim()
    pads[2 * (x.dim() - 1 - ax)], pads[2 * (x.dim() - 1 - ax) + 1] = before, after
    return F.pad(x, pads, value=value)


def MulSingleTo(x, v):
    return x.mul_(v)


def ChannelMulTo(x, scale):
    """``x[..., c] *= scale[c]``."""
    return x.mul_(scale.to(x.dtype))


def Clamp(x, lo, hi):
    return x.clamp(lo, hi)


def CrossSwiglu(x):
    """SwiGLU over interleaved columns: gate = even columns, up = odd columns."""
    xf = x.float()
    return (F.silu(xf[..., 0::2]) * xf[..., 1::2]).to(x.dtype)


def SwigluGptOss(x, alpha=1.702, limit=7.0):
    """gpt-oss gated activation on interleaved (gate, up) columns: clamp, ``gate * sigmoid(alpha * gate) * (up + 1)``."""
    xf = x.float()
    g, u = xf[..., 0::2].clamp(max=limit), xf[..., 1::2].clamp(-limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1)).to(x.dtype)


def MambaSoftplus(x, bias=None):
    return F.softplus(x.float() + (bias.float() if bias is not None else 0.0)).to(x.dtype)


def SigmoidMambaSoftplus(a, b, A_log, dt_bias):
    """Gated-DeltaNet gates from the raw projections: ``(beta, g) = (sigmoid(b), -exp(A_log) * softplus(a + dt_bias))``."""
    return torch.sigmoid(b.float()), -A_log.float().exp() * F.softplus(a.float() + dt_bias.float())


def SigmoidMulTo(x, gate):
    """``x *= sigmoid(gate)`` (gated attention output)."""
    return x.mul_(torch.sigmoid(gate.float()).to(x.dtype))


def AttentionExtendedMask(scores, mask, value=-1e4):
    return scores.masked_fill(mask.bool().expand_as(scores), value)


def ApplyLognAttn(q, logn, position_ids):
    """Qwen-1 long-context scaling: every query row is multiplied by ``logn[position]``."""
    return (q.float() * logn.float()[position_ids.long()].reshape(-1, *([1] * (q.dim() - 1)))).to(q.dtype)


def CumSumLastDim(x):
    return x.float().cumsum(-1).to(x.dtype)


def MakeDecayMask(g_cumsum):
    """``exp(G_i - G_j)`` for ``j <= i`` and 0 above the diagonal, from the running log-decay of a chunk (chunked delta rule)."""
    d = (g_cumsum.float()[..., :, None] - g_cumsum.float()[..., None, :]).tril().exp().tril()
    return d


def ApplyChunkDecayByLastLogG(k, g_cumsum):
    """``k_j * exp(G_last - G_j)``: keys weighted for the carry of a chunk's state into the next chunk."""
    return k.float() * (g_cumsum.float()[..., -1:, None] - g_cumsum.float()[..., :, None]).exp().reshape(*g_cumsum.shape, 1)


def TransferAttn(attn):
    """``(I - A)^-1`` of a strictly lower triangular ``A`` by forward substitution (the in-chunk solve of the delta rule)."""
    T = attn.float().clone()
    c = T.shape[-1]
    for i in range(1, c):
        T[..., i, :i] = T[..., i, :i] + (T[..., i, :i, None] * T[..., :i, :i]).sum(-2)
    return T + torch.eye(c, device=T.device, dtype=T.dtype)


def Conv1DPerChannel(x, weight, bias=None, pad_left=None):
    """Depth-wise causal convolution; x ``[B, C, L]``, weight ``[C, K]``: output ``[B, C, L]`` (left padding K-1 by default)."""
    K = weight.shape[-1]
    xp = F.pad(x.float(), (K - 1 if pad_left is None else pad_left, 0))
    return F.conv1d(xp, weight.float().unsqueeze(1), bias.float() if bias is not None else None, groups=x.shape[1]).to(x.dtype)


def Conv2D(x, weight, bias=None, stride=1, padding=0):
    return F.conv2d(x.float(), weight.float(), bias.float() if bias is not None else None, stride=stride, padding=padding).to(x.dtype)


def RecurrentGatedDeltaRule(q, k, v, g, beta, state):
    """One sequence through the gated delta rule, token by token; see ``ops.linear_attn``.  ``state`` is updated in place."""
    from . import linear_attn as L

    Dk = q.shape[-1]
    return L.gated_delta_recurrent_ref(L.l2norm(q.float()) * Dk ** -0.5, L.l2norm(k.float()), v.float(), g.float(), beta.float(), state)


def ChunkGatedDeltaRulePrefill(q, k, v, g, beta, state, chunk=64):
    """Same result chunk by chunk with matrix products (prefill form)."""
    from . import linear_attn as L

    Dk = q.shape[-1]
    return L.gated_delta_chunked(L.l2norm(q.float()) * Dk ** -0.5, L.l2norm(k.float()), v.float(), g.float(), beta.float(), state, chunk)


def RotatePosition2D(x, position_ids, sin, cos, rotary_dim):
    """ChatGLM 2-D rotation: the first half of the head rotates with the position ids, the second with the block ids;
    x ``[T, H, D]``, position_ids ``[2, T]``."""
    D = x.shape[-1]
    a = A.apply_rope_ref(x[..., :D // 2], position_ids[0], cos, sin, A.ROPE_NEOX, min(2 * rotary_dim, D // 2))
    b = A.apply_rope_ref(x[..., D // 2:], position_ids[1], cos, sin, A.ROPE_NEOX, min(2 * rotary_dim, D // 2))
    return torch.cat([a, b], dim=-1)


def LlamaRotatePosition2DPart(x, position_ids, sin, cos, rotary_dim, part):
    """Neox rotation of the first ``part`` dims only (partial rotary)."""
    return A.apply_rope_ref(x, position_ids, cos, sin, A.ROPE_NEOX, min(part, 2 * rotary_dim))


def Qwen35InterleavedRope(x, position_ids, sin, cos, rotary_dim):
    """Interleaved multi-axis rope of Qwen3.5: with text-only inputs the three position axes coincide and the rotation is
    the half-split rotation over ``rotary_dim`` dims."""
    return A.apply_rope_ref(x, position_ids, cos, sin, A.ROPE_NEOX, rotary_dim)


def ScaleQRatory(q, scale):
    return (q.float() * scale).to(q.dtype)


def QKVRMSNormRope(qkv, positions, num_q_heads, num_kv_heads, head_dim, cos, sin, q_norm, k_norm, eps, rope_mode=A.ROPE_NEOX, rot=None):
    """Split + per-head RMSNorm + RoPE without the cache append: returns ``(q, k, v)``."""
    T = qkv.shape[0]
    q, k, v = qkv.split([num_q_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * head_dim], dim=-1)
    q, k = q.reshape(T, num_q_heads, head_dim), k.reshape(T, num_kv_heads, head_dim)
    if q_norm is not None:
        q, k = A._head_norm_ref(q, q_norm, eps, 0.0), A._head_norm_ref(k, k_norm, eps, 0.0)
    q = A.apply_rope_ref(q, positions, cos, sin, rope_mode, rot or head_dim)
    k = A.apply_rope_ref(k, positions, cos, sin, rope_mode, rot or head_dim)
    return q.reshape(T, -1), k.reshape(T, -1), v


def MergeAttention(x, qkv_w, qkv_b, o_w, o_b, positions, slots, k_pool, v_pool, page_table, kv_lens, cu_q, num_q_heads, num_kv_heads,
                   head_dim, cos, sin, scale=None, is_decode=False):
    """The reference's merged attention operator (QKV projection, RoPE, cache append, paged attention, output projection)."""
    scale = scale if scale is not None else head_dim ** -0.5
    q = A.qkv_post(B.linear(x, qkv_w, qkv_b), positions, slots, k_pool, v_pool, num_q_heads, num_kv_heads, head_dim, cos, sin)
    a = AttentionPaged(q, k_pool, v_pool, page_table, kv_lens, cu_q, scale, num_q_heads, num_kv_heads, head_dim, is_decode)
    return B.linear(a, o_w, o_b)


def MLP(x, gate_up_w, down_w, interleaved=False):
    """The reference's fused MLP operator: ``down(silu(gate(x)) * up(x))``."""
    return B.linear(B.linear(x, gate_up_w, swiglu=True, interleaved=interleaved), down_w)


def CopyKVCache(dst_pool, src_pool, dst_pages, src_pages):
    """Copy whole pages between pools (prefix sharing / defragmentation)."""
    dst_pool[torch.as_tensor(dst_pages, device=dst_pool.device).long()] = src_pool[torch.as_tensor(src_pages, device=src_pool.device).long()]
    return dst_pool


AppendPagedCacheBatch = AppendPagedCache


def GeneratePagedBatchParams(page_lists, lengths, page_len=A.PAGE_LEN):
    """Host lists -> ``(page_table [B, P] int32, kv_lens [B] int32, last_page_len [B] int32)`` for a batch of requests."""
    Bn = len(page_lists)
    P = max(1, max(len(p) for p in page_lists))
    pt = torch.zeros(Bn, P, dtype=torch.int32)
    for b, pg in enumerate(page_lists):
        pt[b, :len(pg)] = torch.tensor(pg, dtype=torch.int32)
    kv = torch.tensor(lengths, dtype=torch.int32)
    return pt, kv, ((kv - 1) % page_len + 1).to(torch.int32)


def GenerateAppendPagedCacheBatchParams(page_lists, starts, counts, page_len=A.PAGE_LEN):
    """Cache slots of ``counts[b]`` new tokens starting at position ``starts[b]`` of every request, packed."""
    out = []
    for pg, s, n in zip(page_lists, starts, counts):
        out += [pg[(s + i) // page_len] * page_len + (s + i) % page_len for i in range(n)]
    return torch.tensor(out, dtype=torch.int32)


# ---- batch variants: one call over a list of per-request tensors ------------------------------------------------------------
def SplitBatch(x, axis, parts): return list(torch.split(x, x.shape[axis] // parts, dim=axis))
def CatBatch(xs, axis): return torch.cat(list(xs), dim=axis)
def MulBatch(xs, v): return [x * v for x in xs]
def MatMulBatch(As, Bs, alpha=1.0): return [MatMul(a, b, alpha) for a, b in zip(As, Bs)]
def MatMulTransBBatch(As, Bs, alpha=1.0): return [MatMulTransB(a, b, alpha) for a, b in zip(As, Bs)]
def SoftMaxBatch(xs, axis=-1): return [SoftMax(x, axis) for x in xs]
def CatDirectBatch(dsts, xs, axis): return [CatDirect(d, x, axis) for d, x in zip(dsts, xs)]
def AppendKVCachebatch(caches, xs, axis=0): return [CatDirect(c, x, axis) for c, x in zip(caches, xs)]
def AttentionBatch(qs, ks, vs, masks=None, group=1, scale=None):
    return [Attention(q, k, v, None if masks is None else masks[i], group, scale) for i, (q, k, v) in enumerate(zip(qs, ks, vs))]


# ---- softmax / extended linear / adapters ----------------------------------------------------------
def Softmax(x, axis=-1):
    if B.cpu_native(x) and axis in (-1, x.dim() - 1):
        return C.softmax(x)
    return torch.softmax(x.float(), dim=axis).to(x.dtype)


def SoftmaxBatch(xs, axis=-1):
    return [Softmax(x, axis) for x in xs]


ExTypeNone, ExSwiglu, ExGelu, ExSilu = 0, 1, 2, 3


def CanRunLinearEx(ex_type) -> bool:
    return ex_type in (ExTypeNone, ExSwiglu, ExGelu, ExSilu)


def LinearEx(x, weight, bias=None, ex_type=ExTypeNone):
    """Linear followed by an activation (reference: LinearEx, include/fastllm.h ``LinearExType``).  SwiGLU runs in the GEMM
    epilogue on the GPU; ``weight`` then holds gate rows followed by up rows."""
    if ex_type == ExSwiglu:
        return LinearSwiglu(x, weight, bias)
    y = Linear(x, weight, bias)
    if ex_type == ExGelu:
        return F.gelu(y.float()).to(y.dtype)
    if ex_type == ExSilu:
        return Silu(y)
    return y


def CanRunLinearAdd(x, weight, bias=None, out=None) -> bool: return True
def CanRunLinearSwiglu(x, weight) -> bool: return weight.shape[0] % 2 == 0
def CanRunSwigluLinearAdd(x, weight, bias=None, out=None) -> bool: return x.shape[-1] % 2 == 0
def CanRunMLP() -> bool: return True
def CanRunMergeAttention() -> bool: return True
def CanRunMergeMOE(*_a, **_k) -> bool: return True


def LoraLayer(x, weight, lora_a, lora_b, bias=None, lora_config=None):
    """``y = W x + (alpha / r) * B (A x)`` (reference: LoraLayer, src/fastllm.cpp).  ``lora_config``: ``lora_alpha``, ``r``."""
    cfg = lora_config or {}
    r = float(cfg.get("r", lora_a.shape[0]))
    scale = float(cfg.get("lora_alpha", r)) / r
    y = Linear(x, weight, bias)
    return y + (Linear(Linear(x, lora_a), lora_b).float() * scale).to(y.dtype)


def IA3Layer(x, weight, ia3_l, bias=None, ia3_config=None):
    """(IA)^3: the learned vector rescales the layer's output, or its input for feed-forward layers
    (``ia3_config['if_feedforward']``) (reference: IA3Layer, src/fastllm.cpp)."""
    ff = str((ia3_config or {}).get("if_feedforward", "false")).lower() in ("1", "true")
    if ff:
        return Linear((x.float() * ia3_l.float()).to(x.dtype), weight, bias)
    y = Linear(x, weight, bias)
    return (y.float() * ia3_l.float()).to(y.dtype)


def AppendKVCacheBatch(caches, new):
    """``caches[b]`` (``[heads, len, dim]``) grows by row ``b`` of ``new`` (``[batch, heads, new_len, dim]``)."""
    return [torch.cat([c, new[b].to(c.dtype)], dim=-2) for b, c in enumerate(caches)]


def MergeMLA(q_nope, q_pe, kv_cache, pe_cache, mask, scale):
    """Absorbed multi-head latent attention over contiguous caches: scores from the latent part (``q_nope`` already multiplied
    by W_UK, ``[B, H, lora]`` against ``kv_cache [B, L, lora]``) plus the rotary part, softmax, values = the latent rows.
    (reference: MergeMLA, include/fastllm.h:918; the paged form is ``MergeMLAPaged``)."""
    s = torch.einsum("bhd,bld->bhl", q_nope.float(), kv_cache.float()) + torch.einsum("bhd,bld->bhl", q_pe.float(), pe_cache.float())
    s = s * scale
    if mask is not None and mask.numel():
        s = s.masked_fill(mask.bool().reshape(s.shape[0], 1, -1)[..., :s.shape[-1]], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhl,bld->bhd", p, kv_cache.float()).to(q_nope.dtype)


def ToDataType(x, dtype):
    """Conversion between the float types by name or torch dtype (quantised storage types are built by ``LinearWeight``)."""
    table = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16, "fp32": torch.float32,
             "fp16": torch.float16, "bf16": torch.bfloat16}
    return x.to(table[dtype] if isinstance(dtype, str) else dtype)


def ToDataTypeForceCPU(x, dtype):
    return ToDataType(x.cpu(), dtype)


def GetDataTypeName(dtype) -> str:
    names = {0: "float32", 1: "bfloat16", 2: "int16", 3: "int8", 4: "int4", 5: "int2", 6: "bit", 7: "float16", 8: "int4_nozero",
             9: "int4_group", 10: "fp8_e4m3", 11: "int2_group", 12: "base3_group"}
    if isinstance(dtype, int):
        return names.get(dtype, f"unknown({dtype})")
    return str(dtype).replace("torch.", "")


def NVFP4E8M0ScaleToFloat(v: int) -> float:
    """An e8m0 block scale byte as a float: 2^(v - 127); 255 is NaN."""
    return float("nan") if int(v) == 255 else float(2.0 ** (int(v) - 127))


def LLMSamplingOnly(logits, config=None):
    """One token id from a row of logits with the request's sampling settings (top-k, top-p, temperature)."""
    from ..engine import sampling

    lg = logits.reshape(1, -1).float().clone()
    g = config
    if g is None or not getattr(g, "do_sample", False) or getattr(g, "top_k", 1) == 1:
        return int(lg.argmax())
    return int(sampling.sample(lg.cpu(), [g.top_k], [g.top_p], [g.temperature])[0])


def LLMSampling(logits, config=None, recent_ids=None):
    """Repetition penalty on the recently produced tokens, then ``LLMSamplingOnly``."""
    from ..engine import sampling

    lg = logits.reshape(1, -1).float().clone()
    if config is not None and recent_ids and abs(getattr(config, "repeat_penalty", 1.0) - 1.0) > 1e-8:
        sampling.apply_repeat_penalty(lg, [list(recent_ids)], [config.repeat_penalty])
    return LLMSamplingOnly(lg, config)


# ---- Kimi-K3 operators (Kimi Delta Attention stack; reference: src/devices/cpu/kimi_k3_ops.cpp) ----------
def KimiK3RMSNorm(x, weight, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def KimiK3L2Norm(x, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def KimiK3RMSNormSigmoidGate(x, gate, weight, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float() * torch.sigmoid(gate.float())).to(x.dtype)


def KimiK3SiTUAndMul(gate, up, beta=1.0, linear_beta=0.0):
    """``beta * tanh(g / beta) * sigmoid(g)`` times the (optionally tanh-bounded) up projection."""
    g, u = gate.float(), up.float()
    situ = beta * torch.tanh(g / beta) * torch.sigmoid(g)
    if linear_beta > 0:
        u = linear_beta * torch.tanh(u / linear_beta)
    return (situ * u).to(gate.dtype)


def KimiK3CausalConv1D(x, weight, kernel_size, cache=None):
    """Depth-wise causal convolution over ``[batch, seq, channels]`` followed by SiLU; with ``cache``
    (``[batch, kernel - 1, channels]``) the sequence continues from the cached inputs and the cache is advanced in place."""
    Bn, S, Cn = x.shape
    w = weight.reshape(Cn, kernel_size).float()
    hist = cache.float() if cache is not None else torch.zeros(Bn, kernel_size - 1, Cn, device=x.device)
    full = torch.cat([hist, x.float()], dim=1)                              # [B, K-1+S, C]
    win = full.unfold(1, kernel_size, 1)                                    # [B, S, C, K]
    y = (win * w[None, None]).sum(-1)
    if cache is not None:
        cache.copy_(full[:, -(kernel_size - 1):].to(cache.dtype))
    return F.silu(y).to(x.dtype)


def KimiK3UpdatePackedConvCache(q, k, v, history, tokens, cache):
    """Advance the packed q | k | v convolution cache (``[batch, history, Cq + Ck + Cv]``) by the first ``tokens`` rows of the
    projected inputs, without evaluating the convolution."""
    new = torch.cat([q[:, :tokens], k[:, :tokens], v[:, :tokens]], dim=-1).to(cache.dtype)
    full = torch.cat([cache, new], dim=1)
    cache.copy_(full[:, -history:])
    return cache


def _kda_gates(raw_gate, raw_beta, a_log, dt_bias, lower_bound):
    H, D = raw_gate.shape[-2], raw_gate.shape[-1]
    a = a_log.float().reshape(H, 1) if a_log.numel() == H else a_log.float().reshape(1, D)
    gate = lower_bound * torch.sigmoid(torch.exp(a) * (raw_gate.float() + dt_bias.float().reshape(H, D)))
    return gate, torch.sigmoid(raw_beta.float())


def KimiK3RecurrentKDA(q, k, v, raw_gate, raw_beta, a_log, dt_bias, lower_bound=-5.0, state=None, output_aux=True, tokens=None,
                       state_only=False):
    """Kimi Delta Attention, recurrent form over ``[batch, seq, heads, dim]``: per-channel decay
    ``exp(lower_bound * sigmoid(exp(A) * (g + dt_bias)))`` on the rows of the ``[dim, dim]`` state, delta-rule write with
    ``beta = sigmoid(raw_beta)``, read-out scaled by ``dim^-1/2``.  Returns (output, state, decay, beta)."""
    Bn, S, H, D = k.shape
    n = S if tokens is None else int(tokens)
    if state is None:
        state = torch.zeros(Bn, H, D, D, dtype=torch.float32, device=k.device)
    gate, beta = _kda_gates(raw_gate, raw_beta, a_log, dt_bias, lower_bound)
    out = None if state_only else torch.empty(Bn, S, H, D, dtype=torch.float32, device=k.device)
    kf, vf = k.float(), v.float()
    qf = None if state_only else q.float()
    for t in range(n):
        state.mul_(torch.exp(gate[:, t]).unsqueeze(-1))                      # row c of every head's state decays by its own gate
        pred = torch.einsum("bhc,bhcv->bhv", kf[:, t], state)
        delta = (vf[:, t] - pred) * beta[:, t].unsqueeze(-1)
        state.add_(kf[:, t].unsqueeze(-1) * delta.unsqueeze(-2))
        if not state_only:
            out[:, t] = torch.einsum("bhc,bhcv->bhv", qf[:, t], state) * D ** -0.5
    o = None if state_only else out.to(q.dtype)
    return (o, state, gate, beta) if output_aux else (o, state)


def KimiK3RecurrentKDAOutputOnly(q, k, v, raw_gate, raw_beta, a_log, dt_bias, lower_bound=-5.0, state=None):
    return KimiK3RecurrentKDA(q, k, v, raw_gate, raw_beta, a_log, dt_bias, lower_bound, state, output_aux=False)


def KimiK3RecurrentKDAUpdateState(k, v, raw_gate, raw_beta, a_log, dt_bias, lower_bound, tokens, state):
    return KimiK3RecurrentKDA(None, k, v, raw_gate, raw_beta, a_log, dt_bias, lower_bound, state, output_aux=False, tokens=tokens,
                              state_only=True)[1]


def KimiK3AttnRes(prefix_sum, block_residual, projection, norm, eps=1e-5):
    """Attention over residual blocks: every candidate (the running prefix sum and each stored block residual,
    ``[tokens, blocks, hidden]``) is scored by its RMS-normalised projection on ``norm * projection``; the output is the
    softmax-weighted mix of the candidates."""
    w = (norm.float() * projection.float())
    cand = torch.cat([block_residual.float(), prefix_sum.float().unsqueeze(1)], dim=1)            # [T, blocks + 1, hidden]
    scores = (cand * torch.rsqrt(cand.pow(2).mean(-1, keepdim=True) + eps) * w).sum(-1)
    p = torch.softmax(scores, dim=-1)
    return (p.unsqueeze(-1) * cand).sum(1).to(prefix_sum.dtype)


def KimiK3CausalAttention(q, k, v, scale):
    """Plain causal softmax attention over ``[batch, seq, heads, dim]`` (grouped KV heads are repeated)."""
    Bn, S, H, D = q.shape
    rep = H // k.shape[2]
    kf, vf = k.float().repeat_interleave(rep, 2), v.float().repeat_interleave(rep, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) * scale
    s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=q.device), 1), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vf).to(q.dtype)


def KimiK3RoutedExperts(x, index, score, w1s, w2s, w3s, beta=1.0, linear_beta=0.0):
    """Routed experts with the SiTU activation: ``sum_k score * w2[e](situ(w1[e] x) * bound(w3[e] x))``."""
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    T, topk = index.shape
    for t in range(T):
        for j in range(topk):
            e = int(index[t, j])
            h = KimiK3SiTUAndMul(Linear(x[t:t + 1], w1s[e]), Linear(x[t:t + 1], w3s[e]), beta, linear_beta)
            out[t] += float(score[t, j]) * Linear(h, w2s[e])[0].float()
    return out.to(x.dtype)


# ---- process-wide settings under the reference's names (the implementations live in fastllm_b200.llm) --------------
def _llm():
    from .. import llm

    return llm


def SetThreads(n): _llm().set_cpu_threads(n)
def GetThreads(): return _llm().get_cpu_threads()
def SetLowMemMode(on): _llm().set_cpu_low_mem(on)
def GetLowMemMode(): return _llm().get_cpu_low_mem()
def SetKVCacheInCPU(on): _llm().set_cpu_kvcache(on)
def GetKVCacheInCPU(): return _llm().get_cpu_kvcache()
def SetHistoryCacheInCPU(on): _llm().set_cpu_historycache(on)
def GetHistoryCacheInCPU(): return _llm().get_cpu_historycache()
def SetCudaEmbedding(on): _llm().set_cuda_embedding(on)
def GetCudaEmbedding(): return bool(_llm()._settings.get("cuda_embedding", True))
GetCudaEmbeddingRequested = GetCudaEmbedding
def SetCudaSharedExpert(on): _llm().set_cuda_shared_expert(on)
def GetCudaSharedExpert(): return bool(_llm()._settings.get("cuda_shared_expert", True))
def SetCudaSlabMB(mb): _llm().set_cuda_slab(mb)
def GetCudaSlabMB(): return int(_llm()._settings.get("cuda_slab", 0) or 0)
def EnableAMX(on): _llm().set_enable_amx(on)
def GetEnableAMX(): return bool(_llm()._settings.get("enable_amx", False))
def SetGpuMemRatio(r): _llm().set_gpu_mem_ratio(r)
def GetGpuMemRatio(): return float(_llm()._settings.get("gpu_mem_ratio", 0.9) or 0.9)
def SetMaxTokens(n): _llm().set_max_tokens(n)
def GetMaxTokens(): return _llm()._settings.get("max_tokens")
def SetPageLen(n): _llm().set_page_size(n)
def GetPageLen(): return int(_llm()._settings.get("page_size", 128) or 128)
def SetMoeDeviceLayers(n): _llm().set_moe_device_layers(n)
def GetMoeDeviceLayers(): return int(_llm()._settings.get("moe_device_layers", -1) or -1)
def SetDeviceMap(device_map): _llm().set_device_map(device_map)
def SetMoeDeviceMap(device_map): _llm().set_device_map(device_map, is_moe=True)
def SetLayeredMoeDeviceMap(device_map): _llm().set_layered_moe_device_map(device_map)
def SetModelLoadProgressCallback(cb): _llm().set_model_load_progress_callback(cb)
def ClearModelLoadProgressCallback(): _llm().set_model_load_progress_callback(None)


def ReportModelLoadProgress(stage, current, total):
    from ..serving import progress

    progress.emit(stage, current, total)


def HasDeviceType(name) -> bool: return bool(_llm().has_device(name))
def PrintInstructionInfo(): return _llm().print_ins_info()


def SelectDeviceFromMap(device_map: dict, layer: int, n_layers: int) -> str:
    """Device of ``layer`` under a ratio map like ``{'cuda:0': 3, 'cuda:1': 1}`` (layers are split in proportion, in order)."""
    from ..loader.shard import split_layers_by_map

    return str(split_layers_by_map(n_layers, device_map)[layer])


def ApplyDeviceMap(device_map: dict, layer: int, n_layers: int) -> str:
    return SelectDeviceFromMap(device_map, layer, n_layers)


def SetCurrentThreadExecutor(executor=None):
    """Install the executor ``ops.executor.GetExecutor`` returns (device order, forced placement, operand migration)."""
    from . import executor as E

    E.SetCurrentThreadExecutor(executor)


def ClearAllPagedCacheManagers():
    """Paged caches belong to engines here; dropping the engines frees them.  Releases cached allocator blocks."""
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def ClearProfiler():
    """Start a fresh per-kernel timing table (``ops._lib.KernelProfile``)."""
    from . import _lib

    _lib.start_profile()


def PrintProfiler():
    from . import _lib

    p = _lib.stop_profile()
    if p is not None:
        for name, row in sorted(p.report().items(), key=lambda kv: -kv[1].get("ms", 0.0) if isinstance(kv[1], dict) else 0.0):
            print(name, row)


def GetModelTypeFromFile(path: str) -> str:
    """``model_type`` of a checkpoint folder (config.json), a GGUF file (``general.architecture``) or a ``.flm`` file."""
    import json
    import os

    if os.path.isdir(path):
        return str(json.load(open(os.path.join(path, "config.json"))).get("model_type", ""))
    if path.endswith(".gguf"):
        from ..loader import gguf

        return str(gguf.GGUFFile(path).meta.get("general.architecture", ""))
    from ..loader import flm

    return str(flm.read_flm(path)[0].get("model_type", ""))


_step3p5_tables: dict = {}


def Step3p5QKVRMSNormRopeSplitAppendPagedCache(qkv, q_norm_w, k_norm_w, positions, slots, k_pool, v_pool, q_heads, k_heads, head_dim,
                                               rotary_dim, eps, rope_theta, use_llama3=False, llama3_factor=1.0,
                                               llama3_original_max_position=8192, llama3_low_freq_factor=1.0,
                                               llama3_high_freq_factor=4.0, max_positions=131072):
    """Step-3.5 form of the fused QKV post-processing: per-head RMSNorm of Q and K with zero-centred weights (``1 + w``),
    partial rotary embedding with optional Llama-3 frequency scaling, K / V appended to the paged pools.  The same kernel as
    ``QKVRMSNormRopeSplitAppendPagedCache``; the scaling only changes the cos / sin table (cached per setting)."""
    key = (rotary_dim, float(rope_theta), bool(use_llama3), float(llama3_factor), float(llama3_original_max_position),
           float(llama3_low_freq_factor), float(llama3_high_freq_factor), int(max_positions), str(qkv.device))
    if key not in _step3p5_tables:
        scaling = None
        if use_llama3:
            scaling = {"rope_type": "llama3", "factor": llama3_factor, "original_max_position_embeddings": llama3_original_max_position,
                       "low_freq_factor": llama3_low_freq_factor, "high_freq_factor": llama3_high_freq_factor}
        _step3p5_tables[key] = A.build_rope_tables(rotary_dim, max_positions, rope_theta, scaling, device=qkv.device)
    cos, sin = _step3p5_tables[key]
    return A.qkv_post(qkv, positions, slots, k_pool, v_pool, q_heads, k_heads, head_dim, cos, sin, A.ROPE_NEOX, rotary_dim, q_norm_w, k_norm_w,
                      eps, 1.0)
