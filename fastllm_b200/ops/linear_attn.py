"""Gated-DeltaNet linear attention (Qwen3-Next, Qwen3.5): causal depth-wise convolution with a rolling state, the gated
delta rule in recurrent (decode) and chunked (prefill) form, and the gated RMSNorm that follows it.

Reference operators: ``Conv1DPerChannel`` / the ShiftAppendConv1D family (src/devices/cuda/fastllm-cuda.cu:14131-15096),
``RecurrentGatedDeltaRule`` (:16514-17912), ``ChunkGatedDeltaRulePrefill`` with its helpers ``CumSumLastDim`` /
``MakeDecayMask`` / ``CausalMask`` (:6610-6831, 18717-19217); model use in src/models/qwen3_next.cpp and qwen3_5.cpp.

Per request the layer keeps two pieces of state instead of K/V pages:
    conv state  ``[C, K-1]``      the last K-1 inputs of every convolution channel
    rule state  ``[Hv, Dk, Dv]``  fp32, the delta-rule memory of every value head
Both live in per-layer pools indexed by a *state slot* that the engine assigns to a running request.

With ``q, k`` L2-normalised per head, ``q`` scaled by ``Dk^-1/2``, decay ``g_t <= 0`` and write strength ``beta_t``:

    S_t = exp(g_t) S_{t-1} + k_t (beta_t (v_t - (exp(g_t) S_{t-1})^T k_t))^T ,      o_t = S_t^T q_t

CUDA tensors of decode steps run ``csrc/linear_attn.cu`` (one CTA per (request, value head), the state column of a
thread in registers); everything else is the PyTorch definition below, which is also the test oracle.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from .basic import _ptr, _stream, dtype_code

P, I, FLT = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_lib.register_sigs({
    "fb_gdn_conv_update": [P, P, P, P, P, I, I, I, I, I, P],
    "fb_gdn_recurrent": [P, I, P, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, FLT, I, P],
}, ["linear_attn"])

CHUNK = 64


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def rmsnorm_gated(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``w * norm(x)`` in the input dtype, then times ``silu(z)`` (norm before gate)."""
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return ((w * y).float() * F.silu(z.float())).to(x.dtype)


# ---------------------------------------------------------------------------------------------------------------
# causal depth-wise convolution over packed sequences, with the rolling per-request state
# ---------------------------------------------------------------------------------------------------------------
def causal_conv1d(x: torch.Tensor, w: torch.Tensor, conv_state: torch.Tensor, cu_q, slots) -> torch.Tensor:
    """x ``[T, C]`` packed tokens of B requests (``cu_q`` host list of B+1 offsets); w ``[C, K]``; conv_state ``[S, C, K-1]``;
    slots: host list of B state slots.  Returns ``silu(conv(x))`` ``[T, C]`` and advances each request's state."""
    K = w.shape[1]
    out = torch.empty_like(x)
    wf = w.float()
    for b, slot in enumerate(slots):
        t0, t1 = cu_q[b], cu_q[b + 1]
        if t1 <= t0:
            continue
        hist = conv_state[slot].float()                             # [C, K-1]
        seq = torch.cat([hist, x[t0:t1].float().t()], dim=1)         # [C, K-1 + n]
        conv_state[slot] = seq[:, -(K - 1):].to(conv_state.dtype)
        y = F.conv1d(seq.unsqueeze(0), wf.unsqueeze(1), groups=wf.shape[0])[0]   # [C, n]
        out[t0:t1] = F.silu(y).t().to(x.dtype)
    return out


def causal_conv1d_decode(x: torch.Tensor, w: torch.Tensor, conv_state: torch.Tensor, slots_dev: torch.Tensor) -> torch.Tensor:
    """One token per request: x ``[B, C]``, slots_dev int32 ``[B]`` on the device.  One launch on CUDA."""
    B, C = x.shape
    K = w.shape[1]
    if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and conv_state.dtype == x.dtype and w.dtype == x.dtype and K <= 8:
        out = torch.empty_like(x)
        rc = _lib.kernels().fb_gdn_conv_update(_ptr(x), _ptr(w), _ptr(conv_state), _ptr(slots_dev), _ptr(out), B, C, K, x.stride(0),
                                               dtype_code(x.dtype), _stream())
        _lib.check(rc, "fb_gdn_conv_update")
        return out
    sl = slots_dev.long()
    hist = conv_state[sl].float()                                    # [B, C, K-1]
    seq = torch.cat([hist, x.float().unsqueeze(-1)], dim=-1)         # [B, C, K]
    conv_state[sl] = seq[:, :, 1:].to(conv_state.dtype)
    return F.silu((seq * w.float().unsqueeze(0)).sum(-1)).to(x.dtype)


# ---------------------------------------------------------------------------------------------------------------
# gated delta rule
# ---------------------------------------------------------------------------------------------------------------
def gated_delta_recurrent_ref(q, k, v, g, beta, state):
    """One sequence, token by token.  q, k ``[n, H, Dk]`` (already normalised and scaled), v ``[n, H, Dv]``, g, beta ``[n, H]``,
    state ``[H, Dk, Dv]`` fp32 (updated in place).  Returns ``[n, H, Dv]`` fp32."""
    n = q.shape[0]
    out = torch.empty(n, v.shape[1], v.shape[2], dtype=torch.float32, device=q.device)
    S = state
    for t in range(n):
        S.mul_(g[t].exp()[:, None, None])
        kv = (S * k[t][:, :, None]).sum(1)                           # [H, Dv]
        delta = (v[t] - kv) * beta[t][:, None]
        S.add_(k[t][:, :, None] * delta[:, None, :])
        out[t] = (S * q[t][:, :, None]).sum(1)
    return out


def gated_delta_chunked(q, k, v, g, beta, state, chunk: int = CHUNK):
    """Same result as the recurrence, computed chunk by chunk with matrix products (the WY / UT-transform form):
    inside a chunk the rule is solved as a unit-lower-triangular system, between chunks the state is carried.
    Shapes as in ``gated_delta_recurrent_ref``."""
    n, H, Dk = q.shape
    Dv = v.shape[-1]
    pad = (chunk - n % chunk) % chunk
    if pad:
        zf = lambda t: F.pad(t, (0, 0) * (t.dim() - 1) + (0, pad))
        q, k, v, g, beta = zf(q), zf(k), zf(v), zf(g), zf(beta)
    N = q.shape[0] // chunk
    # [H, N, c, D]
    rs = lambda t: t.permute(1, 0, 2).reshape(H, N, chunk, t.shape[-1])
    qc, kc, vc = rs(q), rs(k), rs(v)
    gc = g.t().reshape(H, N, chunk)
    bc = beta.t().reshape(H, N, chunk)
    gcs = gc.cumsum(-1)                                               # running log-decay inside the chunk
    kb, vb = kc * bc[..., None], vc * bc[..., None]
    decay = (gcs[..., :, None] - gcs[..., None, :]).tril().exp().tril()       # [H, N, c, c], exp(G_i - G_j) for j <= i
    eye = torch.eye(chunk, device=q.device, dtype=torch.float32)
    strict = torch.tril(torch.ones(chunk, chunk, device=q.device, dtype=torch.bool), -1)
    A = -(kb @ kc.transpose(-1, -2) * decay).masked_fill(~strict, 0)
    # (I - A)^-1 by forward substitution on the rows (unit lower triangular)
    T = A.clone()
    for i in range(1, chunk):
        T[..., i, :i] = T[..., i, :i] + (T[..., i, :i, None] * T[..., :i, :i]).sum(-2)
    T = T + eye
    u = T @ vb                                                        # "new values" before removing the carried state
    w = T @ (kb * gcs.exp()[..., None])
    out = torch.empty(H, N, chunk, Dv, device=q.device, dtype=torch.float32)
    S = state
    upper = torch.triu(torch.ones(chunk, chunk, device=q.device, dtype=torch.bool), 1)
    for c in range(N):
        qi, ki, ui, wi = qc[:, c], kc[:, c], u[:, c], w[:, c]
        attn = (qi @ ki.transpose(-1, -2) * decay[:, c]).masked_fill(upper, 0)
        v_new = ui - wi @ S                                            # [H, c, Dv]
        out[:, c] = (qi * gcs[:, c, :, None].exp()) @ S + attn @ v_new
        glast = gcs[:, c, -1]
        S = S * glast.exp()[:, None, None] + (ki * (glast[:, None] - gcs[:, c]).exp()[..., None]).transpose(-1, -2) @ v_new
    state.copy_(S)
    return out.reshape(H, N * chunk, Dv)[:, :n].permute(1, 0, 2)


def gated_delta_rule(q, k, v, a, b, A_log, dt_bias, rec_state, cu_q, slots, rep: int):
    """Packed prefill / mixed batches.  q, k ``[T, Hk, Dk]``, v ``[T, Hv, Dv]`` (post-convolution), a, b ``[T, Hv]`` raw gate
    projections; ``rep = Hv / Hk``.  Returns ``[T, Hv, Dv]`` in v's dtype; advances ``rec_state[slot]`` of every request."""
    Dk = q.shape[-1]
    qf = l2norm(q.float()) * (Dk ** -0.5)
    kf = l2norm(k.float())
    if rep > 1:
        qf, kf = qf.repeat_interleave(rep, dim=1), kf.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(b.float())
    g = -A_log.float().exp() * F.softplus(a.float() + dt_bias.float())
    vf = v.float()
    out = torch.empty_like(vf)
    for i, slot in enumerate(slots):
        t0, t1 = cu_q[i], cu_q[i + 1]
        if t1 <= t0:
            continue
        S = rec_state[slot]
        if t1 - t0 <= 4:
            out[t0:t1] = gated_delta_recurrent_ref(qf[t0:t1], kf[t0:t1], vf[t0:t1], g[t0:t1], beta[t0:t1], S)
        else:
            out[t0:t1] = gated_delta_chunked(qf[t0:t1], kf[t0:t1], vf[t0:t1], g[t0:t1], beta[t0:t1], S)
    return out.to(v.dtype)


def gated_delta_decode(mixed, a, b, z, A_log, dt_bias, norm_w, eps, rec_state, slots_dev, Hk, Hv, Dk, Dv):
    """One token per request, everything after the convolution in one launch on CUDA: split q/k/v, L2 norms, gates, the
    state update, the read-out, and the gated RMSNorm.  mixed ``[B, 2*Hk*Dk + Hv*Dv]`` (post-convolution), a, b ``[B, Hv]``,
    z ``[B, Hv*Dv]``; returns ``[B, Hv*Dv]`` in the input dtype."""
    B = mixed.shape[0]
    if (mixed.is_cuda and mixed.dtype in (torch.float16, torch.bfloat16) and Dk == 128 and Dv == 128 and Hv % Hk == 0
            and rec_state.dtype == torch.float32 and a.dtype == mixed.dtype and z.dtype == mixed.dtype):
        out = torch.empty((B, Hv * Dv), device=mixed.device, dtype=mixed.dtype)
        rc = _lib.kernels().fb_gdn_recurrent(_ptr(mixed), mixed.stride(0), _ptr(a), a.stride(0), _ptr(b), _ptr(z), _ptr(A_log),
                                             _ptr(dt_bias), _ptr(norm_w), _ptr(rec_state), _ptr(slots_dev), _ptr(out), B, Hk, Hv, Dk, Dv,
                                             z.stride(0), float(eps), dtype_code(mixed.dtype), _stream())
        _lib.check(rc, "fb_gdn_recurrent")
        return out
    kd = Hk * Dk
    q, k, v = mixed[:, :kd].reshape(B, Hk, Dk), mixed[:, kd:2 * kd].reshape(B, Hk, Dk), mixed[:, 2 * kd:].reshape(B, Hv, Dv)
    rep = Hv // Hk
    qf = (l2norm(q.float()) * (Dk ** -0.5)).repeat_interleave(rep, dim=1)
    kf = l2norm(k.float()).repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(b.float())
    g = -A_log.float().exp() * F.softplus(a.float() + dt_bias.float())
    sl = slots_dev.long()
    S = rec_state[sl] * g.exp()[:, :, None, None]                     # [B, Hv, Dk, Dv]
    kv = (S * kf[..., None]).sum(2)
    delta = (v.float() - kv) * beta[..., None]
    S = S + kf[..., None] * delta[:, :, None, :]
    rec_state[sl] = S
    o = (S * qf[..., None]).sum(2).to(mixed.dtype)                     # [B, Hv, Dv]
    return rmsnorm_gated(o, z.reshape(B, Hv, Dv), norm_w, eps).reshape(B, Hv * Dv)


# ---------------------------------------------------------------------------------------------------
# Lightning attention (MiniMax-Text-01 / M1): linear attention with a fixed per-head exponential decay
# ---------------------------------------------------------------------------------------------------
def lightning_slopes(num_heads: int, layer_idx: int, num_layers: int) -> torch.Tensor:
    """Per-head decay rates: ``2^(-8 (h+1) / H)`` scaled down linearly with depth (the last layer decays slowest)."""
    base = 1.0 / (2.0 ** (8.0 / num_heads))
    rate = base ** (torch.arange(num_heads, dtype=torch.float32) + 1.0)
    return rate * (1.0 - layer_idx / (num_layers - 1 + 1e-5) + 1e-5)


def lightning_attention(q, k, v, slope, state, cu_q_host, slots_host, block: int = 256):
    """Packed prefill / chunked prefill.  q, k, v ``[T, H, D]``; slope fp32 ``[H]``; state fp32 ``[slots, H, D, D]`` holds
    ``sum_j decay^(t-j) k_j^T v_j`` per request and is advanced in place.  Blocks of ``block`` tokens: inside a block the
    decayed causal product, across blocks the carried state.  Returns fp32 ``[T, H, D]``.
    Reference: the lightning-attention operators of src/models/minimax.cpp."""
    T, H, D = q.shape
    out = torch.empty((T, H, D), dtype=torch.float32, device=q.device)
    s = slope.to(q.device, torch.float32).view(H, 1, 1)
    for b in range(len(cu_q_host) - 1):
        a, e = int(cu_q_host[b]), int(cu_q_host[b + 1])
        if e <= a:
            continue
        slot = int(slots_host[b])
        S = state[slot].to(torch.float32)
        qb, kb, vb = (t[a:e].to(torch.float32).transpose(0, 1) for t in (q, k, v))        # [H, n, D]
        for i0 in range(0, e - a, block):
            m = min(block, e - a - i0)
            qi, ki, vi = qb[:, i0:i0 + m], kb[:, i0:i0 + m], vb[:, i0:i0 + m]
            idx = torch.arange(1, m + 1, device=q.device, dtype=torch.float32)
            diff = idx[:, None] - idx[None, :]
            diag = torch.where(diff >= 0, torch.exp(-s * diff.clamp(min=0)), torch.zeros((), device=q.device))
            intra = torch.matmul(torch.matmul(qi, ki.transpose(-1, -2)) * diag, vi)
            inter = torch.matmul(qi * torch.exp(-s * idx[:, None]), S)
            out[a + i0:a + i0 + m] = (intra + inter).transpose(0, 1)
            S = S * torch.exp(-s * m) + torch.matmul((ki * torch.exp(-s * (m - idx)[:, None])).transpose(-1, -2), vi)
        state[slot] = S.to(state.dtype)
    return out


def lightning_decode(q, k, v, slope, state, slots):
    """One new token per request (``[B, H, D]``): ``S = decay * S + k^T v``, ``o = q S``; state rows ``slots`` updated."""
    B, H, D = q.shape
    sl = slots.long()
    S = state[sl].to(torch.float32)                                                        # [B, H, D, D]
    ratio = torch.exp(-slope.to(q.device, torch.float32)).view(1, H, 1, 1)
    S = S * ratio + k.to(torch.float32).unsqueeze(-1) * v.to(torch.float32).unsqueeze(-2)
    state[sl] = S.to(state.dtype)
    return torch.matmul(q.to(torch.float32).unsqueeze(-2), S).squeeze(-2)
