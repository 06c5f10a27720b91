"""Mixture-of-experts operators: router top-k, expert FFN, and the latent (MLA) paged attention.

Router semantics follow the reference's ``SelectExpert`` (src/devices/cpu/cpudevice.cpp:8885-8955): the
top-k is taken on ``score + bias`` while the returned weight is the un-biased score, optionally
renormalised and multiplied by ``route_scale``.  Group-limited routing (DeepSeek-V3: keep the
``topk_group`` best of ``n_group`` expert groups, ranked by the sum of their two best biased scores)
does not exist in the reference; it is implemented to the Hugging Face DeepSeek-V3 definition.
"""
from __future__ import annotations

import ctypes

import os

import torch
import torch.nn.functional as F

from . import _lib
from . import basic as B
from .basic import _ptr, _stream
from .quant import LinearWeight


# ---------------------------------------------------------------------------------------------------
def route_topk_ref(logits, bias, topk, score_mode, renorm, n_group=1, topk_group=1, route_scale=1.0):
    lf = logits.float()
    if score_mode == 0:
        sc = torch.softmax(lf, dim=-1)
    elif score_mode == 1:
        sc = torch.sigmoid(lf)
    else:
        sc = lf
    sel = sc + bias.float() if bias is not None else sc.clone()
    M, E = sc.shape
    if n_group > 1 and topk_group < n_group:
        gs = sel.view(M, n_group, E // n_group).topk(2, dim=-1)[0].sum(-1)
        gidx = gs.topk(topk_group, dim=-1)[1]
        gmask = torch.zeros_like(gs).scatter_(1, gidx, 1.0)
        emask = gmask[:, :, None].expand(M, n_group, E // n_group).reshape(M, E)
        sel = sel.masked_fill(emask == 0, float("-inf"))
    idx = sel.topk(topk, dim=-1)[1]
    w = sc.gather(1, idx)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx.to(torch.int32), (w * route_scale).float()


def route_topk(logits, bias, topk, score_mode, renorm, n_group=1, topk_group=1, route_scale=1.0):
    """logits fp32 ``[M, E]`` -> (expert index int32 ``[M, topk]``, weight fp32 ``[M, topk]``)."""
    if not logits.is_cuda or logits.shape[1] > 512:
        return route_topk_ref(logits, bias, topk, score_mode, renorm, n_group, topk_group, route_scale)
    lg = logits.float().contiguous()
    M, E = lg.shape
    idx = torch.empty((M, topk), device=lg.device, dtype=torch.int32)
    w = torch.empty((M, topk), device=lg.device, dtype=torch.float32)
    b = bias.float().contiguous() if bias is not None else None
    rc = _lib.kernels().fb_route_topk(_ptr(lg), _ptr(b), _ptr(idx), _ptr(w), M, E, topk, score_mode, 1 if renorm else 0,
                                      n_group, topk_group, float(route_scale), _stream())
    _lib.check(rc, "fb_route_topk")
    return idx, w


# router projection and expert selection in one launch (csrc/gemm_bf16.cu::gemm_route_kernel), FB_ROUTE_FUSED=1.  Off by default:
# measured on Qwen3-30B-A3B (128 rows, 128 experts, top-8) the one-launch form is 0.2 ms per step SLOWER than GEMM + selection
# kernel (12.33 against 11.98 - 12.21 ms): the selection then runs on the eight CTAs of the GEMM's cluster, 16 tokens each,
# instead of on 32 CTAs that start under the GEMM's tail.
ROUTE_FUSED = __import__("os").environ.get("FB_ROUTE_FUSED", "0") == "1"


def route_fused_ok(x, router_16, topk, n_group=1, topk_group=1) -> bool:
    """The fused kernel covers decode-sized batches (<= 128 rows) of up to 128 experts without group-limited selection."""
    return bool(ROUTE_FUSED and x.is_cuda and x.dim() == 2 and x.dtype in (torch.float16, torch.bfloat16) and router_16 is not None
                and router_16.dtype == x.dtype and x.shape[0] <= 128 and router_16.shape[0] <= 128 and x.shape[1] % 64 == 0
                and topk <= min(32, router_16.shape[0]) and not (n_group > 1 and topk_group < n_group)
                and x.stride(1) == 1 and router_16.is_contiguous())


def route_fused(x, router_16, bias, topk, score_mode, renorm, route_scale=1.0):
    """``route_topk(x @ router^T, ...)`` as one kernel: (expert index int32 ``[M, topk]``, weight fp32 ``[M, topk]``)."""
    M, K = x.shape
    E = router_16.shape[0]
    idx = torch.empty((M, topk), device=x.device, dtype=torch.int32)
    w = torch.empty((M, topk), device=x.device, dtype=torch.float32)
    b = bias.float().contiguous() if bias is not None else None
    rc = _lib.kernels().fb_gemm_route(_ptr(x), _ptr(router_16), M, E, K, x.stride(0), K, 1 if x.dtype == torch.bfloat16 else 0, _ptr(b),
                                      _ptr(idx), _ptr(w), topk, score_mode, 1 if renorm else 0, float(route_scale), _stream())
    _lib.check(rc, "fb_gemm_route")
    return idx, w


def route_group_top1(logits, groups: int, expert_scale=None):
    """Mixture of grouped experts (Pangu Pro MoE): the experts form ``groups`` equal, contiguous groups and the best-scoring
    expert of every group is taken; weight = softmax score (over all experts) x the expert's learned scale, not renormalised.
    Reference: src/models/pangu_moe.cpp:392-430.  Tensor ops only (CUDA-graph safe)."""
    sc = torch.softmax(logits.float(), dim=-1)
    M, E = sc.shape
    per = E // groups
    val, j = sc.view(M, groups, per).max(dim=-1)
    idx = j + torch.arange(groups, device=sc.device)[None, :] * per
    if expert_scale is not None:
        val = val * expert_scale.float()[idx]
    return idx.to(torch.int32), val.float()


# ---------------------------------------------------------------------------------------------------
class ExpertWeights:
    """Routed experts owned by this rank: per-expert gate/up (tile-interleaved) and down weights."""

    def __init__(self, num_experts_total: int, first: int, gate_up: list[LinearWeight], down: list[LinearWeight]):
        self.total = num_experts_total
        self.first = first
        self.count = len(gate_up)
        self.gate_up = gate_up
        self.down = down
        self.stacked = None     # filled by ops.moe_grouped when a grouped kernel can take the whole set
        self.act = "swiglu"     # "gptoss": clamped gate/up, gate * sigmoid(1.702 gate) * (up + 1); "swiglu_clamp": see limit
        self.limit = 0.0        # "swiglu_clamp" (Step-3.5): min(silu(gate), limit) * clamp(up, -limit, limit)
        self.host = False       # expert weights live in CPU memory and run on the native CPU backend (hybrid placement)
        self._host_arrays = None


def glu_gptoss(gu, interleaved: bool, limit: float = 7.0, alpha: float = 1.702):
    """gpt-oss expert activation on a ``[gate | up]`` projection (tile-interleaved when ``interleaved``)."""
    if interleaved:
        n = gu.shape[-1]
        t = gu.reshape(*gu.shape[:-1], n // 128, 2, 64)
        g, u = t[..., 0, :].reshape(*gu.shape[:-1], n // 2), t[..., 1, :].reshape(*gu.shape[:-1], n // 2)
    else:
        g, u = gu.chunk(2, dim=-1)
    g = g.float().clamp(max=limit)
    u = u.float().clamp(min=-limit, max=limit)
    return ((u + 1.0) * (g * torch.sigmoid(g * alpha))).to(gu.dtype)


def glu_clamped(gu, interleaved: bool, limit: float):
    """SwiGLU with the activated gate capped at ``limit`` and the up branch clamped to ``[-limit, limit]``
    (reference: src/models/step3p5.cpp:6604-6612)."""
    if interleaved:
        n = gu.shape[-1]
        t = gu.reshape(*gu.shape[:-1], n // 128, 2, 64)
        g, u = t[..., 0, :].reshape(*gu.shape[:-1], n // 2), t[..., 1, :].reshape(*gu.shape[:-1], n // 2)
    else:
        g, u = gu.chunk(2, dim=-1)
    a = torch.nn.functional.silu(g.float())
    if limit:
        a, u = a.clamp(max=limit), u.float().clamp(min=-limit, max=limit)
    return (a * u.float()).to(gu.dtype)


def local_expert_range(num_experts: int, ep) -> tuple[int, int]:
    """Contiguous block of experts owned by this expert-parallel rank."""
    if ep is None or ep.size == 1:
        return 0, num_experts
    per = (num_experts + ep.size - 1) // ep.size
    lo = min(num_experts, ep.rank * per)
    return lo, min(num_experts, lo + per)


def output_is_complete(ep) -> bool:
    """True when moe_forward already returns the sum over all ranks' experts."""
    return bool(ep is not None and getattr(ep, "combines", False))


def moe_forward(x, idx, wts, experts: ExpertWeights, ep=None):
    """``y[t] = sum_k wts[t,k] * down_e(silu(gate_e x) * up_e x)`` over the experts this rank owns.

    Tokens are grouped by expert; each non-empty local expert runs the two GEMMs on its token group.
    With expert parallelism the result is this rank's partial sum (the caller all-reduces it).
    """
    if experts.host and experts.act == "swiglu":
        return _moe_forward_host(x, idx, wts, experts)
    if experts.stacked is not None and x.is_cuda and experts.act == "swiglu":
        from . import moe_grouped

        y = moe_grouped.forward(x, idx, wts, experts)
        if y is not None:
            return y
    T, H = x.shape
    y = torch.zeros((T, H), device=x.device, dtype=torch.float32)
    flat_e = idx.reshape(-1).long()
    flat_t = torch.arange(T, device=x.device).repeat_interleave(idx.shape[1])
    flat_w = wts.reshape(-1)
    local = (flat_e >= experts.first) & (flat_e < experts.first + experts.count)
    if not bool(local.any()):
        return y.to(x.dtype)
    order = torch.argsort(flat_e[local], stable=True)
    e_sorted = flat_e[local][order]
    t_sorted = flat_t[local][order]
    w_sorted = flat_w[local][order]
    uniq, counts = torch.unique_consecutive(e_sorted, return_counts=True)
    start = 0
    for e, n in zip(uniq.tolist(), counts.tolist()):
        rows = t_sorted[start:start + n]
        xe = x.index_select(0, rows)
        le = e - experts.first
        if experts.act == "gptoss":
            he = experts.down[le](glu_gptoss(experts.gate_up[le](xe), experts.gate_up[le].interleaved))
        elif experts.act == "swiglu_clamp":
            he = experts.down[le](glu_clamped(experts.gate_up[le](xe), experts.gate_up[le].interleaved, experts.limit))
        else:
            he = experts.down[le](experts.gate_up[le](xe, swiglu=True))
        y.index_add_(0, rows, he.float() * w_sorted[start:start + n, None])
        start += n
    return y.to(x.dtype)


_MLA_KERNEL = True      # tests switch this off to compare the kernel with the PyTorch evaluation


def _moe_forward_host(x, idx, wts, experts: ExpertWeights):
    """Routed experts on the host: activations cross PCIe once per layer in each direction, expert weights never move
    (reference: ``--moe_device cpu``, tools/fastllm_pytools/util.py:818-826; docs/mixforward.md)."""
    import ctypes

    from ..models import cpu_native as CN
    from . import cpu

    L = cpu.lib()
    if experts._host_arrays is None:
        keep = []

        class _K:          # minimal holder with the interface NativeCpuModel._lin expects
            def __init__(self):
                self.keep = keep

            _f32 = CN.NativeCpuModel._f32
            _lin = CN.NativeCpuModel._lin

        k = _K()
        n = experts.count
        G = (CN._Lin * n)(*[k._lin(l) for l in experts.gate_up])
        D = (CN._Lin * n)(*[k._lin(l) for l in experts.down])
        L.fbcpu_moe.restype = ctypes.c_int
        L.fbcpu_moe.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        experts._host_arrays = (G, D, keep)
        L.fbnuma_create.restype = ctypes.c_void_p
        L.fbnuma_create.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        L.fbnuma_destroy.argtypes = [ctypes.c_void_p]
        L.fbnuma_moe.restype = ctypes.c_int
        L.fbnuma_moe.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                 ctypes.c_int, ctypes.c_void_p]
        if getattr(experts, "numa", False) and experts.act == "swiglu":
            # every expert cut across the memory nodes; the slices are copies made by the nodes' own threads
            experts._numa_handle = L.fbnuma_create(G, D, n, int(os.environ.get("FB_NUMA_THREADS_PER_NODE", "0")))
    G, D, _ = experts._host_arrays
    T, H = x.shape
    xh = x.detach().to("cpu", torch.float32).contiguous()
    ih = idx.detach().to("cpu", torch.int32).contiguous()
    wh = wts.detach().to("cpu", torch.float32).contiguous()
    out = torch.zeros((T, H), dtype=torch.float32)
    nh = getattr(experts, "_numa_handle", None)
    if nh:
        rc = L.fbnuma_moe(ctypes.c_void_p(nh), xh.data_ptr(), T, H, ih.data_ptr(), wh.data_ptr(), idx.shape[1], experts.first, out.data_ptr())
    else:
        rc = L.fbcpu_moe(xh.data_ptr(), T, H, ih.data_ptr(), wh.data_ptr(), idx.shape[1], experts.first, experts.count, G, D, out.data_ptr())
    if rc != 0:
        raise RuntimeError(f"host MoE failed ({rc})")
    return out.to(x.device, x.dtype)


# ---------------------------------------------------------------------------------------------------
def dsa_select(q_idx, w_idx, idx_pool, fb, topk: int):
    """Sparse-attention selection (DeepSeek-V3.2 / GLM-MoE-DSA indexer): for every query row the ``topk`` keys with the largest
    index score  sum_h w[t, h] * relu(q_idx[t, h] . k_idx[s]) / sqrt(Di)  among the keys it may see.  q_idx ``[T, Hi, Di]``,
    w_idx fp32 ``[T, Hi]``, idx_pool ``[pages, page_len, 1, Di]`` (the index keys of every cached token).  Returns, per request,
    a bool mask ``[rows, L]`` of selected keys (None where the whole context fits into ``topk``)."""
    page_len, Di = idx_pool.shape[1], idx_pool.shape[-1]
    cu = fb.cu_q_host if fb.cu_q_host is not None else fb.cu_q.tolist()
    kv_lens = fb.kv_lens.tolist()
    out = []
    for b in range(len(cu) - 1):
        q0, q1 = cu[b], cu[b + 1]
        L = kv_lens[b]
        if q1 == q0 or L <= topk:
            out.append(None)
            continue
        npg = (L + page_len - 1) // page_len
        kk = idx_pool[fb.page_table[b, :npg].long()].reshape(-1, Di)[:L].float()
        sc = torch.relu(torch.einsum("qhd,kd->qhk", q_idx[q0:q1].float(), kk) * (Di ** -0.5))
        score = torch.einsum("qhk,qh->qk", sc, w_idx[q0:q1])
        nq = q1 - q0
        qpos = torch.arange(L - nq, L, device=score.device)[:, None]
        kpos = torch.arange(L, device=score.device)[None, :]
        score = score.masked_fill(kpos > qpos, float("-inf"))
        top = score.topk(min(topk, L), dim=-1).indices
        out.append(torch.zeros((nq, L), dtype=torch.bool, device=score.device).scatter_(1, top, True))
    return out


def mla_paged_attention(q_full, lat_pool, fb, scale, lora, select=None):
    """Absorbed MLA over the paged latent cache.

    q_full: ``[T, H, lora + rope]`` (q_nope already multiplied by W_UK); lat_pool: ``[pages, page_len, 1,
    lora + rope]``.  Scores use all ``lora + rope`` dims, values are the first ``lora`` dims.  Returns
    ``[T, H, lora]``.  (Reference: MergeMLAPaged, src/devices/cuda/attention/fastllm-attention.cu:3619-3727.)
    """
    T, H, Dq = q_full.shape
    sparse = select is not None and any(m_ is not None for m_ in select)
    if (not sparse and _MLA_KERNEL and fb.is_decode and q_full.is_cuda and lora == 512 and Dq == 576 and q_full.dtype in (torch.float16, torch.bfloat16)
            and lat_pool.dtype == q_full.dtype and lat_pool.shape[1] == 128):
        from .attention import mla_decode

        return mla_decode(q_full, lat_pool, fb.page_table, fb.kv_lens, scale)
    out = torch.zeros((T, H, lora), device=q_full.device, dtype=q_full.dtype)
    page_len = lat_pool.shape[1]
    cu = fb.cu_q_host if fb.cu_q_host is not None else fb.cu_q.tolist()
    kv_lens = fb.kv_lens.tolist()
    on_tc = _MLA_KERNEL and q_full.is_cuda and q_full.dtype in (torch.float16, torch.bfloat16) and Dq % 64 == 0 and lora % 8 == 0
    for b in range(len(cu) - 1):
        q0, q1 = cu[b], cu[b + 1]
        if q1 == q0:
            continue
        L = kv_lens[b]
        npg = (L + page_len - 1) // page_len
        lat16 = lat_pool[fb.page_table[b, :npg].long()].reshape(-1, Dq)
        nq = q1 - q0
        qpos = torch.arange(L - nq, L, device=q_full.device)
        keep = select[b] if select is not None else None
        if on_tc and keep is None:
            # Prefill: every head attends to the SAME latent rows, so the heads fold into the row dimension and both
            # contractions are plain GEMMs on the tensor-core kernels: S[(q, h), k] = Q' . lat^T with fp32 output, softmax in
            # fp32, O = P . lat[:, :lora].  Keys are padded to a multiple of 64 (their probabilities are exactly zero).
            Lp = (L + 63) // 64 * 64
            latp = lat16[:Lp] if lat16.shape[0] >= Lp else torch.cat([lat16, lat16.new_zeros(Lp - lat16.shape[0], Dq)])
            s = B.linear(q_full[q0:q1].reshape(nq * H, Dq), latp.contiguous(), out_f32=True).view(nq, H, Lp)
            p = torch.empty((nq * H, Lp), device=s.device, dtype=q_full.dtype)
            rc = _lib.kernels().fb_softmax_causal_rows(_ptr(s), Lp, _ptr(p), Lp, nq * H, Lp, H, L - nq, float(scale),
                                                       B.dtype_code(q_full.dtype), _stream())
            _lib.check(rc, "fb_softmax_causal_rows")
            out[q0:q1] = B.linear(p, latp[:, :lora].t().contiguous()).view(nq, H, lora)
            continue
        lat = lat16[:L].float()
        s = torch.einsum("qhd,kd->hqk", q_full[q0:q1].float(), lat) * scale
        kpos = torch.arange(L, device=s.device)[None, :]
        s = s.masked_fill(kpos > qpos[:, None], float("-inf"))
        if keep is not None:                       # sparse attention: only the selected keys of every query row
            s = s.masked_fill(~keep[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.einsum("hqk,kl->qhl", p, lat[:, :lora]).to(out.dtype)
    return out
