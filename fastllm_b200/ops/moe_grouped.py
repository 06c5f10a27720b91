"""Grouped expert GEMM path (CUDA): all routed experts of a layer in a handful of launches, no host synchronisation
(CUDA-graph safe).

``prepare_model`` stacks each MoE layer's dense expert weights into ``[E_local * rows, K]`` matrices the grouped kernel
addresses by expert; ``forward`` runs plan -> gather -> grouped gate/up (+SwiGLU) -> grouped down -> weighted combine.
Returns ``None`` for cases the grouped kernels do not take (quantised experts, odd shapes); the caller then uses the
per-expert loop in ``ops.moe``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from . import quant_gemm as QG
from .basic import GEMM_SWIGLU, _ptr, _stream, dtype_code

P, I = ctypes.c_void_p, ctypes.c_int
_lib.register_sigs({
    "fb_moe_plan": [P, I, I, I, I, P, P, P, P, I, P],
    "fb_moe_gather": [P, P, P, I, I, I, P],
    "fb_moe_combine": [P, P, P, P, P, I, I, I, I, P],
    "fb_moe_grouped_gemm": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P],
    "fb_moe_grouped_gemm_quant": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P],
}, ["moe"])

GRAPH_SAFE = True
PAD = 16


class StackedExperts:
    """Expert weights of one layer stacked along the row dim; quantised kinds carry stacked scales in kernel layout."""

    def __init__(self, kind, gate_up, down, n_local, inter, hidden, group=0, gu_scale=None, gu_zero=None, dn_scale=None, dn_zero=None):
        self.kind, self.gate_up, self.down, self.n_local, self.inter, self.hidden, self.group = kind, gate_up, down, n_local, inter, hidden, group
        self.gu_scale, self.gu_zero, self.dn_scale, self.dn_zero = gu_scale, gu_zero, dn_scale, dn_zero
        self.signed = False            # int8: the stacked bytes hold q - 128 (operand form of the integer tensor-core path)
        self.a8 = None                 # (gate_up scale, zero / min, down scale, zero / min) in the integer kernel's layout


def _prepare_a8(st: StackedExperts, experts) -> None:
    """Stacked scale tables for the int8-activation kernels (``[E * rows]`` per channel, ``[E * rows, K / 128]`` per group);
    int8 weight bytes are switched to q - 128 in place, once, together with the per-expert views of the same storage."""
    shift = 128.0 if st.kind == "int8" else 0.0
    if st.kind == "int8" and not st.signed:
        already = [w.signed for w in experts.gate_up + experts.down]
        if all(already):                           # the per-expert weights were switched before they were stacked
            st.signed = True
        elif any(already):
            raise RuntimeError("experts of one layer mix q and q - 128 int8 storage")
        else:
            st.gate_up.view(torch.uint8).bitwise_xor_(0x80)
            st.down.view(torch.uint8).bitwise_xor_(0x80)
            st.signed = True
            for w in experts.gate_up + experts.down:
                w.signed = True
    if st.kind == "int4g":          # the stacked (scale, min) pair tables [E, groups, N, 2] of the 16-bit route serve both
        st.a8 = (st.gu_scale, None, st.dn_scale, None)
        return
    cat = lambda ws, f: torch.cat([f(w).float().reshape(w.n, -1) for w in ws], dim=0).contiguous()
    st.a8 = (cat(experts.gate_up, lambda w: w.scale), cat(experts.gate_up, lambda w: w.zero) - shift,
             cat(experts.down, lambda w: w.scale), cat(experts.down, lambda w: w.zero) - shift)


def _stack_scales(ws):
    from .quant_gemm import _kernel_tensors

    sc, ze = zip(*[_kernel_tensors(w)[:2] for w in ws])
    scale = torch.stack([t.contiguous() for t in sc]).contiguous()
    zero = torch.stack([t.contiguous() for t in ze]).contiguous() if ze[0] is not None else None
    return scale, zero


def stack_experts(experts) -> StackedExperts | None:
    gu, dn = experts.gate_up, experts.down
    if not gu:
        return None
    kind = gu[0].kind
    if any(w.kind != kind or not w.interleaved or w.bias is not None for w in gu) or any(w.kind != kind or w.bias is not None for w in dn):
        return None
    two_i, hidden = gu[0].n, gu[0].k
    if two_i % 128 != 0 or hidden % 128 != 0 or (two_i // 2) % 64 != 0:
        return None
    g = torch.cat([w.w for w in gu], dim=0).contiguous()
    d = torch.cat([w.w for w in dn], dim=0).contiguous()
    if kind == "dense":
        return StackedExperts(kind, g, d, len(gu), two_i // 2, hidden)
    if kind == "int4g" and (gu[0].group % 64 != 0 or hidden % gu[0].group != 0 or (two_i // 2) % gu[0].group != 0):
        return None
    if kind == "fp8" and (two_i // 2) % 128 != 0:
        return None
    if kind == "fp4" and gu[0].group not in (16, 32):
        return None
    gs, gz = _stack_scales(gu)
    ds, dz = _stack_scales(dn)
    st = StackedExperts(kind, g, d, len(gu), two_i // 2, hidden, gu[0].group, gs, gz, ds, dz)
    if kind == "fp4":
        st.fp4_f16w = all(QG._kernel_tensors(w)[2] for w in gu + dn)
    return st


def prepare_model(m) -> None:
    """Stack the experts of every MoE layer; the per-expert tensors are replaced by views of the stacked matrices."""
    for lw in m.layers:
        ex = lw.mlp.experts
        if ex is None or ex.count == 0 or ex.host or ex.act != "swiglu" or any(l.bias is not None for l in ex.gate_up + ex.down):
            continue
        st = stack_experts(ex)
        if st is None:
            continue
        ex.stacked = st
        st.signed = st.kind == "int8" and all(w.signed for w in ex.gate_up + ex.down)
        two_i, H = 2 * st.inter, st.hidden
        for e in range(ex.count):       # drop the duplicate storage: per-expert weights become views of the stacked matrices
            ex.gate_up[e].w = st.gate_up[e * two_i:(e + 1) * two_i]
            ex.down[e].w = st.down[e * H:(e + 1) * H]
        if QG.INT_A8 and st.kind in ("int8", "int4g") and st.gate_up.is_cuda and (st.kind == "int8" or st.group == 128) \
                and H % 128 == 0 and st.inter % 128 == 0:
            _prepare_a8(st, ex)                    # scale tables of the integer path, before any CUDA graph is captured


def forward(x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, experts, add: torch.Tensor | None = None, combine: bool = True):
    """``combine=False`` stops before the weighted sum and returns ``(ys, pos, wts)`` for a fused cross-rank combine."""
    st = experts.stacked
    if st is None or x.dtype not in (torch.float16, torch.bfloat16):
        return None
    T, H = x.shape
    topk = idx.shape[1]
    E = st.n_local
    dev = x.device
    lib = _lib.kernels()
    rows_cap = T * topk + E * PAD + 128
    # chunk size: a few times the mean rows per expert, so the activation tile is not mostly padding; experts that get
    # more rows simply run more chunks
    mean = max(1, (T * topk) // max(1, experts.total))
    hint = 16 if mean <= 6 else 32 if mean <= 12 else 64 if mean <= 24 else 128
    if st.kind == "int4g" and QG.INT_A8 and mean <= 12:
        hint = 16          # the 16-row integer kernel has dedicated unpack warps; a second chunk re-reads its weights from L2
    max_rows = min(T, 0xFFFF) | (hint << 16)
    counts = torch.empty(E, device=dev, dtype=torch.int32)
    offsets = torch.empty(E, device=dev, dtype=torch.int32)
    pos = torch.empty((T, topk), device=dev, dtype=torch.int32)
    total = torch.empty(1, device=dev, dtype=torch.int32)
    idx = idx.contiguous()
    wts = wts.float().contiguous()
    s = _stream()
    _lib.check(lib.fb_moe_plan(_ptr(idx), T, topk, experts.first, E, _ptr(counts), _ptr(offsets), _ptr(pos), _ptr(total), PAD, s), "fb_moe_plan")
    dt = dtype_code(x.dtype)
    fp8_native = st.kind == "fp8" and QG.FP8_NATIVE and H % 128 == 0 and st.inter % 128 == 0
    int_a8 = QG.INT_A8 and (st.kind == "int8" or (st.kind == "int4g" and st.group == 128)) and H % 128 == 0 and st.inter % 128 == 0
    if int_a8 and st.a8 is None:
        _prepare_a8(st, experts)
    act = torch.empty((rows_cap, st.inter), device=dev, dtype=x.dtype)
    ys = torch.empty((rows_cap, H), device=dev, dtype=x.dtype)
    if fp8_native:
        # gather fused with the e4m3 quantisation of the rows (the 16-bit sorted copy is never materialised)
        ld_a = (rows_cap + 128 + 3) // 4 * 4
        xq = torch.empty((rows_cap, H), device=dev, dtype=torch.uint8)
        sa = torch.empty((H // 128, ld_a), device=dev, dtype=torch.float32)
        _lib.check(lib.fb_moe_gather_quant_fp8(_ptr(x.contiguous()), _ptr(pos), _ptr(xq), _ptr(sa), ld_a, T, topk, H, dt, s),
                   "fb_moe_gather_quant_fp8")
    elif int_a8:
        # gather fused with the int8 quantisation of the rows
        xq, sa, sx, ld_a = QG.quant_act_i8(x.contiguous(), pos=pos, topk=topk, rows_cap=rows_cap)
    else:
        xs = torch.empty((rows_cap, H), device=dev, dtype=x.dtype)
        _lib.check(lib.fb_moe_gather(_ptr(x.contiguous()), _ptr(pos), _ptr(xs), T, topk, H, s), "fb_moe_gather")
    if st.kind == "dense":
        _lib.check(lib.fb_moe_grouped_gemm(_ptr(xs), _ptr(st.gate_up), _ptr(act), _ptr(None), _ptr(counts), _ptr(offsets), rows_cap, E,
                                           2 * st.inter, H, st.inter, max_rows, dt, GEMM_SWIGLU, T * topk, s), "fb_moe_grouped_gemm(gate_up)")
        _lib.check(lib.fb_moe_grouped_gemm(_ptr(act), _ptr(st.down), _ptr(ys), _ptr(None), _ptr(counts), _ptr(offsets), rows_cap, E,
                                           H, st.inter, H, max_rows, dt, 0, T * topk, s), "fb_moe_grouped_gemm(down)")
    elif fp8_native:
        # W8A8: e4m3 x e4m3 grouped GEMMs; the SwiGLU output is quantised again for the down projection
        _lib.check(lib.fb_moe_grouped_gemm_fp8(_ptr(xq), H, _ptr(sa), ld_a, _ptr(st.gate_up), _ptr(st.gu_scale), _ptr(act), _ptr(counts),
                                               _ptr(offsets), E, 2 * st.inter, H, rows_cap, st.inter, dt, GEMM_SWIGLU, max_rows, T * topk, s),
                   "fb_moe_grouped_gemm_fp8(gate_up)")
        aq, sb, ld_b = QG.quant_act_fp8(act, total)
        _lib.check(lib.fb_moe_grouped_gemm_fp8(_ptr(aq), st.inter, _ptr(sb), ld_b, _ptr(st.down), _ptr(st.dn_scale), _ptr(ys), _ptr(counts),
                                               _ptr(offsets), E, H, st.inter, rows_cap, H, dt, 0, max_rows, T * topk, s),
                   "fb_moe_grouped_gemm_fp8(down)")
    elif int_a8 and st.kind == "int4g" and QG.I4_GEMV and mean <= 2 and max(H, st.inter) <= 16384:
        # about one row per expert: CUDA-core dp4a kernel, one 128-row weight tile per CTA, rows of an expert in passes of four
        gs, _, ds, _ = st.a8
        _lib.check(lib.fb_gemv_i4(_ptr(xq), H, _ptr(sa), _ptr(sx), ld_a, _ptr(st.gate_up), _ptr(gs), _ptr(act), 0, 2 * st.inter, H, st.inter,
                                  dt, GEMM_SWIGLU, _ptr(counts), _ptr(offsets), E, s), "fb_gemv_i4(gate_up)")
        aq, sb, sbx, ld_b = QG.quant_act_i8(act, rows_used=total)
        _lib.check(lib.fb_gemv_i4(_ptr(aq), st.inter, _ptr(sb), _ptr(sbx), ld_b, _ptr(st.down), _ptr(ds), _ptr(ys), 0, H, st.inter, H,
                                  dt, 0, _ptr(counts), _ptr(offsets), E, s), "fb_gemv_i4(down)")
    elif int_a8:
        wk = 1 if st.kind == "int8" else 2
        gs, gz, ds, dz = st.a8
        _lib.check(lib.fb_gemm_i8(_ptr(xq), H, _ptr(sa), _ptr(sx), ld_a, _ptr(st.gate_up), _ptr(gs), _ptr(gz), _ptr(act), _ptr(None),
                                  _ptr(None), T * topk, 2 * st.inter, H, st.inter, 0, dt, GEMM_SWIGLU, wk, 1, _ptr(counts), _ptr(offsets), E,
                                  rows_cap, max_rows, s), "fb_gemm_i8(gate_up)")
        aq, sb, sbx, ld_b = QG.quant_act_i8(act, rows_used=total)
        _lib.check(lib.fb_gemm_i8(_ptr(aq), st.inter, _ptr(sb), _ptr(sbx), ld_b, _ptr(st.down), _ptr(ds), _ptr(dz), _ptr(ys), _ptr(None),
                                  _ptr(None), T * topk, H, st.inter, H, 0, dt, 0, wk, 1, _ptr(counts), _ptr(offsets), E, rows_cap, max_rows, s),
                   "fb_gemm_i8(down)")
    else:
        qm = {"int8": 1, "int4g": 2, "fp8": 3, "fp4": 4}[st.kind]
        grp = -1 if st.signed else (st.group or 0)           # -1: int8 bytes hold q - 128
        f16w = QG.GEMM_FP4_F16W if (st.kind == "fp4" and getattr(st, "fp4_f16w", False)) else 0
        _lib.check(lib.fb_moe_grouped_gemm_quant(_ptr(xs), _ptr(st.gate_up), _ptr(st.gu_scale), _ptr(st.gu_zero), _ptr(act), _ptr(counts),
                                                 _ptr(offsets), rows_cap, E, 2 * st.inter, H, st.inter, max_rows, dt, qm, grp,
                                                 GEMM_SWIGLU | f16w, T * topk, s), "fb_moe_grouped_gemm_quant(gate_up)")
        _lib.check(lib.fb_moe_grouped_gemm_quant(_ptr(act), _ptr(st.down), _ptr(st.dn_scale), _ptr(st.dn_zero), _ptr(ys), _ptr(counts),
                                                 _ptr(offsets), rows_cap, E, H, st.inter, H, max_rows, dt, qm, grp, f16w, T * topk, s),
                   "fb_moe_grouped_gemm_quant(down)")
    if not combine:
        return ys, pos, wts
    out = torch.empty((T, H), device=dev, dtype=x.dtype)
    _lib.check(lib.fb_moe_combine(_ptr(ys), _ptr(pos), _ptr(wts), _ptr(add), _ptr(out), T, topk, H, dt, s), "fb_moe_combine")
    return out
