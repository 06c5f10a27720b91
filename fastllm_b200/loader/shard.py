"""Turn canonical (Llama-style) named tensors into the per-rank weights of a ``DecoderModel``.

Covers what the reference does at load time: merging q/k/v into one QKV matrix and gate/up into one
matrix with their quantisation metadata (weightMergeRules, src/model.cpp:3943-4090), splitting for
tensor parallelism -- QKV by KV head, gate/up as paired halves, O/down along the input dim
(BuildMultiCudaRowSplitScheme, src/devices/multicuda/fastllm-multicuda.cu:882-980) -- expert placement
for expert parallelism (src/devices/multicuda/multicudadevice.cpp:6226-6236) and quantising to the
requested ``--dtype`` / ``--moe_dtype``.
"""
from __future__ import annotations

import torch

from ..ops import basic as B
from ..ops import moe as MOE
from ..ops.quant import LinearWeight, normalize_wdtype


def _shard_rows(w, rank, size):
    n = w.shape[0] // size
    return w[rank * n:(rank + 1) * n]


def _shard_cols(w, rank, size):
    n = w.shape[1] // size
    return w[:, rank * n:(rank + 1) * n]


def _heads_rows(w, head_dim, h0, h1):
    return w[h0 * head_dim:h1 * head_dim]


def _to(t, m):
    if t is None:
        return None
    if t.is_floating_point() and t.dtype not in (torch.float8_e4m3fn,):
        t = t.to(m.dtype)
    return t.to(m.device).contiguous()


def split_layers_by_map(num_layers: int, device_map: dict) -> list:
    """``{'cuda:0': 3, 'cuda:1': 2}`` -> one device per layer, contiguous blocks in proportion to the weights
    (reference: SelectDeviceFromMap / ApplyDeviceMap, src/fastllm.cpp:5178-5204)."""
    items = [(torch.device(k), float(v)) for k, v in device_map.items() if float(v) > 0]
    total = sum(v for _, v in items)
    out, acc = [], 0.0
    for dev, v in items:
        acc += v
        upto = num_layers if dev is items[-1][0] else round(num_layers * acc / total)
        out.extend([dev] * max(0, upto - len(out)))
    out.extend([items[-1][0]] * (num_layers - len(out)))
    return out[:num_layers]


class _HostPlacement:
    """Stand-in for the model when a weight is built for the CPU (expert offload): same dtype rules, CPU device."""

    def __init__(self, m):
        self.device = torch.device("cpu")
        self.dtype = m.dtype if m.dtype != torch.float32 else torch.float32
        self.on_cuda = False


def _q_src(w, m, wdtype):
    """Weight on the model's device; an fp32 source that is about to be quantised keeps its precision (4-bit checkpoints
    de-quantised in fp32 get their own grid back from the group-wise quantiser)."""
    if w is not None and w.dtype == torch.float32 and normalize_wdtype(wdtype)[0] == "int4g":
        return w.to(m.device).contiguous()
    return _to(w, m)


def _lin(m, w, wdtype, bias=None, interleaved=False):
    return LinearWeight.from_dense(_q_src(w, m, wdtype), wdtype, _to(bias, m), interleaved, act_dtype=m.dtype)


def _gate_up(m, gate, up, wdtype, bias_g=None, bias_u=None):
    """Merge gate and up into the tile-interleaved layout (CUDA) or plain stacking (CPU)."""
    if m.on_cuda and gate.shape[0] % 64 == 0:
        w = B.interleave_gate_up(_q_src(gate, m, wdtype), _q_src(up, m, wdtype))
        b = B.interleave_gate_up(_to(bias_g, m), _to(bias_u, m)) if bias_g is not None else None
        return LinearWeight.from_dense(w, wdtype, b, True, act_dtype=m.dtype)
    w = torch.cat([_q_src(gate, m, wdtype), _q_src(up, m, wdtype)], dim=0)
    b = torch.cat([_to(bias_g, m), _to(bias_u, m)]) if bias_g is not None else None
    return LinearWeight.from_dense(w, wdtype, b, False, act_dtype=m.dtype)


def build_layer(m, i: int, t: dict, wdtype="dense", moe_wdtype=None):
    """Fill ``m.layers[i]`` from the canonical tensors of layer ``i`` (dict is consumed)."""
    from ..models.decoder import LayerWeights

    cfg, tp = m.cfg, m.tp
    p = f"model.layers.{i}."
    lw = LayerWeights()
    a, f = lw.attn, lw.mlp
    g = lambda k: t.get(p + k)
    a.ln = _to(g("input_layernorm.weight"), m)
    if g("input_layernorm.bias") is not None:                   # LayerNorm families: the bias rides beside its weight
        m.ln_bias[id(a.ln)] = _to(g("input_layernorm.bias"), m)
    if g("pre_feedforward_layernorm.weight") is not None:       # Gemma-2/3: pre- and post-norm around both sub-layers
        a.post_ln = _to(g("post_attention_layernorm.weight"), m)
        f.ln = _to(g("pre_feedforward_layernorm.weight"), m)
        f.post_ln = _to(g("post_feedforward_layernorm.weight"), m)
    else:
        f.ln = _to(g("post_attention_layernorm.weight"), m)
        a.post_ln = _to(g("post_self_attn_layernorm.weight"), m)     # GLM-4
        f.post_ln = _to(g("post_mlp_layernorm.weight"), m)
    if cfg.layer_windows is not None and i < len(cfg.layer_windows):
        a.window = int(cfg.layer_windows[i])
    elif cfg.sliding_window and cfg.sliding_window < cfg.max_position:
        a.window = int(cfg.sliding_window)
    rs = float(cfg.residual_scale)

    def _rs(w):           # residual multiplier folded into the projections that feed the residual stream
        return w if (w is None or rs == 1.0) else (w.float() * rs).to(w.dtype)
    r, n = tp.rank, tp.size
    base_w, base_mw = wdtype, (moe_wdtype or wdtype)

    def W(name):          # per-tensor weight dtype (dtype_config rules may override the default)
        f_ = getattr(m, "wdtype_for", None)
        return f_(p + name) if f_ else base_w

    def MW(name):
        f_ = getattr(m, "moe_wdtype_for", None)
        return f_(p + name) if f_ else base_mw

    if cfg.layer_is_linear(i):
        lw.lin = build_linear_attn(m, g, a.ln, W, i)
    elif cfg.use_mla:
        nope, rope, vd, lora = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        Hl = cfg.num_heads // n
        qd = nope + rope
        if g("self_attn.q_a_proj.weight") is not None:
            a.q_a = _lin(m, g("self_attn.q_a_proj.weight"), wdtype)
            a.q_a_norm = _to(g("self_attn.q_a_layernorm.weight"), m)
            a.q_b = _lin(m, _heads_rows(g("self_attn.q_b_proj.weight"), qd, r * Hl, (r + 1) * Hl), wdtype)
        else:
            a.q_b = _lin(m, _heads_rows(g("self_attn.q_proj.weight"), qd, r * Hl, (r + 1) * Hl), wdtype)
        a.kv_a = _lin(m, g("self_attn.kv_a_proj_with_mqa.weight"), wdtype)
        a.kv_a_norm = _to(g("self_attn.kv_a_layernorm.weight"), m)
        kvb = g("self_attn.kv_b_proj.weight").to(torch.float32).view(cfg.num_heads, nope + vd, lora)[r * Hl:(r + 1) * Hl]
        a.w_uk = _to(kvb[:, :nope, :], m)
        a.w_uv = _to(kvb[:, nope:, :], m)
        a.o = _lin(m, _shard_cols(_rs(g("self_attn.o_proj.weight")), r, n), wdtype)
        if cfg.index_topk and g("self_attn.indexer.wq_b.weight") is not None:
            # sparse-attention indexer: small projections, the same on every rank
            a.idx_wq = _lin(m, g("self_attn.indexer.wq_b.weight"), "dense")
            a.idx_wk = _lin(m, g("self_attn.indexer.wk.weight"), "dense")
            a.idx_k_norm = (g("self_attn.indexer.k_norm.weight").to(m.device, torch.float32),
                            g("self_attn.indexer.k_norm.bias").to(m.device, torch.float32))
            a.idx_weights = g("self_attn.indexer.weights_proj.weight").to(m.device, torch.float32).contiguous()
            m.has_indexer = True
    else:
        D = cfg.head_dim
        heads_i = cfg.layer_heads[i] if cfg.layer_heads else cfg.num_heads
        Hq_l = heads_i // n
        if cfg.layer_heads:
            a.heads = Hq_l
        if cfg.layer_rope:
            a.rope = cfg.layer_rope[i]
        Hkv_l = m.num_kv_heads_local
        kv0 = (r * cfg.num_kv_heads) // n if cfg.num_kv_heads >= n else r // m.kv_replicas
        if g("self_attn.qkv_proj.weight") is not None:        # already merged (phi3-style): [q | k | v]
            w = g("self_attn.qkv_proj.weight")
            if cfg.model_type == "internlm2":
                # InternLM2 groups the rows per KV head: [G query heads, 1 key head, 1 value head] x num_kv_heads
                G = cfg.num_heads // cfg.num_kv_heads
                wg = w.reshape(cfg.num_kv_heads, G + 2, D, w.shape[-1])
                w = torch.cat([wg[:, :G].reshape(-1, w.shape[-1]), wg[:, G].reshape(-1, w.shape[-1]), wg[:, G + 1].reshape(-1, w.shape[-1])], dim=0)
            if cfg.model_type in ("moss", "codegen"):
                # CodeGen keeps four blocks of [query | value | key] rows, each covering a quarter of the heads
                w4 = w.reshape(4, 3, cfg.num_heads * D // 4, w.shape[-1])
                w = torch.cat([w4[:, 0].reshape(-1, w.shape[-1]), w4[:, 2].reshape(-1, w.shape[-1]), w4[:, 1].reshape(-1, w.shape[-1])], dim=0)
            qw, kw, vw = w.split([heads_i * D, cfg.num_kv_heads * D, cfg.num_kv_heads * D], dim=0)
            bq = bk = bv = None
            if g("self_attn.qkv_proj.bias") is not None:
                bq, bk, bv = g("self_attn.qkv_proj.bias").split([heads_i * D, cfg.num_kv_heads * D, cfg.num_kv_heads * D])
        else:
            qw, kw, vw = g("self_attn.q_proj.weight"), g("self_attn.k_proj.weight"), g("self_attn.v_proj.weight")
            bq, bk, bv = g("self_attn.q_proj.bias"), g("self_attn.k_proj.bias"), g("self_attn.v_proj.bias")
            if kw is None and g("self_attn.kv_proj.weight") is not None:
                # TeleChat: one projection with rows [head][key | value]
                kvw = g("self_attn.kv_proj.weight").reshape(cfg.num_kv_heads, 2, D, -1)
                kw, vw = kvw[:, 0].reshape(cfg.num_kv_heads * D, -1), kvw[:, 1].reshape(cfg.num_kv_heads * D, -1)
                kvb = g("self_attn.kv_proj.bias")
                if kvb is not None:
                    kvb = kvb.reshape(cfg.num_kv_heads, 2, D)
                    bk, bv = kvb[:, 0].reshape(-1), kvb[:, 1].reshape(-1)
                    if bq is None:
                        bq = torch.zeros(heads_i * D, dtype=kvb.dtype)
                elif bq is not None:
                    bk = bv = torch.zeros(cfg.num_kv_heads * D, dtype=bq.dtype)
            if cfg.attn_output_gate:
                # q_proj carries [query | gate] per head: the gate rows become their own projection
                qg = qw.reshape(cfg.num_heads, 2, D, qw.shape[-1])
                qw, gate_w = qg[:, 0].reshape(cfg.num_heads * D, -1), qg[:, 1].reshape(cfg.num_heads * D, -1)
                gate_b = None
                if bq is not None:
                    bg_ = bq.reshape(cfg.num_heads, 2, D)
                    bq, gate_b = bg_[:, 0].reshape(-1), bg_[:, 1].reshape(-1)
                a.out_gate = _lin(m, _heads_rows(gate_w, D, r * Hq_l, (r + 1) * Hq_l), W("self_attn.q_proj.weight"),
                                  _heads_rows(gate_b, D, r * Hq_l, (r + 1) * Hq_l) if gate_b is not None else None)
        w = torch.cat([_heads_rows(qw, D, r * Hq_l, (r + 1) * Hq_l), _heads_rows(kw, D, kv0, kv0 + Hkv_l),
                       _heads_rows(vw, D, kv0, kv0 + Hkv_l)], dim=0)
        b = None
        if bq is not None:
            b = torch.cat([_heads_rows(bq, D, r * Hq_l, (r + 1) * Hq_l), _heads_rows(bk, D, kv0, kv0 + Hkv_l),
                           _heads_rows(bv, D, kv0, kv0 + Hkv_l)])
        a.qkv = _lin(m, w, W("self_attn.qkv_proj.weight"), b)
        ob = _rs(g("self_attn.o_proj.bias"))
        a.o = _lin(m, _shard_cols(_rs(g("self_attn.o_proj.weight")), r, n), W("self_attn.o_proj.weight"), ob if (ob is not None and r == 0) else None)
        qn, kn = g("self_attn.q_norm.weight"), g("self_attn.k_norm.weight")
        if qn is None:
            qn, kn = g("self_attn.query_layernorm.weight"), g("self_attn.key_layernorm.weight")     # Hunyuan names
        if cfg.qk_norm_full and qn is not None and n > 1:
            # one norm over all heads: every rank keeps the weights of its own heads (the squares are summed across ranks)
            qn, kn = qn[r * Hq_l * D:(r + 1) * Hq_l * D], kn[kv0 * D:(kv0 + Hkv_l) * D]
        a.q_norm, a.k_norm = _to(qn, m), _to(kn, m)
        gp = g("self_attn.g_proj.weight")
        if gp is not None and cfg.head_gate:            # one gate per query head on the attention output
            a.head_gate = _lin(m, gp[r * Hq_l:(r + 1) * Hq_l], "dense")
        sk = g("self_attn.sinks")
        if sk is not None:
            a.sinks = sk[r * Hq_l:(r + 1) * Hq_l].to(m.device, torch.float32).contiguous()
    # ---- feed-forward ----
    if cfg.layer_is_moe(i) and g("mlp.experts.gate_up_proj") is not None and cfg.moe_act == "gptoss":
        # gpt-oss: stacked experts [E, H, 2I] with gate / up in alternating columns, biases on every projection
        f.router = g("mlp.router.weight").to(m.device, torch.float32).contiguous()
        f.router_logit_bias = g("mlp.router.bias").to(m.device, torch.float32).contiguous()
        gup, gub = g("mlp.experts.gate_up_proj"), g("mlp.experts.gate_up_proj_bias")
        dwn, dwb = g("mlp.experts.down_proj"), g("mlp.experts.down_proj_bias")
        lo, hi = MOE.local_expert_range(cfg.num_experts, m.ep)
        gu, dn = [], []
        for e in range(lo, hi):
            gw, uw = gup[e][:, 0::2].t().contiguous(), gup[e][:, 1::2].t().contiguous()
            gu.append(_gate_up(m, gw, uw, MW("mlp.experts.gate_up_proj"), gub[e][0::2].contiguous(), gub[e][1::2].contiguous()))
            dn.append(_lin(m, _rs(dwn[e].t().contiguous()), MW("mlp.experts.down_proj"), _rs(dwb[e])))
        f.experts = MOE.ExpertWeights(cfg.num_experts, lo, gu, dn)
        f.experts.act = "gptoss"
    elif cfg.layer_is_moe(i):
        f.router = g("mlp.gate.weight").to(m.device, torch.float32).contiguous()
        rb = g("mlp.gate.e_score_correction_bias")
        f.router_bias = rb.reshape(-1).to(m.device, torch.float32).contiguous() if rb is not None else None
        rsc = g("mlp.router_scale")                                  # Pangu Pro MoE: learned per-expert output scale
        f.router_scale = rsc.reshape(-1).to(m.device, torch.float32).contiguous() if rsc is not None else None
        lo, hi = MOE.local_expert_range(cfg.num_experts, m.ep)
        moe_tp = (m.ep is None or m.ep.size == 1) and n > 1      # no EP: shard every expert's intermediate dim
        gu, dn = [], []
        host = getattr(m, "moe_device", None) == "cpu" and m.on_cuda and (getattr(m, "moe_device_layers", -1) < 0 or i < m.moe_device_layers)
        em = _HostPlacement(m) if host else m
        stk = [g(f"mlp.experts.stacked_{nm}") for nm in ("gate", "up", "down")]      # Step-3.5: [E, rows, cols] per projection
        for e in range(lo, hi):
            gw, uw, dw = (g(f"mlp.experts.{e}.{nm}.weight") for nm in ("gate_proj", "up_proj", "down_proj"))
            if gw is None and stk[0] is not None:
                gw, uw, dw = stk[0][e], stk[1][e], stk[2][e]
            span = g(f"mlp.experts.{e}.gate_up_span") if getattr(m, "moe_disk", False) else None
            t.pop(p + f"mlp.experts.{e}.gate_up_span", None)
            if span is not None and not moe_tp and (host or not m.on_cuda) and span.dtype == em.dtype \
                    and normalize_wdtype(MW(f"mlp.experts.{e}.gate_proj.weight"))[0] == "dense":
                # disk placement: [gate; up] and down stay views of the checkpoint's file mapping
                gu.append(LinearWeight("dense", span, dtype=em.dtype, interleaved=False))
                dn.append(LinearWeight("dense", dw, dtype=em.dtype))
                for nm in ("gate_proj", "up_proj", "down_proj"):
                    t.pop(p + f"mlp.experts.{e}.{nm}.weight", None)
                continue
            if moe_tp:
                gw, uw, dw = _shard_rows(gw, r, n), _shard_rows(uw, r, n), _shard_cols(dw, r, n)
            gu.append(_gate_up(em, gw, uw, MW(f"mlp.experts.{e}.gate_proj.weight")))
            dn.append(_lin(em, dw, MW(f"mlp.experts.{e}.down_proj.weight")))
            for nm in ("gate_proj", "up_proj", "down_proj"):
                t.pop(p + f"mlp.experts.{e}.{nm}.weight", None)
        f.experts = MOE.ExpertWeights(cfg.num_experts, lo, gu, dn)
        if cfg.swiglu_limits and float(cfg.swiglu_limits[i]) != 0.0:
            f.experts.limit = float(cfg.swiglu_limits[i])
            f.experts.act = "swiglu_clamp"
        f.experts.host = host
        f.experts.numa = bool(host and getattr(m, "moe_numa", False))
        sp = "mlp.shared_expert." if g("mlp.shared_expert.gate_proj.weight") is not None else "mlp.shared_experts."
        if g(sp + "gate_proj.weight") is not None:
            f.shared_gate_up = _gate_up(m, _shard_rows(g(sp + "gate_proj.weight"), r, n), _shard_rows(g(sp + "up_proj.weight"), r, n), wdtype)
            f.shared_down = _lin(m, _shard_cols(g(sp + "down_proj.weight"), r, n), wdtype)
            sg = g("mlp.shared_expert_gate.weight")
            f.shared_gate = _to(sg, m) if sg is not None else None
    elif not cfg.mlp_gated:
        ub, db = g("mlp.up_proj.bias"), _rs(g("mlp.down_proj.bias"))
        f.up = _lin(m, _shard_rows(g("mlp.up_proj.weight"), r, n), W("mlp.up_proj.weight"), _shard_rows(ub, r, n) if ub is not None else None)
        f.down = _lin(m, _shard_cols(_rs(g("mlp.down_proj.weight")), r, n), W("mlp.down_proj.weight"), db if (db is not None and r == 0) else None)
    else:
        if g("mlp.gate_up_proj.weight") is not None:           # merged [gate | up]
            gw, uw = g("mlp.gate_up_proj.weight").chunk(2, dim=0)
        else:
            gw, uw = g("mlp.gate_proj.weight"), g("mlp.up_proj.weight")
        bg, bu, bd = g("mlp.gate_proj.bias"), g("mlp.up_proj.bias"), g("mlp.down_proj.bias")
        f.gate_up = _gate_up(m, _shard_rows(gw, r, n), _shard_rows(uw, r, n), W("mlp.gate_proj.weight"),
                             _shard_rows(bg, r, n) if bg is not None else None, _shard_rows(bu, r, n) if bu is not None else None)
        bd = _rs(bd)
        f.down = _lin(m, _shard_cols(_rs(g("mlp.down_proj.weight")), r, n), W("mlp.down_proj.weight"), bd if (bd is not None and r == 0) else None)
    if cfg.swiglu_limits_shared:
        f.act_limit = float(cfg.swiglu_limits_shared[i])
    while len(m.layers) <= i:
        m.layers.append(None)
    m.layers[i] = lw


def build_linear_attn(m, g, ln, W, layer_idx: int = 0):
    """Gated-DeltaNet weights of one layer for this rank.  Accepts the grouped layout of Qwen3-Next (``in_proj_qkvz`` /
    ``in_proj_ba``, rows grouped per key head) and the plain layout of Qwen3.5 (``in_proj_qkv``, ``in_proj_z``, ``in_proj_b``,
    ``in_proj_a``); heads are sharded over the tensor-parallel ranks by key head."""
    from ..models.decoder import LinearAttnWeights

    cfg, tp = m.cfg, m.tp
    r, n = tp.rank, tp.size
    Hk, Hv, Dk, Dv, K = cfg.lin_num_k_heads, cfg.lin_num_v_heads, cfg.lin_k_dim, cfg.lin_v_dim, cfg.lin_conv_kernel
    rep = Hv // Hk
    la = LinearAttnWeights()
    la.ln = ln
    if cfg.lin_kind == "lightning":
        # MiniMax-Text-01 / M1: fused projection with rows [head][q | k | v], output gate, norm over all heads; by head over ranks
        from ..ops.linear_attn import lightning_slopes

        Hl, D = Hv // n, Dv
        la.kind = "lightning"
        la.in_proj = _lin(m, g("self_attn.qkv_proj.weight")[r * Hl * 3 * D:(r + 1) * Hl * 3 * D], W("self_attn.qkv_proj.weight"))
        la.gate = _lin(m, g("self_attn.output_gate.weight")[r * Hl * D:(r + 1) * Hl * D], W("self_attn.output_gate.weight"))
        la.norm_w = _to(g("self_attn.norm.weight")[r * Hl * D:(r + 1) * Hl * D], m)
        la.out = _lin(m, g("self_attn.out_proj.weight")[:, r * Hl * D:(r + 1) * Hl * D], W("self_attn.out_proj.weight"))
        la.slope = lightning_slopes(Hv, layer_idx, cfg.num_layers)[r * Hl:(r + 1) * Hl].to(m.device).contiguous()
        la.Hk, la.Hv, la.Dk, la.Dv = Hl, Hl, D, D
        return la
    if g("linear_attn.in_proj_qkvz.weight") is not None:
        w = g("linear_attn.in_proj_qkvz.weight")
        Hd = w.shape[-1]
        wg = w.reshape(Hk, 2 * Dk + 2 * rep * Dv, Hd)
        qw, kw = wg[:, :Dk].reshape(Hk * Dk, Hd), wg[:, Dk:2 * Dk].reshape(Hk * Dk, Hd)
        vw = wg[:, 2 * Dk:2 * Dk + rep * Dv].reshape(Hv * Dv, Hd)
        zw = wg[:, 2 * Dk + rep * Dv:].reshape(Hv * Dv, Hd)
        ba = g("linear_attn.in_proj_ba.weight").reshape(Hk, 2 * rep, Hd)
        bw, aw = ba[:, :rep].reshape(Hv, Hd), ba[:, rep:].reshape(Hv, Hd)
    else:
        w = g("linear_attn.in_proj_qkv.weight")
        qw, kw, vw = w.split([Hk * Dk, Hk * Dk, Hv * Dv], dim=0)
        zw, bw, aw = g("linear_attn.in_proj_z.weight"), g("linear_attn.in_proj_b.weight"), g("linear_attn.in_proj_a.weight")
    cw = g("linear_attn.conv1d.weight").reshape(2 * Hk * Dk + Hv * Dv, K)
    cq, ck, cv = cw.split([Hk * Dk, Hk * Dk, Hv * Dv], dim=0)
    Hk_l, Hv_l = Hk // n, Hv // n
    hs = lambda t, d, H_l: t[r * H_l * d:(r + 1) * H_l * d]
    in_w = torch.cat([hs(qw, Dk, Hk_l), hs(kw, Dk, Hk_l), hs(vw, Dv, Hv_l), hs(zw, Dv, Hv_l), hs(bw, 1, Hv_l), hs(aw, 1, Hv_l)], dim=0)
    pad = (-in_w.shape[0]) % 8                      # the GEMM wants a multiple of 8 output rows
    if pad:
        in_w = torch.cat([in_w, torch.zeros(pad, in_w.shape[1], dtype=in_w.dtype, device=in_w.device)], dim=0)
    la.in_proj = _lin(m, in_w, W("linear_attn.in_proj_qkvz.weight"))
    la.conv_w = _to(torch.cat([hs(cq, Dk, Hk_l), hs(ck, Dk, Hk_l), hs(cv, Dv, Hv_l)], dim=0), m)
    la.A_log = g("linear_attn.A_log")[r * Hv_l:(r + 1) * Hv_l].to(m.device, torch.float32).contiguous()
    la.dt_bias = g("linear_attn.dt_bias")[r * Hv_l:(r + 1) * Hv_l].to(m.device, torch.float32).contiguous()
    la.norm_w = _to(g("linear_attn.norm.weight"), m)
    la.out = _lin(m, g("linear_attn.out_proj.weight")[:, r * Hv_l * Dv:(r + 1) * Hv_l * Dv], W("linear_attn.out_proj.weight"))
    la.Hk, la.Hv, la.Dk, la.Dv = Hk_l, Hv_l, Dk, Dv
    return la


def build_mtp(m, t: dict, wdtype="dense", moe_wdtype=None):
    """Multi-token-prediction module from the canonical tensors of layer ``num_layers`` (DeepSeek-V3 naming: ``enorm``,
    ``hnorm``, ``eh_proj``, ``shared_head.norm`` [, ``shared_head.head``] beside an ordinary decoder layer)."""
    from ..models.decoder import MTPModule

    L = m.cfg.num_layers
    p = f"model.layers.{L}."
    mt = MTPModule()
    mt.norm_e, mt.norm_h = _to(t.pop(p + "enorm.weight"), m), _to(t.pop(p + "hnorm.weight"), m)
    mt.fc = _lin(m, t.pop(p + "eh_proj.weight"), "dense")
    mt.final_norm = _to(t.pop(p + "shared_head.norm.weight"), m)
    hw = t.pop(p + "shared_head.head.weight", None)
    t.pop(p + "embed_tokens.weight", None)                       # a copy of the model's table
    if hw is not None and m.tp.size == 1 and m.lm_head is not None and tuple(hw.shape) == (m.lm_head.n, m.lm_head.k) and not m.cfg.tie_embeddings:
        same = m.lm_head.kind == "dense" and torch.equal(_to(hw, m), m.lm_head.w)
        mt.head = None if same else _lin(m, hw, "dense")
    build_layer(m, L, t, wdtype, moe_wdtype)
    mt.layer = m.layers.pop()                                     # not part of the decoder stack
    m.mtp = mt


def build_top(m, t: dict, wdtype="dense"):
    cfg, tp = m.cfg, m.tp
    m.embed = _to(t["model.embed_tokens.weight"], m)
    m.final_norm = _to(t["model.norm.weight"], m)
    if t.get("model.norm.bias") is not None:
        m.ln_bias[id(m.final_norm)] = _to(t["model.norm.bias"], m)
    head = t.get("lm_head.weight")
    hb = t.get("lm_head.bias")                 # CodeGen / MOSS, GPT-J
    if head is None or cfg.tie_embeddings:
        head = t["model.embed_tokens.weight"]
    if tp.size > 1:
        per = (cfg.vocab_size + tp.size - 1) // tp.size
        per = (per + 127) // 128 * 128
        lo = min(cfg.vocab_size, tp.rank * per)
        hi = min(cfg.vocab_size, lo + per)
        m.vocab_shard = (lo, hi)
        shard = head[lo:hi]
        if shard.shape[0] < per:   # keep every rank's shard the same shape (pad rows score -inf via zero weights + mask)
            pad = torch.zeros((per - shard.shape[0], shard.shape[1]), dtype=shard.dtype, device=shard.device)
            shard = torch.cat([shard, pad], dim=0)
        if hb is not None:
            hb = torch.cat([hb[lo:hi], torch.zeros(per - (hi - lo), dtype=hb.dtype, device=hb.device)])
        # lm_head stays 16-bit: its rounding decides the sampled token
        m.lm_head = _lin(m, shard, "dense", hb)
    else:
        if head is t["model.embed_tokens.weight"] and m.embed is not None and hb is None:
            m.lm_head = LinearWeight("dense", m.embed, dtype=m.dtype)
        else:
            m.lm_head = _lin(m, head, "dense", hb)


def finalize_model(m, top_fn, layer_fn, wdtype="dense", moe_wdtype=None):
    """``top_fn()`` / ``layer_fn(i)`` return dicts of canonical tensors; they are consumed one layer at a time."""
    from ..serving import progress

    home = m.device
    staged = getattr(m, "layer_devices", None)
    build_top(m, top_fn(), wdtype)
    for i in range(m.cfg.num_layers):
        if staged is not None:
            m.device = staged[i]           # the builders place tensors on m.device
        build_layer(m, i, layer_fn(i), wdtype, moe_wdtype)
        progress.emit("load_weights", i + 1, m.cfg.num_layers)
    m.device = home
    if staged is not None:                 # the head runs where the last layer left the activations
        last = staged[-1]
        m.final_norm = m.final_norm.to(last)
        hw = m.lm_head
        hw.w = hw.w.to(last)
        for name in ("scale", "zero", "bias"):
            t = getattr(hw, name)
            if t is not None:
                setattr(hw, name, t.to(last))
    if m.on_cuda:
        from ..ops import moe_grouped

        moe_grouped.prepare_model(m)
    return m
