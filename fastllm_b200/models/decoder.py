"""Generic paged-KV decoder used by every causal-LM family (dense GQA, MoE, MLA).

Model families differ only in configuration (``ModelConfig``) and weight naming (``loader/hf.py``); the
layer stack below covers what the reference implements per family in src/models/{llama,qwen2,qwen3,
qwen3_moe,deepseekv2,glm4_moe,...}.cpp.  The per-layer sequence on CUDA is

    RMSNorm -> QKV GEMM -> fused (QK-norm + RoPE + paged-KV append) -> paged attention ->
    O-proj GEMM (+residual in the epilogue) -> RMSNorm -> gate/up GEMM (+SwiGLU in the epilogue) ->
    down GEMM (+residual in the epilogue)

With tensor parallelism the two row-parallel GEMMs (O-proj, down) hand their partial sums to
``parallel.tp`` for the all-reduce (+residual).  All tensors are plain ``torch.Tensor`` attributes:
there is no autograd and no nn.Module overhead on the decode path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from ..ops import attention as A
from ..ops import basic as B
from ..ops import moe as MOE
from ..ops.quant import LinearWeight
from .config import ModelConfig


@dataclass
class ForwardBatch:
    """One scheduler step: packed new tokens of all scheduled requests (prefill chunks and/or decodes)."""
    ids: torch.Tensor            # int32 [T]
    positions: torch.Tensor      # int32 [T]
    slots: torch.Tensor          # int32 [T]   cache slot of each new token (-1 = do not store)
    page_table: torch.Tensor     # int32 [B, P]
    kv_lens: torch.Tensor        # int32 [B]   cached tokens per request after this step's append
    cu_q: torch.Tensor           # int32 [B+1]
    logit_rows: torch.Tensor | None = None   # int64 [R] rows of the packed batch that need logits
    is_decode: bool = False      # every request contributes exactly one token
    cu_q_host: list | None = None
    decode_ws: A.DecodeWorkspace | None = None
    decode_planned: bool = False
    state_slots: torch.Tensor | None = None      # int32 [B]: recurrent-state slot of each request (linear-attention layers)
    state_slots_host: list | None = None
    # prompts with images: rows whose embedding is given (image tokens) and (time, row, column) rotary positions [3, T]
    embed_rows: torch.Tensor | None = None
    embed_vals: torch.Tensor | None = None
    rope_pos3: torch.Tensor | None = None
    expert_rows: torch.Tensor | None = None      # rows evaluated with a model's visual-expert weights (models/cogvlm.py)
    keep_hidden: bool = False                    # leave the final-normed rows of the whole batch in ``model.last_hidden``
    kv_max_host: int = 0                         # longest context of the batch, known on the host (sparse-attention switch)


@dataclass
class TPInfo:
    rank: int = 0
    size: int = 1
    comm: object | None = None   # parallel.tp.TPComm

    def all_reduce(self, t, residual=None):
        if self.size == 1:
            return t if residual is None else t + residual
        return self.comm.all_reduce(t, residual)


class AttentionWeights:
    def __init__(self):
        self.ln = None
        self.qkv: LinearWeight | None = None
        self.o: LinearWeight | None = None
        self.q_norm = None
        self.k_norm = None
        self.post_ln = None      # sandwich norm on the attention output (Gemma-2 / GLM-4)
        self.sinks = None        # per-head sink logits (gpt-oss)
        self.out_gate: LinearWeight | None = None   # per-head output gate projection (Qwen3-Next: sigmoid(gate) * attention)
        self.window = 0          # sliding-window length of this layer (0: full causal attention)
        self.heads = None        # this rank's query heads in this layer when layers differ (Step-3.5 / Laguna)
        self.rope = None         # {"theta", "rot_dim", "scaling"} when the layer has its own rotary tables
        self.head_gate: LinearWeight | None = None  # [heads, H] projection: one gate per query head on the attention output
        # MLA
        self.q_a: LinearWeight | None = None
        self.q_a_norm = None
        self.q_b: LinearWeight | None = None
        self.kv_a: LinearWeight | None = None      # -> [kv_lora + rope]
        self.kv_a_norm = None
        self.w_uk = None       # [H, nope, kv_lora]   absorbed K up-projection
        self.w_uv = None       # [H, v_dim, kv_lora]  absorbed V up-projection
        self.w_uk_t = None     # [H, kv_lora, nope] in the activation dtype (operand layout of the batched absorb GEMM)
        self.w_uv_c = None
        # sparse-attention indexer (DeepSeek-V3.2 / GLM-MoE-DSA)
        self.idx_wq: LinearWeight | None = None    # [Hi * Di, q_lora]
        self.idx_wk: LinearWeight | None = None    # [Di, hidden]
        self.idx_k_norm = None                      # LayerNorm (weight, bias) of the index keys
        self.idx_weights = None                     # fp32 [Hi, hidden]: per-head weights of the index score


class LinearAttnWeights:
    """Gated-DeltaNet layer (this rank's heads): one merged input projection with output columns
    ``[q | k | v | z | b | a]``, the depth-wise convolution over ``[q | k | v]``, per-head decay parameters, the gated norm
    and the output projection."""

    def __init__(self):
        self.ln = None
        self.in_proj: LinearWeight | None = None
        self.conv_w = None        # [C, K]
        self.A_log = None         # fp32 [Hv]
        self.dt_bias = None       # fp32 [Hv]
        self.norm_w = None        # [Dv]
        self.out: LinearWeight | None = None
        self.Hk = self.Hv = self.Dk = self.Dv = 0
        # lightning attention (kind == "lightning"): in_proj is the fused q/k/v projection (per head q | k | v), gate the
        # output-gate projection, slope the per-head decay rates, norm_w spans all of this rank's heads
        self.kind = "gdn"
        self.gate: LinearWeight | None = None
        self.slope = None


class MLPWeights:
    def __init__(self):
        self.ln = None
        self.gate_up: LinearWeight | None = None
        self.up: LinearWeight | None = None      # two-matrix MLPs (no gate): up -> activation -> down
        self.down: LinearWeight | None = None
        self.post_ln = None      # sandwich norm on the MLP output
        self.act_limit = 0.0     # clamp inside the dense / shared-expert SwiGLU (Step-3.5); 0: none
        # MoE
        self.router = None          # fp32 [E, H]
        self.router_16 = None       # 16-bit copy for the tensor-core router GEMM
        self.router_bias = None     # fp32 [E]   selection-only correction bias (DeepSeek-V3)
        self.router_scale = None    # fp32 [E]   learned per-expert output scale (Pangu Pro MoE)
        self.router_logit_bias = None   # fp32 [E] bias of the router projection itself (gpt-oss)
        self.experts: MOE.ExpertWeights | None = None
        self.shared_gate_up: LinearWeight | None = None
        self.shared_down: LinearWeight | None = None
        self.shared_gate = None     # [1, H] sigmoid gate (qwen2_moe)


class LayerWeights:
    def __init__(self):
        self.attn = AttentionWeights()
        self.mlp = MLPWeights()
        self.lin: LinearAttnWeights | None = None      # set instead of ``attn`` projections on linear-attention layers


class MTPModule:
    """One multi-token-prediction module: the embedding of token i + 1 and the final-normed hidden row of position i are
    normalised, concatenated and projected back to the model width, pass one decoder layer with its own KV pages, a final
    norm and the model's output head -- the logits predict token i + 2.  (DeepSeek-V3 ``model.layers.<L>.{enorm, hnorm, eh_proj,
    shared_head.norm}``; Qwen3.5 ``mtp.{pre_fc_norm_embedding, pre_fc_norm_hidden, fc, layers.0, norm}``.)
    Reference: src/models/qwen3_5.cpp:20875-20884 (input fusion), :13868-13940 (draft chain)."""

    def __init__(self):
        self.norm_e = None
        self.norm_h = None
        self.fc: LinearWeight | None = None        # [H, 2H]: columns [embedding | hidden]
        self.layer: LayerWeights | None = None
        self.final_norm = None
        self.head: LinearWeight | None = None       # None: the model's own output head


class DecoderModel:
    """Weights + forward pass of one tensor-parallel rank."""

    def __init__(self, cfg: ModelConfig, device, dtype=torch.bfloat16, tp: TPInfo | None = None, ep=None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.tp = tp or TPInfo()
        self.ep = ep                       # parallel.ep.EPInfo or None
        self.embed = None                  # [vocab(/tp), H]
        self.layers: list[LayerWeights] = []
        self.final_norm = None
        self.lm_head: LinearWeight | None = None
        self.vocab_shard = (0, cfg.vocab_size)
        self.on_cuda = self.device.type == "cuda"
        self.num_heads_local = cfg.num_heads // self.tp.size
        self.num_kv_heads_local = max(1, cfg.num_kv_heads // self.tp.size)
        self.kv_replicas = max(1, self.tp.size // cfg.num_kv_heads)
        self._rope = None
        self._fused_active = False
        self._beta = 1.0                  # scale of the running sub-layer's contribution (DeepNorm-style residual models)
        self.layer_devices = None          # per-layer devices for the layer-split placement (None: everything on self.device)
        self.rope_mode = {"neox": A.ROPE_NEOX, "interleaved": A.ROPE_INTERLEAVED, "none": A.ROPE_NONE}[cfg.rope_mode]
        self.rot_dim = cfg.qk_rope_head_dim if cfg.use_mla else (cfg.rotary_dim or cfg.head_dim)
        self.attn_scale = cfg.attn_scale_override if cfg.attn_scale_override else 1.0 / math.sqrt(cfg.q_head_dim)
        # families whose attention needs options outside the tensor-core kernels run the PyTorch evaluation (not graph-safe)
        self.general_attn = bool(cfg.qk_norm_after_rope or cfg.qk_norm_full)
        self.kv8_decode_ok = False
        self.ln_bias = {}                  # LayerNorm families: id(norm weight) -> its bias
        self.mtp: MTPModule | None = None  # draft head for speculative decoding
        self.last_hidden = None
        if cfg.use_mla and cfg.rope_scaling and cfg.rope_scaling.get("mscale_all_dim"):
            ms = 0.1 * float(cfg.rope_scaling["mscale_all_dim"]) * math.log(float(cfg.rope_scaling.get("factor", 1.0))) + 1.0
            self.attn_scale *= ms * ms

    # -----------------------------------------------------------------------------------------------
    def rope_tables(self, max_pos: int | None = None, device=None, local: bool = False):
        if local and self.cfg.rope_local_theta:
            # sliding-window layers of Gemma-3: their own base, no scaling
            t = self.__dict__.get("_rope_local")
            if t is None:
                mp = max_pos or min(self.cfg.max_position, 1 << 17)
                t = self._rope_local = A.build_rope_tables(self.rot_dim, mp, self.cfg.rope_local_theta, None, self.device)
            return t if device is None or torch.device(device) == self.device else (t[0].to(device), t[1].to(device))
        if device is not None and torch.device(device) != self.device:
            key = str(torch.device(device))
            cache = self.__dict__.setdefault("_rope_by_device", {})
            if key not in cache:
                cos, sin = self.rope_tables(max_pos)
                cache[key] = (cos.to(device), sin.to(device))
            return cache[key]
        if self._rope is None:
            mp = max_pos or min(self.cfg.max_position, 1 << 17)
            scaling = self.cfg.rope_scaling
            if self.cfg.use_mla and scaling:
                # DeepSeek applies the yarn magnitude to the softmax scale (above), not to cos/sin
                scaling = dict(scaling)
                scaling["attention_factor"] = 1.0
            self._rope = A.build_rope_tables(self.rot_dim, mp, self.cfg.rope_theta, scaling, self.device)
        return self._rope

    def _layer_geom(self, lw, device, local: bool = False):
        """(query heads, cos, sin, rotary width) of one attention layer: its own where the layers differ."""
        Hq = lw.heads or self.num_heads_local
        if lw.rope is None:
            ov = self.__dict__.get("_rope_override")
            if ov is not None:                   # per-token rows of this forward pass (3-D rotary positions), indexed by row
                return Hq, ov[0], ov[1], self.rot_dim
            cos, sin = self.rope_tables(device=device, local=local)
            return Hq, cos, sin, self.rot_dim
        spec = lw.rope
        key = (float(spec["theta"]), int(spec["rot_dim"]), id(spec.get("scaling")), str(torch.device(device)))
        cache = self.__dict__.setdefault("_rope_layers", {})
        if key not in cache:
            mp = min(self.cfg.max_position, 1 << 17)
            cache[key] = A.build_rope_tables(int(spec["rot_dim"]), mp, float(spec["theta"]), spec.get("scaling"), device)
        cos, sin = cache[key]
        return Hq, cos, sin, int(spec["rot_dim"])

    def _head_gate(self, lw, x, a, Hq, D):
        """Multiply every head of the attention output by its learned gate: sigmoid (Step-3.5) or softplus (Laguna)."""
        gt = lw.head_gate(x).float()
        gt = torch.sigmoid(gt) if self.cfg.head_gate == "sigmoid" else F.softplus(gt)
        return (a.reshape(-1, Hq, D).float() * gt[:, :, None]).reshape(a.shape).to(a.dtype)

    def kv_cache_shape(self, num_pages: int):
        """Per-layer page-pool shapes of this rank: (K shape, V shape or None for MLA)."""
        c = self.cfg
        if c.use_mla:
            # one spare page at the end: rows that must not be cached (padded decode rows) are written there
            idx = (num_pages + 1, A.PAGE_LEN, 1, c.index_head_dim) if (c.index_topk and getattr(self, "has_indexer", False)) else None
            return (num_pages + 1, A.PAGE_LEN, 1, c.kv_lora_rank + c.qk_rope_head_dim), idx
        s = (num_pages, A.PAGE_LEN, self.num_kv_heads_local, c.head_dim)
        return s, s

    def kv_bytes_per_page(self) -> int:
        ks, vs = self.kv_cache_shape(1)
        n = math.prod(ks) + (math.prod(vs) if vs else 0)
        paged_layers = sum(1 for i in range(self.cfg.num_layers) if not self.cfg.layer_is_linear(i)) + (1 if self.mtp is not None else 0)
        return n * max(1, paged_layers) * torch.finfo(getattr(self, "kv_dtype", None) or self.dtype).bits // 8

    def linear_state_shapes(self, n_slots: int):
        """Per linear-attention layer: (convolution window pool, delta-rule state pool) shapes for ``n_slots`` requests."""
        c = self.cfg
        Hk, Hv = c.lin_num_k_heads // self.tp.size, c.lin_num_v_heads // self.tp.size
        if c.lin_kind == "lightning":          # no convolution window; one [D, D] state per head
            return (n_slots, 0, 0), (n_slots, Hv, c.lin_k_dim, c.lin_v_dim)
        C = 2 * Hk * c.lin_k_dim + Hv * c.lin_v_dim
        return (n_slots, C, c.lin_conv_kernel - 1), (n_slots, Hv, c.lin_k_dim, c.lin_v_dim)

    def linear_state_bytes_per_slot(self) -> int:
        if not self.cfg.has_linear_attn:
            return 0
        cs, rs = self.linear_state_shapes(1)
        n_lin = sum(1 for i in range(self.cfg.num_layers) if self.cfg.layer_is_linear(i))
        return n_lin * (math.prod(cs) * torch.finfo(self.dtype).bits // 8 + math.prod(rs) * 4)

    def set_kv_cache_dtype(self, name: str | None) -> None:
        """``fp8_e4m3``: keys and values are stored as unscaled e4m3 (half the cache bytes); attention then runs on the
        general (gather + PyTorch) path, the tcgen05 attention kernels read 16-bit pages only.
        Reference: basellm::SetKVCacheDataType (src/models/basellm.cpp:3567-3580), ``--kv_cache_dtype``."""
        name = (name or "auto").lower()
        if name in ("auto", ""):
            return
        table = {"fp8": torch.float8_e4m3fn, "fp8_e4m3": torch.float8_e4m3fn, "float8": torch.float8_e4m3fn,
                 "float16": torch.float16, "half": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
                 "float32": torch.float32, "fp32": torch.float32}
        if name not in table:
            raise ValueError("kv_cache_dtype should be float32, float16, bfloat16 or fp8_e4m3")
        dt = table[name]
        if dt == self.dtype:
            return
        if self.cfg.use_mla:
            raise NotImplementedError("the MLA latent cache is kept in the activation dtype")
        self.kv_dtype = dt
        self.general_attn = True              # prefill (and everything the decode kernel does not cover) evaluates attention in PyTorch
        c = self.cfg
        # e4m3 pages: decode runs the tensor-core kernel's KV8 mode when the fused post-processing can express the layer
        self.kv8_decode_ok = bool(dt == torch.float8_e4m3fn and self.on_cuda and c.head_dim == 128 and not c.use_mla
                                  and not (c.qk_norm_after_rope or c.qk_norm_full) and not c.rope_local_theta
                                  and self.dtype in (torch.float16, torch.bfloat16))
        self._cpu_runner = False              # the whole-model CPU runner owns fp32 pages

    # -----------------------------------------------------------------------------------------------
    def _attention(self, lw: AttentionWeights, x, fb: ForwardBatch, kv, residual, next_ln, consumer=None):
        c = self.cfg
        if c.use_mla:
            return self._mla_attention(lw, x, fb, kv, residual, next_ln, consumer)
        Hkv, D = self.num_kv_heads_local, c.head_dim
        Hq, cos, sin, rot = self._layer_geom(lw, x.device)
        k_pool, v_pool = kv
        variant = bool(c.attn_softcap or lw.window or lw.sinks is not None)
        # sliding window, sink logits and soft-capping run inside the decode kernels; what the fused post-processing cannot
        # express (norm after RoPE, one norm over all heads, e4m3 pages) and every prefill of a variant layer take the
        # PyTorch evaluation
        kernel_variant = (variant and fb.is_decode and x.is_cuda and D == 128 and not (c.qk_norm_after_rope or c.qk_norm_full)
                          and k_pool.dtype == x.dtype and not c.rope_local_theta)
        if (self.kv8_decode_ok and (fb.is_decode or not variant) and x.is_cuda and x.dim() == 2
                and k_pool.dtype == torch.float8_e4m3fn):
            # e4m3 pages: the post-processing launch (norm + RoPE) appends K / V as e4m3 bytes; decode reads the raw pages on the
            # fp8 tensor core (all launches CUDA-graph safe), prefill de-quantises the pages it reads
            T = x.shape[0]
            q8 = None
            if fb.is_decode and A.KV8_MMA and fb.decode_ws is not None and T <= fb.decode_ws.max_batch:
                q8 = fb.decode_ws.q8_terms(Hq * D)             # the post-processing launch also writes the queries' two e4m3 terms
            q = A.qkv_post(lw.qkv(x), fb.positions, fb.slots, k_pool, v_pool, Hq, Hkv, D, cos, sin, self.rope_mode, rot,
                           lw.q_norm, lw.k_norm, c.rms_eps, c.norm_unit_offset, q8=q8)
            if fb.is_decode:
                a = A.attn_decode(q, k_pool, v_pool, fb.page_table, fb.kv_lens, self.attn_scale, Hq, Hkv, D, ws=fb.decode_ws,
                                  planned=fb.decode_planned, window=int(lw.window or 0), softcap=float(c.attn_softcap or 0.0),
                                  sinks=lw.sinks, q8_ready=q8 is not None)
            else:                # prefill: the tensor-core prefill kernel over a 16-bit scratch copy of the pages it reads
                a = A.attn_prefill(q, k_pool, v_pool, fb.page_table, fb.kv_lens, fb.cu_q, self.attn_scale, Hq, Hkv, D,
                                   cu_q_host=fb.cu_q_host)
            if lw.out_gate is not None:
                a = (a.float() * torch.sigmoid(lw.out_gate(x).float())).to(a.dtype)
            if lw.head_gate is not None:
                a = self._head_gate(lw, x, a, Hq, D)
            return self._row_parallel_norm(lw.o, a, residual, next_ln, lw.post_ln, consumer)
        if (self.general_attn or variant) and not kernel_variant:
            a = self._attention_general(lw, lw.qkv(x), fb, kv)
            if lw.head_gate is not None:
                a = self._head_gate(lw, x, a, Hq, D)
            return self._row_parallel_norm(lw.o, a, residual, next_ln, lw.post_ln, consumer)
        # decode-sized batches with head_dim 128: projection, per-head norm, RoPE and cache append are one launch
        q = A.qkv_proj_post(x, lw.qkv, fb.positions, fb.slots, k_pool, v_pool, Hq, Hkv, D, cos, sin, self.rope_mode, rot,
                            lw.q_norm, lw.k_norm, c.rms_eps, c.norm_unit_offset) if x.dim() == 2 else None
        if q is None:
            q = A.qkv_post(lw.qkv(x), fb.positions, fb.slots, k_pool, v_pool, Hq, Hkv, D, cos, sin, self.rope_mode, rot,
                           lw.q_norm, lw.k_norm, c.rms_eps, c.norm_unit_offset)
        if fb.is_decode:
            qm = 0
            if lw.o.kind != "dense" and lw.post_ln is None:
                from ..ops import quant_gemm

                qm = quant_gemm.act_quant_mode(lw.o, q.shape[0])
                qm = qm if qm in (1, 2) else 0
            a = A.attn_decode(q, k_pool, v_pool, fb.page_table, fb.kv_lens, self.attn_scale, Hq, Hkv, D, ws=fb.decode_ws,
                              planned=fb.decode_planned, quant_mode=qm, window=int(lw.window or 0), softcap=float(c.attn_softcap or 0.0),
                              sinks=lw.sinks)
        else:
            a = A.attn_prefill(q, k_pool, v_pool, fb.page_table, fb.kv_lens, fb.cu_q, self.attn_scale, Hq, Hkv, D,
                               cu_q_host=fb.cu_q_host)
        if lw.out_gate is not None:
            a = (a.float() * torch.sigmoid(lw.out_gate(x).float())).to(a.dtype)
        if lw.head_gate is not None:
            a = self._head_gate(lw, x, a, Hq, D)
        return self._row_parallel_norm(lw.o, a, residual, next_ln, lw.post_ln, consumer)

    def _linear_attention(self, lw: LinearAttnWeights, x, fb: ForwardBatch, state, residual, next_ln, consumer=None):
        """Gated-DeltaNet token mixer over the request's convolution window and delta-rule state
        (reference: src/models/qwen3_next.cpp; operators RecurrentGatedDeltaRule / ChunkGatedDeltaRulePrefill)."""
        from ..ops import linear_attn as L

        c = self.cfg
        conv_state, rec_state = state
        if lw.kind == "lightning":
            return self._lightning_attention(lw, x, fb, rec_state, residual, next_ln, consumer)
        kd, vd = lw.Hk * lw.Dk, lw.Hv * lw.Dv
        C = 2 * kd + vd
        proj = lw.in_proj(x)                                   # [T, C + vd + 2 Hv]
        mixed, z = proj[:, :C], proj[:, C:C + vd]
        b, a = proj[:, C + vd:C + vd + lw.Hv], proj[:, C + vd + lw.Hv:C + vd + 2 * lw.Hv]
        T = x.shape[0]
        if fb.is_decode:
            y = L.causal_conv1d_decode(mixed, lw.conv_w, conv_state, fb.state_slots)
            core = L.gated_delta_decode(y, a, b, z, lw.A_log, lw.dt_bias, lw.norm_w, c.rms_eps, rec_state, fb.state_slots,
                                        lw.Hk, lw.Hv, lw.Dk, lw.Dv)
        else:
            y = L.causal_conv1d(mixed, lw.conv_w, conv_state, fb.cu_q_host, fb.state_slots_host)
            q, k, v = y[:, :kd].reshape(T, lw.Hk, lw.Dk), y[:, kd:2 * kd].reshape(T, lw.Hk, lw.Dk), y[:, 2 * kd:].reshape(T, lw.Hv, lw.Dv)
            o = L.gated_delta_rule(q, k, v, a, b, lw.A_log, lw.dt_bias, rec_state, fb.cu_q_host, fb.state_slots_host, lw.Hv // lw.Hk)
            core = L.rmsnorm_gated(o, z.reshape(T, lw.Hv, lw.Dv), lw.norm_w, c.rms_eps).reshape(T, vd)
        return self._row_parallel_norm(lw.out, core, residual, next_ln, consumer=consumer)

    def _lightning_attention(self, lw: LinearAttnWeights, x, fb: ForwardBatch, rec_state, residual, next_ln, consumer=None):
        """Lightning attention layer of MiniMax-Text-01 / M1: SiLU on the fused q/k/v projection, decayed linear attention
        over the request's ``[H, D, D]`` state, RMSNorm over all heads, sigmoid output gate, output projection
        (reference: src/models/minimax.cpp)."""
        from ..ops import linear_attn as L

        c = self.cfg
        T = x.shape[0]
        H, D = lw.Hv, lw.Dv
        qkv = torch.nn.functional.silu(lw.in_proj(x).float()).reshape(T, H, 3 * D)
        q, k, v = qkv[..., :D], qkv[..., D:2 * D], qkv[..., 2 * D:]
        if fb.is_decode:
            o = L.lightning_decode(q, k, v, lw.slope, rec_state, fb.state_slots)
        else:
            o = L.lightning_attention(q, k, v, lw.slope, rec_state, fb.cu_q_host, fb.state_slots_host, c.lin_block)
        o = o.reshape(T, H * D)
        ss = o.pow(2).sum(-1, keepdim=True)
        if self.tp.size > 1:                  # the norm spans all heads: the ranks add up their heads' squares
            ss = self.tp.all_reduce(ss.contiguous(), None)
        o = o * torch.rsqrt(ss / (c.num_heads * D) + c.rms_eps) * lw.norm_w.float()
        core = (torch.sigmoid(lw.gate(x).float()) * o).to(x.dtype)
        return self._row_parallel_norm(lw.out, core, residual, next_ln, consumer=consumer)

    def _row_ids(self, T: int, device):
        """``arange(T)`` int32 on ``device`` (cached: CUDA graphs need stable addresses)."""
        cache = self.__dict__.setdefault("_row_id_cache", {})
        key = (str(device), T)
        if key not in cache:
            cache[key] = torch.arange(T, device=device, dtype=torch.int32)
        return cache[key]

    def _attention_general(self, lw: AttentionWeights, qkv, fb: ForwardBatch, kv):
        """Attention for the less common variants (sliding window, sinks, logit soft-capping, norm after RoPE)."""
        c = self.cfg
        Hkv, D = self.num_kv_heads_local, c.head_dim
        T = qkv.shape[0]
        Hq, cos, sin, rot = self._layer_geom(lw, qkv.device, local=bool(lw.window))
        q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
        q, k, v = q.reshape(T, Hq, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D)
        norm = lambda t, w: A._head_norm_ref(t, w, c.rms_eps, c.norm_unit_offset) if w is not None else t
        if c.qk_norm_full:           # one norm over the whole projection (all heads of all ranks)
            def norm(t, w, total_heads=None):
                if w is None:
                    return t
                tf = t.reshape(T, -1).float()
                ss = tf.pow(2).sum(-1, keepdim=True)
                heads = t.shape[1]
                if self.tp.size > 1:     # this rank holds some of the heads: the ranks add up their squares
                    ss = self.tp.all_reduce(ss.contiguous(), None)
                    heads = heads * self.tp.size
                return (tf * torch.rsqrt(ss / (heads * D) + c.rms_eps) * (w.float() + c.norm_unit_offset)).reshape(t.shape).to(t.dtype)
        if not c.qk_norm_after_rope:
            q, k = norm(q, lw.q_norm), norm(k, lw.k_norm)
        q = A.apply_rope_ref(q, fb.positions, cos, sin, self.rope_mode, rot)
        k = A.apply_rope_ref(k, fb.positions, cos, sin, self.rope_mode, rot)
        if c.qk_norm_after_rope:
            q, k = norm(q, lw.q_norm), norm(k, lw.k_norm)
        k_pool, v_pool = kv
        valid = fb.slots >= 0
        sl = fb.slots[valid].long()
        k_pool.view(-1, Hkv, D)[sl] = k[valid].to(k_pool.dtype)
        v_pool.view(-1, Hkv, D)[sl] = v[valid].to(v_pool.dtype)
        return A.paged_attention_general(q.reshape(T, Hq * D).to(qkv.dtype), k_pool, v_pool, fb.page_table, fb.kv_lens, fb.cu_q,
                                         self.attn_scale, Hq, Hkv, D, window=lw.window, sinks=lw.sinks, softcap=c.attn_softcap)

    def _row_parallel(self, w: LinearWeight, x, residual):
        """Row-parallel linear (input dim sharded): partial GEMM, then sum over ranks, plus the residual."""
        if self.tp.size == 1:
            return w(x, residual=residual)
        return self.tp.comm.row_linear(w, x, residual)

    def _norm(self, h, ln_w):
        if self.cfg.norm_kind == "layernorm":
            return F.layer_norm(h.float(), (h.shape[-1],), ln_w.float(), self.ln_bias[id(ln_w)].float() if id(ln_w) in self.ln_bias else None,
                                self.cfg.rms_eps).to(h.dtype)
        qm = 0
        if h.is_cuda and h.dim() == 2:
            cons = self._norm_consumers().get(id(ln_w))
            if cons is not None:
                from ..ops import quant_gemm

                qm = quant_gemm.act_quant_mode(cons, h.shape[0])
        return B.rmsnorm(h, ln_w, self.cfg.rms_eps, unit_offset=self.cfg.norm_unit_offset, quant_mode=qm)

    def _norm_consumers(self) -> dict:
        """Norm weight -> the single quantised projection that reads that norm's output (its quantiser is fused into the norm)."""
        m = getattr(self, "_norm_cons", None)
        if m is None:
            m = {}
            for lw in self.layers:
                if lw.attn.ln is not None and lw.attn.qkv is not None and lw.attn.qkv.kind != "dense":
                    m[id(lw.attn.ln)] = lw.attn.qkv
                if lw.mlp.ln is not None and lw.mlp.gate_up is not None and lw.mlp.experts is None and lw.mlp.gate_up.kind != "dense":
                    m[id(lw.mlp.ln)] = lw.mlp.gate_up
            self._norm_cons = m
        return m

    @staticmethod
    def _waits_itself(consumer) -> bool:
        """True when ``consumer`` (the projection that reads the normalised rows next) runs the dense tensor-core GEMM,
        whose producer thread can wait for a deferred all-gather after it has requested its first weight tiles."""
        return (consumer is not None and consumer.kind == "dense" and LinearWeight.active_adapter is None
                and consumer.k % 64 == 0 and consumer.n % 8 == 0)

    def _row_parallel_norm(self, w: LinearWeight, x, h, next_ln, post_ln=None, consumer=None):
        """``h += row_parallel_linear(x)`` then ``RMSNorm(h)`` for the next block.  Returns (h, x_norm).

        With the fused NVLink path this is ONE kernel (GEMM + reduce-scatter + residual + norm + all-gather); when the
        next reader of the normalised rows is ``consumer`` (a dense projection), the kernel does not wait for the
        all-gather to land: that wait moves into the consumer's GEMM, behind its weight prefetch.
        """
        c = self.cfg
        if next_ln is None:              # parallel block: the attention output joins the residual, the MLP's call normalises
            return self._row_parallel(w, x, h), None
        if self._beta != 1.0:            # DeepNorm-style residual: the sub-layer's contribution is scaled (linear in x)
            x = x * self._beta
        if post_ln is not None:          # sandwich norm: normalise the sub-layer output, then add it to the residual stream
            y = self._norm(self._row_parallel(w, x, None), post_ln)
            h = h + y
            return h, self._norm(h, next_ln)
        if self._fused_active:
            defer = self._waits_itself(consumer)
            r = self.tp.comm.fused.gemm_ar_norm(w, x, next_ln, c.rms_eps, c.norm_unit_offset, True, defer=defer)
            if r is None:
                part = w(x)
                r = self.tp.comm.fused.ar_norm(part, next_ln, c.rms_eps, c.norm_unit_offset, True, defer=defer)
            return r
        h = self._row_parallel(w, x, h)
        return h, self._norm(h, next_ln)

    def _reduce_norm(self, partial, h, next_ln, needs_reduce: bool):
        """Same for a partial sum that did not come from a single GEMM (mixture-of-experts output)."""
        c = self.cfg
        if needs_reduce and self._fused_active:
            return self.tp.comm.fused.ar_norm(partial, next_ln, c.rms_eps, c.norm_unit_offset, True)
        if needs_reduce:
            h = self.tp.all_reduce(partial, h)
        elif self._fused_active:
            h = self.tp.comm.fused.load_h(partial + h)
        else:
            h = partial + h
        return h, self._norm(h, next_ln)

    def _mla_attention(self, lw: AttentionWeights, x, fb: ForwardBatch, kv, residual, next_ln, consumer=None):
        """Absorbed multi-head latent attention over a paged latent cache (kv_lora + rope dims per token).

        Reference: src/models/deepseekv2.cpp:283-697 (q_nope x W_UK -> MergeMLAPaged -> x W_UV -> o_proj).
        """
        c = self.cfg
        H = self.num_heads_local
        nope, rope, lora, vd = c.qk_nope_head_dim, c.qk_rope_head_dim, c.kv_lora_rank, c.v_head_dim
        T = x.shape[0]
        qr = None
        if lw.q_a is not None:
            qr = B.rmsnorm(lw.q_a(x), lw.q_a_norm, c.latent_norm_eps or c.rms_eps)
            q = lw.q_b(qr)
        else:
            q = lw.q_b(x)
        ckv = lw.kv_a(x)                                   # [T, lora + rope]
        cos, sin = self.rope_tables()
        lat_pool = kv[0]
        # latent norm + rope of the shared key into the cache entry, rope of the heads' rotary query parts: one launch
        q_full = torch.empty((T, H, lora + rope), device=x.device, dtype=x.dtype)
        A.mla_post(ckv, q, q_full, lat_pool, fb.positions, fb.slots, lw.kv_a_norm, cos, sin, H, nope, rope, lora, self.rope_mode,
                   c.latent_norm_eps or c.rms_eps)
        # absorb: q_lat[h] = q_nope[h] @ W_UK[h] -> attention in latent space with a single shared "KV head"; one batched
        # tensor-core launch over the heads, written straight into q_full[..., :lora]
        if lw.w_uk_t is None:
            lw.w_uk_t = lw.w_uk.transpose(1, 2).to(x.dtype).contiguous()      # [H, lora, nope]
            lw.w_uv_c = lw.w_uv.to(x.dtype).contiguous()                      # [H, vd, lora]
        B.linear_batched(q, lw.w_uk_t, H, nope + rope, q_full.view(T, H * (lora + rope)), lora + rope)
        sel = None
        if lw.idx_wq is not None and kv[1] is not None and qr is not None:
            # index keys of the new tokens: projection, LayerNorm, rotate-half rotary on the leading rope dims, into their own
            # paged pool (rows that must not be cached go to the spare last slot) -- tensor ops only, CUDA-graph safe
            Di, Hi = c.index_head_dim, c.index_n_heads
            idx_pool = kv[1]
            ki = F.layer_norm(lw.idx_wk(x).float(), (Di,), lw.idx_k_norm[0], lw.idx_k_norm[1], 1e-6)
            ki = A.apply_rope_ref(ki[:, None, :], fb.positions, cos, sin, A.ROPE_NEOX, rope)[:, 0]
            flat = idx_pool.view(-1, Di)
            sl = torch.where(fb.slots >= 0, fb.slots, torch.full_like(fb.slots, flat.shape[0] - 1)).long()
            flat.index_copy_(0, sl, ki.to(flat.dtype))
            if fb.kv_max_host > c.index_topk:
                # some context is longer than the selection size: every query keeps its index_topk best-scoring keys
                qi = A.apply_rope_ref(lw.idx_wq(qr).view(T, Hi, Di), fb.positions, cos, sin, A.ROPE_NEOX, rope)
                wi = torch.matmul(x.float(), lw.idx_weights.t()) * (Hi ** -0.5)
                sel = MOE.dsa_select(qi, wi, idx_pool, fb, c.index_topk)
        o_lat = MOE.mla_paged_attention(q_full, lat_pool, fb, self.attn_scale, lora, sel)   # [T, H, lora]
        o = torch.empty((T, H * vd), device=x.device, dtype=x.dtype)
        B.linear_batched(o_lat.reshape(T, H * lora), lw.w_uv_c, H, lora, o, vd)
        return self._row_parallel_norm(lw.o, o, residual, next_ln, consumer=consumer)

    @staticmethod
    def _glu(gu, act: str, interleaved: bool):
        """``act(gate) * up`` for gated MLPs whose activation is not SiLU (GeGLU of the Gemma family, ...): one kernel."""
        return B.glu_act(gu, act, interleaved)

    # -----------------------------------------------------------------------------------------------
    def _router_logits(self, lw: MLPWeights, x):
        """fp32 router logits.  On CUDA the router runs through the tensor-core GEMM with 16-bit operands and fp32
        accumulation / output; on CPU in fp32."""
        if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and lw.router.shape[0] % 8 == 0:
            if lw.router_16 is None:
                lw.router_16 = lw.router.to(x.dtype).contiguous()
            return B.linear(x, lw.router_16, out_f32=True)
        return torch.matmul(x.float(), lw.router.t())

    def _mlp(self, lw: MLPWeights, x, residual, layer_idx, next_ln, consumer=None):
        c = self.cfg
        if lw.experts is None and lw.up is not None:         # two-matrix MLP: up -> activation -> down
            u = lw.up(x).float()
            code = B.GLU_ACTS.get(c.hidden_act, 1)
            act = (F.silu(u) if code == 0 else F.gelu(u, approximate="tanh") if code == 1 else F.gelu(u) if code == 2 else torch.relu(u)).to(x.dtype)
            return self._row_parallel_norm(lw.down, act, residual, next_ln, lw.post_ln, consumer)
        if lw.experts is None:
            if lw.act_limit:
                act = MOE.glu_clamped(lw.gate_up(x), lw.gate_up.interleaved, lw.act_limit)
            elif c.hidden_act in ("silu", "swiglu"):
                act = lw.gate_up(x, swiglu=True)
            else:
                act = self._glu(lw.gate_up(x), c.hidden_act, lw.gate_up.interleaved)
            return self._row_parallel_norm(lw.down, act, residual, next_ln, lw.post_ln, consumer)
        # ---- mixture of experts ----
        fused_route = False
        if x.is_cuda and lw.router_logit_bias is None and not c.route_group_top1 and x.dtype in (torch.float16, torch.bfloat16):
            if lw.router_16 is None and lw.router.shape[0] % 8 == 0:
                lw.router_16 = lw.router.to(x.dtype).contiguous()
            fused_route = MOE.route_fused_ok(x, lw.router_16, c.num_experts_per_tok, c.n_group, c.topk_group)
        if fused_route:
            # decode-sized batch, one weight tile of experts: the router GEMM selects the experts in its epilogue
            idx, wts = MOE.route_fused(x, lw.router_16, lw.router_bias, c.num_experts_per_tok,
                                       0 if c.scoring_func == "softmax" else 1, c.norm_topk_prob, c.routed_scaling_factor)
        else:
            logits = self._router_logits(lw, x)
            if lw.router_logit_bias is not None:
                logits = logits + lw.router_logit_bias
            if c.route_group_top1:
                idx, wts = MOE.route_group_top1(logits, c.num_experts_per_tok, lw.router_scale)
            else:
                idx, wts = MOE.route_topk(logits, lw.router_bias, c.num_experts_per_tok,
                                          0 if c.scoring_func == "softmax" else 1, c.norm_topk_prob, c.n_group, c.topk_group,
                                          c.routed_scaling_factor)
        if self._beta != 1.0:
            wts = wts * self._beta
        shared = None
        if lw.shared_gate_up is not None:
            if lw.act_limit:
                shared = lw.shared_down(MOE.glu_clamped(lw.shared_gate_up(x), lw.shared_gate_up.interleaved, lw.act_limit))
            else:
                shared = lw.shared_down(lw.shared_gate_up(x, swiglu=True))
            if self._beta != 1.0:
                shared = shared * self._beta
            if lw.shared_gate is not None:
                shared = shared * torch.sigmoid(torch.matmul(x.float(), lw.shared_gate.float().t())).to(shared.dtype)
        if self._fused_active and lw.experts.stacked is not None and not self.tp.comm.fused._big(x.shape[0]):
            # expert-parallel combine fused with the cross-rank reduction + residual + norm (one kernel)
            from ..ops import moe_grouped

            parts = moe_grouped.forward(x, idx, wts, lw.experts, combine=False)
            if parts is not None:
                ys, pos, w32 = parts
                r = self.tp.comm.fused.moe_combine_ar_norm(ys, pos, w32, shared, next_ln, c.rms_eps, c.norm_unit_offset, True)
                if r is not None:
                    return r
        y = MOE.moe_forward(x, idx, wts, lw.experts, self.ep)
        if shared is not None:
            y = y + shared
        return self._reduce_norm(y, residual, next_ln, self.tp.size > 1)

    # -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, fb: ForwardBatch, kv_caches) -> torch.Tensor:
        """Returns fp32 logits ``[R, vocab_local]`` for ``fb.logit_rows`` (all rows if None)."""
        c = self.cfg
        T = fb.ids.shape[0]
        if not self.on_cuda and T <= 32 and fb.rope_pos3 is None and fb.embed_rows is None and not fb.keep_hidden:
            native = self._native_cpu()
            if native is not None:
                return native.forward(fb, kv_caches)
        fused = self.tp.comm.fused if (self.tp.size > 1 and self.tp.comm is not None) else None
        self._fused_active = bool(fused is not None and self.on_cuda and fused.usable(T, c.hidden_size) and not c.post_norms
                                  and not c.postnorm_residual and not c.parallel_block and c.norm_kind == "rms")
        if fb.is_decode and self.on_cuda and fb.decode_ws is not None and not fb.decode_planned:
            fb.decode_ws.plan(fb.kv_lens)
            fb.decode_planned = True
        if self.layer_devices is not None:
            return self._forward_staged(fb, kv_caches)
        h = self.embed_tokens(fb.ids)
        if fb.embed_rows is not None:
            h[fb.embed_rows] = fb.embed_vals.to(h.dtype)
        self._rope_override = None
        if fb.rope_pos3 is not None:
            from .vision import mrope_tables

            sec = (c.raw.get("rope_parameters") or c.raw.get("rope_scaling") or {}).get("mrope_section") or [self.rot_dim // 2, 0, 0]
            self._rope_override = mrope_tables(fb.rope_pos3.cpu(), self.rot_dim, c.rope_theta, sec, h.device)
            fb.positions = torch.arange(T, dtype=torch.int32, device=h.device)       # rows of the per-token tables
        if self._fused_active:
            h = fused.load_h(h)
        n_layers = len(self.layers)
        l0 = self.layers[0]
        x = self._norm(h, l0.lin.ln if l0.lin is not None else l0.attn.ln)
        for i, lw in enumerate(self.layers):
            # the projection that reads each fused collective's output first (it can take over the all-gather wait)
            mlp_first = lw.mlp.gate_up if lw.mlp.experts is None else None
            if c.postnorm_residual:
                # y = alpha * norm(x) + beta * f(norm(x)): the normalised rows are the residual
                fa, fbeta, la, lbeta, ma, mbeta = c.resid_factors
                alpha, self._beta = (la, lbeta) if lw.lin is not None else (fa, fbeta)
                h = x * alpha if alpha != 1.0 else x
            if c.parallel_block:
                h, _ = self._attention(lw.attn, x, fb, kv_caches[i], h, None, None)       # h + attention(x); the MLP reads x too
            elif lw.lin is not None:
                h, x = self._linear_attention(lw.lin, x, fb, kv_caches[i], h, lw.mlp.ln, mlp_first)
            else:
                h, x = self._attention(lw.attn, x, fb, kv_caches[i], h, lw.mlp.ln, mlp_first)
            if c.postnorm_residual:
                self._beta = mbeta
                h = x * ma if ma != 1.0 else x
            if i + 1 < n_layers:
                nl = self.layers[i + 1]
                next_ln = nl.lin.ln if nl.lin is not None else nl.attn.ln
                na = nl.attn
                nxt = nl.lin.in_proj if nl.lin is not None else ((na.q_a if na.q_a is not None else na.q_b) if c.use_mla else na.qkv)
            else:
                next_ln = self.final_norm
                nxt = self.lm_head if fb.logit_rows is None else None
            h, x = self._mlp(lw.mlp, x, h, i, next_ln, nxt)
        self._beta = 1.0
        self._rope_override = None
        # x is RMSNorm(h) with the final norm weight (row-wise, so selecting rows afterwards is equivalent)
        if fb.keep_hidden:
            B.flush_pending_wait()
            self.last_hidden = x
        if fb.logit_rows is not None:
            B.flush_pending_wait()
            x = x.index_select(0, fb.logit_rows)
        logits = self.lm_head(x, out_f32=True)
        B.flush_pending_wait()          # no-op unless the head ran outside the GEMM that waits itself
        if c.logit_scale != 1.0:
            logits = logits * c.logit_scale
        if c.final_softcap:
            logits = torch.tanh(logits / c.final_softcap) * c.final_softcap
        return logits

    def mtp_forward(self, fb: ForwardBatch, hidden: torch.Tensor, kv_caches):
        """Draft head over the packed rows of ``fb``: ``fb.ids`` are the tokens FOLLOWING each row's position, ``hidden`` the
        final-normed rows of the main model (or of this head, when drafts are chained).  The layer appends to its own page
        pools (``kv_caches[num_layers]``).  Returns (fp32 logits of ``fb.logit_rows``, final-normed rows of the head)."""
        mt, c = self.mtp, self.cfg
        saved = self._fused_active
        self._fused_active = False
        try:
            e = self.embed_tokens(fb.ids)
            z = mt.fc(torch.cat([self._norm(e, mt.norm_e), self._norm(hidden.to(e.dtype), mt.norm_h)], dim=-1))
            lw = mt.layer
            x = self._norm(z, lw.attn.ln)
            h, x = self._attention(lw.attn, x, fb, kv_caches[c.num_layers], z, lw.mlp.ln, None)
            h, x = self._mlp(lw.mlp, x, h, c.num_layers, mt.final_norm, None)
            B.flush_pending_wait()
            rows = x if fb.logit_rows is None else x.index_select(0, fb.logit_rows)
            logits = (mt.head or self.lm_head)(rows, out_f32=True)
            B.flush_pending_wait()
            if c.logit_scale != 1.0:
                logits = logits * c.logit_scale
            return logits, x
        finally:
            self._fused_active = saved

    def _forward_staged(self, fb: ForwardBatch, kv_caches) -> torch.Tensor:
        """Layer-split placement (``--device "{'cuda:0': 3, 'cuda:1': 2}"`` / ``cudapp``): every layer runs on its own
        device, the residual stream and the normalised activations are handed over by a peer copy at stage boundaries.
        Sequential like the reference's device map (src/fastllm.cpp:5178-5204, src/executor.cpp:211-339), no micro-batching."""
        c = self.cfg
        n_layers = len(self.layers)
        fbs: dict = {}

        def batch_on(dev):
            key = str(dev)
            if key not in fbs:
                mv = lambda t: t.to(dev, non_blocking=True) if t is not None else None
                fbs[key] = ForwardBatch(ids=mv(fb.ids), positions=mv(fb.positions), slots=mv(fb.slots), page_table=mv(fb.page_table),
                                        kv_lens=mv(fb.kv_lens), cu_q=mv(fb.cu_q), logit_rows=mv(fb.logit_rows), is_decode=fb.is_decode,
                                        cu_q_host=fb.cu_q_host)
            return fbs[key]

        ln_cache = self.__dict__.setdefault("_ln_by_device", {})

        def ln_on(w, dev):
            if w.device == dev:
                return w
            key = (id(w), str(dev))
            if key not in ln_cache:
                ln_cache[key] = w.to(dev)
            return ln_cache[key]

        dev = self.layer_devices[0]
        with torch.cuda.device(dev):
            h = self.embed_tokens(batch_on(dev).ids)
            x = self._norm(h, self.layers[0].attn.ln)
        for i, lw in enumerate(self.layers):
            nd = self.layer_devices[i]
            if nd != dev:
                h, x = h.to(nd), x.to(nd)
                dev = nd
            with torch.cuda.device(dev):
                h, x = self._attention(lw.attn, x, batch_on(dev), kv_caches[i], h, lw.mlp.ln)
                next_ln = self.layers[i + 1].attn.ln if i + 1 < n_layers else self.final_norm
                h, x = self._mlp(lw.mlp, x, h, i, ln_on(next_ln, dev))
        with torch.cuda.device(dev):
            rows = batch_on(dev).logit_rows
            if rows is not None:
                x = x.index_select(0, rows)
            logits = self.lm_head(x, out_f32=True)
            if c.logit_scale != 1.0:
                logits = logits * c.logit_scale
        return logits.to(self.device)

    def _native_cpu(self):
        """The whole-model native CPU runner for this model, or None when the architecture is outside its coverage."""
        from ..ops.quant import LinearWeight

        if LinearWeight.active_adapter is not None:
            return None                       # run-time adapters are applied by the per-operator path
        if getattr(self, "_cpu_runner", None) is None:
            from . import cpu_native

            self._cpu_runner = cpu_native.NativeCpuModel(self) if cpu_native.eligible(self) else False
        return self._cpu_runner or None

    def embed_tokens(self, ids):
        """Token embedding; the table is replicated on every tensor-parallel rank (no collective needed)."""
        h = B.embedding(ids, self.embed)
        if self.cfg.embed_scale != 1.0:
            h = h * self.cfg.embed_scale
        return h


# ---------------------------------------------------------------------------------------------------
# random initialisation of a full model of the given architecture (benchmarks and tests)
# ---------------------------------------------------------------------------------------------------
def _randn(shape, std, device, dtype, gen):
    # generate in fp32 chunks on the target device to bound peak memory
    return (torch.randn(shape, device=device, dtype=torch.float32, generator=gen) * std).to(dtype)


def _name_seed(seed: int, name: str) -> int:
    """Stable per-tensor seed: every tensor's values depend on (seed, name) only, not on what was drawn before it, so a
    rank can skip the tensors it does not keep (the other ranks' experts) and still agree with its peers on the rest."""
    import zlib

    return (seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF


def random_init(cfg: ModelConfig, device, dtype=torch.bfloat16, tp: TPInfo | None = None, ep=None, seed: int = 0,
                std: float = 0.02, wdtype: str = "auto", moe_wdtype: str | None = None, moe_device: str | None = None,
                expert_pool: int = 0) -> DecoderModel:
    """Build a model with N(0, std) weights and unit norm weights, sharded for this TP/EP rank.

    Every rank draws the full tensor from the same seed and keeps its shard, so a TP group is numerically
    a sharding of one model.  ``wdtype`` / ``moe_wdtype`` select weight quantisation (see ops.quant).
    ``expert_pool`` > 0: of a layer's local experts only the first ``expert_pool`` are drawn from the generator, the others
    are scaled copies of those (same storage size and traffic; spares the random-number passes for models with hundreds of
    experts, where drawing 80 G values per rank takes minutes).
    """
    from ..loader.shard import finalize_model   # local import: loader depends on this module

    tp = tp or TPInfo()
    m = DecoderModel(cfg, device, dtype, tp, ep)
    m.moe_numa = moe_device == "numa"
    m.moe_device = "cpu" if m.moe_numa else moe_device         # "cpu": routed experts stay in host memory (hybrid placement)
    dev = m.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    H = cfg.hidden_size
    raw: dict[str, torch.Tensor] = {}

    def mk(name, shape, s=std):
        gen.manual_seed(_name_seed(seed, name))
        raw[name] = _randn(shape, s, dev, dtype, gen)

    def ones(name, n):
        # unit gain: weight 1, or 0 for families whose norms multiply by (1 + weight); the gated delta-net norm is always plain
        unit = 0.0 if (cfg.norm_unit_offset == 1.0 and not name.endswith("linear_attn.norm.weight")) else 1.0
        raw[name] = torch.full((n,), unit, device=dev, dtype=dtype)

    # The state dict is produced layer by layer and consumed immediately to bound memory.
    def layer_tensors(i):
        raw.clear()
        p = f"model.layers.{i}."
        ones(p + "input_layernorm.weight", H)
        if cfg.norm_kind == "layernorm":
            mk(p + "input_layernorm.bias", (H,))
        if not cfg.parallel_block:
            ones(p + "post_attention_layernorm.weight", H)
        if cfg.layer_is_linear(i) and cfg.lin_kind == "lightning":
            HD = cfg.num_heads * cfg.head_dim
            mk(p + "self_attn.qkv_proj.weight", (3 * HD, H))
            mk(p + "self_attn.output_gate.weight", (HD, H))
            ones(p + "self_attn.norm.weight", HD)
            mk(p + "self_attn.out_proj.weight", (H, HD))
        elif cfg.layer_is_linear(i):
            Hk, Hv, Dk, Dv = cfg.lin_num_k_heads, cfg.lin_num_v_heads, cfg.lin_k_dim, cfg.lin_v_dim
            lp = p + "linear_attn."
            mk(lp + "in_proj_qkvz.weight", (2 * Hk * Dk + 2 * Hv * Dv, H))
            mk(lp + "in_proj_ba.weight", (2 * Hv, H))
            mk(lp + "conv1d.weight", (2 * Hk * Dk + Hv * Dv, 1, cfg.lin_conv_kernel), 0.3)
            gen.manual_seed(_name_seed(seed, lp + "A_log"))
            raw[lp + "A_log"] = torch.log(torch.rand(Hv, device=dev, generator=gen) * 4 + 0.5)
            raw[lp + "dt_bias"] = torch.ones(Hv, device=dev, dtype=torch.float32)
            ones(lp + "norm.weight", Dv)
            mk(lp + "out_proj.weight", (H, Hv * Dv))
        elif cfg.use_mla:
            qd = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
            if cfg.q_lora_rank:
                mk(p + "self_attn.q_a_proj.weight", (cfg.q_lora_rank, H))
                ones(p + "self_attn.q_a_layernorm.weight", cfg.q_lora_rank)
                mk(p + "self_attn.q_b_proj.weight", (cfg.num_heads * qd, cfg.q_lora_rank))
            else:
                mk(p + "self_attn.q_proj.weight", (cfg.num_heads * qd, H))
            mk(p + "self_attn.kv_a_proj_with_mqa.weight", (cfg.kv_lora_rank + cfg.qk_rope_head_dim, H))
            ones(p + "self_attn.kv_a_layernorm.weight", cfg.kv_lora_rank)
            mk(p + "self_attn.kv_b_proj.weight", (cfg.num_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank))
            mk(p + "self_attn.o_proj.weight", (H, cfg.num_heads * cfg.v_head_dim))
            if cfg.index_topk and cfg.q_lora_rank:
                Hi, Di = cfg.index_n_heads, cfg.index_head_dim
                mk(p + "self_attn.indexer.wq_b.weight", (Hi * Di, cfg.q_lora_rank))
                mk(p + "self_attn.indexer.wk.weight", (Di, H))
                raw[p + "self_attn.indexer.k_norm.weight"] = torch.ones(Di, device=dev, dtype=torch.float32)
                raw[p + "self_attn.indexer.k_norm.bias"] = torch.zeros(Di, device=dev, dtype=torch.float32)
                mk(p + "self_attn.indexer.weights_proj.weight", (Hi, H))
        else:
            D = cfg.head_dim
            nh = cfg.layer_heads[i] if cfg.layer_heads else cfg.num_heads
            mk(p + "self_attn.q_proj.weight", (nh * D * (2 if cfg.attn_output_gate else 1), H))
            mk(p + "self_attn.k_proj.weight", (cfg.num_kv_heads * D, H))
            mk(p + "self_attn.v_proj.weight", (cfg.num_kv_heads * D, H))
            mk(p + "self_attn.o_proj.weight", (H, nh * D))
            if cfg.head_gate:
                mk(p + "self_attn.g_proj.weight", (nh, H))
            if cfg.attention_bias:
                mk(p + "self_attn.q_proj.bias", (nh * D,))
                mk(p + "self_attn.k_proj.bias", (cfg.num_kv_heads * D,))
                mk(p + "self_attn.v_proj.bias", (cfg.num_kv_heads * D,))
            if cfg.qk_norm:
                ones(p + "self_attn.q_norm.weight", cfg.num_heads * D if cfg.qk_norm_full else D)
                ones(p + "self_attn.k_norm.weight", cfg.num_kv_heads * D if cfg.qk_norm_full else D)
        if cfg.layer_is_moe(i):
            mk(p + "mlp.gate.weight", (cfg.num_experts, H))
            if cfg.router_bias:
                raw[p + "mlp.gate.e_score_correction_bias"] = torch.zeros(cfg.num_experts, device=dev, dtype=torch.float32)
            if cfg.route_group_top1:
                raw[p + "mlp.router_scale"] = torch.ones(cfg.num_experts, device=dev, dtype=torch.float32)
            lo, hi = MOE.local_expert_range(cfg.num_experts, ep)
            I = cfg.moe_intermediate_size
            # tensors are seeded by name, so only this rank's experts are drawn (with MoE tensor parallelism: all of them)
            for e in range(lo, hi):
                for nm, shp in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
                    if expert_pool > 0 and e - lo >= expert_pool:
                        base = raw[p + f"mlp.experts.{lo + (e - lo) % expert_pool}.{nm}.weight"]
                        raw[p + f"mlp.experts.{e}.{nm}.weight"] = base * (1.0 + ((e - lo) // expert_pool) / 64.0)
                    else:
                        mk(p + f"mlp.experts.{e}.{nm}.weight", shp)
            if cfg.num_shared_experts:
                SI = cfg.shared_expert_intermediate_size
                sp = p + ("mlp.shared_expert." if cfg.shared_expert_gate else "mlp.shared_experts.")
                mk(sp + "gate_proj.weight", (SI, H))
                mk(sp + "up_proj.weight", (SI, H))
                mk(sp + "down_proj.weight", (H, SI))
                if cfg.shared_expert_gate:
                    mk(p + "mlp.shared_expert_gate.weight", (1, H))
        else:
            I = cfg.intermediate_size
            if cfg.mlp_gated:
                mk(p + "mlp.gate_proj.weight", (I, H))
            mk(p + "mlp.up_proj.weight", (I, H))
            mk(p + "mlp.down_proj.weight", (H, I))
            if cfg.mlp_bias and not cfg.mlp_gated:
                mk(p + "mlp.up_proj.bias", (I,))
                mk(p + "mlp.down_proj.bias", (H,))
        return raw

    def top_tensors():
        raw.clear()
        mk("model.embed_tokens.weight", (cfg.vocab_size, H))
        ones("model.norm.weight", H)
        if cfg.norm_kind == "layernorm":
            mk("model.norm.bias", (H,))
        if not cfg.tie_embeddings:
            mk("lm_head.weight", (cfg.vocab_size, H))
        return raw

    finalize_model(m, top_tensors, layer_tensors, wdtype=wdtype, moe_wdtype=moe_wdtype)
    if cfg.mtp_layers:
        from ..loader.shard import build_mtp

        L = cfg.num_layers
        t = dict(layer_tensors(L))
        p = f"model.layers.{L}."
        raw.clear()
        ones(p + "enorm.weight", H)
        ones(p + "hnorm.weight", H)
        mk(p + "eh_proj.weight", (H, 2 * H))
        ones(p + "shared_head.norm.weight", H)
        t.update(raw)
        build_mtp(m, t, wdtype, moe_wdtype)
    return m
