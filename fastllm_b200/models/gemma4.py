"""Gemma-4 text decoder (dense and mixture-of-experts variants).

What sets the family apart from the shared decoder (``models/decoder.py``):

* sliding-window layers and full-attention layers differ in head width (``head_dim`` / ``global_head_dim``) and may differ
  in KV heads, so every layer owns page pools of its own shape;
* the last ``num_kv_shared_layers`` layers project no keys / values: they read the pages of the last earlier layer of their
  type; with ``attention_k_eq_v`` the full-attention layers use the key projection for the values too;
* queries, keys (with a learned scale) and values (without) are RMS-normalised per head, the softmax scale is 1;
* full-attention layers rotate only the leading fraction of the rotate-half pairs ("proportional" rotary);
* a second embedding table gives every layer a small per-token input that gates a low-rank update after the MLP;
* with ``enable_moe_block`` a routed expert block runs beside the dense MLP, each behind its own norms;
* every layer ends with a stored scalar, the logits with tanh soft-capping.

The forward pass is evaluated with the framework's linear layers (any run-time weight format) and the paged PyTorch
attention; it runs on one rank.  Reference: src/models/gemma4.cpp (Gemma4Model::ForwardBatch, weight names :60-140).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..ops import attention as A
from ..ops import basic as B
from ..ops.quant import LinearWeight
from .config import ModelConfig
from .decoder import DecoderModel, ForwardBatch


def _rms(x, w, eps):
    xf = x.float()
    y = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    return (y * w.float() if w is not None else y).to(x.dtype)


class _Layer:
    pass


class Gemma4Model(DecoderModel):
    def __init__(self, cfg: ModelConfig, device, dtype=torch.bfloat16, tp=None, ep=None):
        super().__init__(cfg, device, dtype, tp, ep)
        if self.tp.size != 1:
            raise NotImplementedError("gemma4 runs on one rank")
        r = cfg.raw
        L = cfg.num_layers
        self.general_attn = True                      # PyTorch paged attention: not captured in CUDA graphs
        lt = r.get("layer_types") or ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(L)]
        lt = list(lt)
        lt[-1] = "full_attention"
        self.layer_kinds = lt
        self.d_local = int(r.get("head_dim", 256))
        self.d_global = int(r.get("global_head_dim") or self.d_local)
        self.k_eq_v = bool(r.get("attention_k_eq_v", False))
        self.kv_local = int(r.get("num_key_value_heads", cfg.num_heads))
        self.kv_global = int(r.get("num_global_key_value_heads") or self.kv_local) if self.k_eq_v else self.kv_local
        self.window = int(r.get("sliding_window", 512))
        self.first_shared = L - int(r.get("num_kv_shared_layers", 0) or 0)
        self.pli = int(r.get("hidden_size_per_layer_input", 0) or 0)
        self.moe = bool(r.get("enable_moe_block", False))
        self.top_k = int(r.get("top_k_experts") or 0)
        self.softcap = float(r.get("final_logit_softcapping") or 0.0)
        self.act = r.get("hidden_activation", "gelu_pytorch_tanh")
        rp = r.get("rope_parameters") or {}
        self.rope_spec = {"sliding_attention": dict(rp.get("sliding_attention") or {"rope_type": "default", "rope_theta": 10000.0}),
                          "full_attention": dict(rp.get("full_attention") or {"rope_type": "proportional", "partial_rotary_factor": 0.25,
                                                                                "rope_theta": 1000000.0})}
        self.g4: list[_Layer] = []
        self._tables = {}

    # ---- geometry -------------------------------------------------------------------------------------------------
    def layer_dims(self, i: int):
        """(head width, KV heads) of layer ``i``."""
        full = self.layer_kinds[i] == "full_attention"
        return (self.d_global if full else self.d_local), (self.kv_global if full else self.kv_local)

    def kv_donor(self, i: int) -> int:
        """The layer whose pages layer ``i`` reads: itself, or the last layer of its type before the sharing region."""
        if i < self.first_shared or self.first_shared <= 0:
            return i
        prev = self.layer_kinds[:self.first_shared]
        return len(prev) - 1 - prev[::-1].index(self.layer_kinds[i])

    def kv_cache_shape_layer(self, i: int, num_pages: int):
        if self.kv_donor(i) != i:
            return None
        d, kv = self.layer_dims(i)
        s = (num_pages, A.PAGE_LEN, kv, d)
        return s, s

    def kv_cache_shape(self, num_pages: int):
        return self.kv_cache_shape_layer(0, num_pages)

    def kv_bytes_per_page(self) -> int:
        n = 0
        for i in range(self.cfg.num_layers):
            s = self.kv_cache_shape_layer(i, 1)
            if s is not None:
                n += 2 * math.prod(s[0])
        return n * torch.finfo(getattr(self, "kv_dtype", None) or self.dtype).bits // 8

    def _rope_for(self, kind: str, device):
        key = (kind, str(device))
        if key not in self._tables:
            spec = self.rope_spec[kind]
            D = self.d_global if kind == "full_attention" else self.d_local
            theta = float(spec.get("rope_theta", 10000.0))
            mp = min(self.cfg.max_position, 1 << 17)
            if spec.get("rope_type", "default") == "proportional":
                # the leading `angles` rotate-half pairs turn, at frequencies spaced over the whole head; the rest stay put
                angles = int(float(spec.get("partial_rotary_factor", 1.0)) * D // 2)
                inv = torch.zeros(D // 2, dtype=torch.float64)
                inv[:angles] = 1.0 / (theta ** (torch.arange(0, 2 * angles, 2, dtype=torch.float64) / D))
                inv = inv / float(spec.get("factor", 1.0))
            else:
                inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
            ang = torch.arange(mp, dtype=torch.float64)[:, None] * inv[None, :]
            self._tables[key] = (ang.cos().float().to(device), ang.sin().float().to(device))
        return self._tables[key]

    # ---- forward --------------------------------------------------------------------------------------------------
    def forward(self, fb: ForwardBatch, kv_caches) -> torch.Tensor:
        c = self.cfg
        eps = c.rms_eps
        ids = fb.ids.long()
        T = ids.shape[0]
        H, L = c.hidden_size, c.num_layers
        h = self.embed[ids] * torch.tensor(H ** 0.5, dtype=self.embed.dtype)
        per_layer = None
        if self.pli:
            P = self.pli
            tok = (self.embed_per_layer[ids] * torch.tensor(P ** 0.5, dtype=self.embed_per_layer.dtype)).reshape(T, L, P)
            proj = (self.pl_model_proj(h) * (H ** -0.5)).reshape(T, L, P)
            per_layer = (_rms(proj, self.pl_proj_norm, eps) + tok) * (2.0 ** -0.5)
        valid = fb.slots >= 0
        sl = fb.slots[valid].long()
        for i, lw in enumerate(self.g4):
            kind = self.layer_kinds[i]
            D, Hkv = self.layer_dims(i)
            Hq = c.num_heads
            cos, sin = self._rope_for(kind, h.device)
            x = _rms(h, lw.input_ln, eps)
            q = _rms(lw.q(x).reshape(T, Hq, D), lw.q_norm, eps)
            q = A.apply_rope_ref(q, fb.positions, cos, sin, A.ROPE_NEOX, D)
            k_pool, v_pool = kv_caches[i]
            if lw.k is not None:
                k_raw = lw.k(x).reshape(T, Hkv, D)
                v_raw = lw.v(x).reshape(T, Hkv, D) if lw.v is not None else k_raw
                k = A.apply_rope_ref(_rms(k_raw, lw.k_norm, eps), fb.positions, cos, sin, A.ROPE_NEOX, D)
                v = _rms(v_raw, None, eps)
                k_pool.view(-1, Hkv, D)[sl] = k[valid].to(k_pool.dtype)
                v_pool.view(-1, Hkv, D)[sl] = v[valid].to(v_pool.dtype)
            a = A.paged_attention_general(q.reshape(T, Hq * D).to(h.dtype), k_pool, v_pool, fb.page_table, fb.kv_lens, fb.cu_q, 1.0,
                                          Hq, Hkv, D, window=self.window if kind == "sliding_attention" else 0)
            h = h + _rms(lw.o(a), lw.post_attn_ln, eps)
            res = h
            y = lw.down(B.glu_act(lw.gate_up(_rms(h, lw.pre_ff_ln, eps)), self.act, lw.gate_up.interleaved))
            if self.moe:
                y1 = _rms(y, lw.post_ff_ln_1, eps)
                rin = _rms(res, None, eps) * lw.router_scale.to(h.dtype) * (H ** -0.5)
                pr = torch.softmax(torch.matmul(rin.float(), lw.router.float().t()), dim=-1)
                w, idx = pr.topk(self.top_k, dim=-1)
                w = w / w.sum(-1, keepdim=True) * lw.per_expert_scale.float()[idx]
                xin = _rms(res, lw.pre_ff_ln_2, eps)
                y2 = torch.zeros((T, H), dtype=torch.float32, device=h.device)
                for e in idx.unique().tolist():
                    rows, pos = torch.where(idx == e)
                    he = lw.exp_down[e](B.glu_act(lw.exp_gate_up[e](xin[rows]), self.act, lw.exp_gate_up[e].interleaved))
                    y2.index_add_(0, rows, he.float() * w[rows, pos, None])
                y = y1 + _rms(y2.to(h.dtype), lw.post_ff_ln_2, eps)
            h = res + _rms(y, lw.post_ff_ln, eps)
            if self.pli:
                g = F.gelu(lw.pl_gate(h).float(), approximate="tanh").to(h.dtype) * per_layer[:, i, :].to(h.dtype)
                h = h + _rms(lw.pl_proj(g), lw.post_pl_norm, eps)
            h = h * lw.scalar
        x = _rms(h, self.final_norm, eps)
        if fb.logit_rows is not None:
            x = x.index_select(0, fb.logit_rows)
        logits = self.lm_head(x, out_f32=True)
        if self.softcap:
            logits = torch.tanh(logits / self.softcap) * self.softcap
        return logits


def build(ck, cfg: ModelConfig, device, dtype, wdtype="dense", moe_wdtype=None) -> Gemma4Model:
    """Fill a ``Gemma4Model`` from a checkpoint index (``loader.hf.HFCheckpoint``-like: ``has`` / ``raw`` / ``collect``)."""
    m = Gemma4Model(cfg, device, dtype)
    dev = m.device
    on_cuda = dev.type == "cuda"
    to = lambda t: None if t is None else t.to(dev, dtype).contiguous()

    def lin(w, kind=wdtype):
        return LinearWeight.from_dense(to(w), kind, None, False, act_dtype=dtype)

    def gate_up(gw, uw, kind=wdtype):
        if on_cuda and gw.shape[0] % 64 == 0:
            return LinearWeight.from_dense(B.interleave_gate_up(to(gw), to(uw)), kind, None, True, act_dtype=dtype)
        return LinearWeight.from_dense(torch.cat([to(gw), to(uw)], dim=0), kind, None, False, act_dtype=dtype)

    m.embed = to(ck.raw("model.embed_tokens.weight"))
    m.final_norm = to(ck.raw("model.norm.weight"))
    head = ck.raw("lm_head.weight") if ck.has("lm_head.weight") and not cfg.tie_embeddings else None
    m.lm_head = LinearWeight("dense", m.embed, dtype=dtype) if head is None else lin(head, "dense")
    if m.pli:
        m.embed_per_layer = to(ck.raw("model.embed_tokens_per_layer.weight"))
        m.pl_model_proj = lin(ck.raw("model.per_layer_model_projection.weight"), "dense")
        m.pl_proj_norm = to(ck.raw("model.per_layer_projection_norm.weight"))
    for i in range(cfg.num_layers):
        t = ck.collect(f"model.layers.{i}.")
        g = lambda k: t.get(f"model.layers.{i}." + k)
        lw = _Layer()
        lw.input_ln, lw.post_attn_ln = to(g("input_layernorm.weight")), to(g("post_attention_layernorm.weight"))
        lw.pre_ff_ln, lw.post_ff_ln = to(g("pre_feedforward_layernorm.weight")), to(g("post_feedforward_layernorm.weight"))
        lw.q, lw.o = lin(g("self_attn.q_proj.weight")), lin(g("self_attn.o_proj.weight"))
        lw.q_norm, lw.k_norm = to(g("self_attn.q_norm.weight")), to(g("self_attn.k_norm.weight"))
        shared = m.kv_donor(i) != i
        lw.k = None if shared else lin(g("self_attn.k_proj.weight"))
        vw = g("self_attn.v_proj.weight")
        lw.v = None if (shared or vw is None) else lin(vw)
        lw.gate_up = gate_up(g("mlp.gate_proj.weight"), g("mlp.up_proj.weight"))
        lw.down = lin(g("mlp.down_proj.weight"))
        sc = g("layer_scalar")
        lw.scalar = float(sc.reshape(-1)[0]) if sc is not None else 1.0
        if m.pli:
            lw.pl_gate, lw.pl_proj = lin(g("per_layer_input_gate.weight"), "dense"), lin(g("per_layer_projection.weight"), "dense")
            lw.post_pl_norm = to(g("post_per_layer_input_norm.weight"))
        if m.moe:
            lw.router = g("router.proj.weight").to(dev, torch.float32).contiguous()
            lw.router_scale = to(g("router.scale"))
            lw.per_expert_scale = g("router.per_expert_scale").to(dev, torch.float32)
            lw.post_ff_ln_1, lw.post_ff_ln_2 = to(g("post_feedforward_layernorm_1.weight")), to(g("post_feedforward_layernorm_2.weight"))
            lw.pre_ff_ln_2 = to(g("pre_feedforward_layernorm_2.weight"))
            mk = moe_wdtype or wdtype
            gu, dn = g("experts.gate_up_proj"), g("experts.down_proj")
            lw.exp_gate_up, lw.exp_down = [], []
            for e in range(gu.shape[0]):
                gw, uw = gu[e].chunk(2, dim=0)
                lw.exp_gate_up.append(gate_up(gw, uw, mk))
                lw.exp_down.append(lin(dn[e], mk))
        m.g4.append(lw)
    return m
