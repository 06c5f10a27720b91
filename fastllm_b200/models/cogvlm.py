"""CogVLM: a Llama-style decoder whose image tokens run through their own attention and MLP weights ("visual expert"),
behind an EVA-CLIP vision transformer with a 2x2 convolutional down-sampler and a gated projector.

Reference: src/models/cogvlm.cpp (:160-260 the vision path, :284-455 the decoder with the expert switch, :487-520 the position
ids).  What runs where:

* The language expert's weights are the decoder's ordinary weights, so text-only prefill chunks and every decode step take the
  framework's kernels (and CUDA graphs) unchanged.
* A prefill chunk that holds image tokens is evaluated by ``CogVLMModel._forward_mixed``: both experts' projections on their own
  rows, rotary embedding, paged KV append and attention with PyTorch ops.  This happens once per image.
* Sequence layout: ``[bos] [boi, G x G patch tokens, eoi] text...``; the rows ``boi .. last patch`` use the visual expert
  (a row is "visual" when it and its successor are image tokens, as in the model's own definition, which leaves ``eoi`` to the
  language expert).  Rotary positions: bos 0, boi 1, every patch 2, eoi 3, text 4, 5, ... (the reference's table leaves the
  last patch at position 0, cogvlm.cpp:499-507; the model's definition, which this file follows, gives it 2 like the others).
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

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


class CogVLMVision:
    """EVA-CLIP tower: patch convolution, class token, learned positions, post-norm transformer layers (``x + LN(f(x))``),
    2x2 stride-2 convolution over the patch grid, gated projector to the decoder width, learned ``boi`` / ``eoi`` rows."""

    def __init__(self, vc: dict, w: dict, device, dtype):
        self.hidden = int(vc["hidden_size"])
        self.heads = int(vc["num_heads"])
        self.layers = int(vc["num_hidden_layers"])
        self.patch = int(vc["patch_size"])
        self.image_size = int(vc["image_size"])
        self.eps = float(vc.get("layer_norm_eps", 1e-6))
        self.grid = self.image_size // self.patch // 2
        self.tokens = self.grid * self.grid + 2
        self.device, self.dtype = device, dtype
        self.w = {k: v.to(device=device, dtype=dtype) for k, v in w.items()}

    def _lin(self, x, name):
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _ln(self, x, name, eps):
        return F.layer_norm(x.float(), (x.shape[-1],), self.w[name + ".weight"].float(), self.w[name + ".bias"].float(), eps).to(x.dtype)

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[N, 3, S, S]`` normalised pixels -> ``[N, G * G + 2, decoder width]``."""
        w = self.w
        x = F.conv2d(pixels.to(device=self.device, dtype=self.dtype), w["patch_embedding.proj.weight"], w.get("patch_embedding.proj.bias"),
                     stride=self.patch)
        N = x.shape[0]
        x = x.flatten(2).transpose(1, 2)
        x = torch.cat([w["patch_embedding.cls_embedding"].reshape(1, 1, -1).expand(N, -1, -1), x], dim=1)
        x = x + w["patch_embedding.position_embedding.weight"][None, :x.shape[1]]
        L, Hd = x.shape[1], self.hidden // self.heads
        for i in range(self.layers):
            p = f"transformer.layers.{i}."
            qkv = self._lin(x, p + "attention.query_key_value").reshape(N, L, 3, self.heads, Hd).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
            a = self._lin(a.transpose(1, 2).reshape(N, L, self.hidden), p + "attention.dense")
            x = x + self._ln(a, p + "input_layernorm", self.eps)
            m = self._lin(F.gelu(self._lin(x, p + "mlp.fc1")), p + "mlp.fc2")
            x = x + self._ln(m, p + "post_attention_layernorm", self.eps)
        x = x[:, 1:]
        g = int(math.isqrt(x.shape[1]))
        x = F.conv2d(x.reshape(N, g, g, self.hidden).permute(0, 3, 1, 2), w["conv.weight"], w.get("conv.bias"), stride=2)
        x = x.flatten(2).transpose(1, 2)
        y = F.gelu(self._ln(self._lin(x, "linear_proj.linear_proj"), "linear_proj.norm1", 1e-5))
        y = self._lin(F.silu(self._lin(y, "linear_proj.gate_proj")) * self._lin(y, "linear_proj.dense_h_to_4h"), "linear_proj.dense_4h_to_h")
        boi = w["boi"].reshape(1, 1, -1).expand(N, -1, -1)
        eoi = w["eoi"].reshape(1, 1, -1).expand(N, -1, -1)
        return torch.cat([boi, y, eoi], dim=1)


class VisualExpert:
    """One layer's visual-expert projections."""

    def __init__(self):
        self.qkv: LinearWeight | None = None
        self.o: LinearWeight | None = None
        self.gate_up: LinearWeight | None = None
        self.down: LinearWeight | None = None


class CogVLMModel(DecoderModel):
    def __init__(self, cfg: ModelConfig, device, dtype=torch.bfloat16, tp=None, ep=None):
        super().__init__(cfg, device, dtype, tp, ep)
        self.vexp: list[VisualExpert] = []
        self.vision: CogVLMVision | None = None
        self.image_token_id = int(cfg.raw.get("pad_token_id", 0) or 0)      # placeholder id of the image rows (their embeddings are replaced)

    @torch.no_grad()
    def forward(self, fb: ForwardBatch, kv_caches) -> torch.Tensor:
        rows = getattr(fb, "expert_rows", None)
        if rows is None or rows.numel() == 0 or not self.vexp:
            return super().forward(fb, kv_caches)
        return self._forward_mixed(fb, kv_caches, rows)

    def _both(self, x, lang: LinearWeight, vis: LinearWeight, vrows, lrows):
        out = None
        if lrows.numel():
            yl = lang(x.index_select(0, lrows))
            out = torch.empty((x.shape[0], yl.shape[-1]), dtype=yl.dtype, device=x.device)
            out[lrows] = yl
        yv = vis(x.index_select(0, vrows))
        if out is None:
            out = torch.empty((x.shape[0], yv.shape[-1]), dtype=yv.dtype, device=x.device)
        out[vrows] = yv.to(out.dtype)
        return out

    def _forward_mixed(self, fb: ForwardBatch, kv_caches, vrows) -> torch.Tensor:
        c = self.cfg
        T = fb.ids.shape[0]
        Hq, Hkv, D = self.num_heads_local, self.num_kv_heads_local, c.head_dim
        h = self.embed_tokens(fb.ids)
        if fb.embed_rows is not None:
            h[fb.embed_rows] = fb.embed_vals.to(h.dtype)
        is_v = torch.zeros(T, dtype=torch.bool, device=h.device)
        is_v[vrows] = True
        lrows = torch.nonzero(~is_v).flatten()
        pos = fb.rope_pos3[0].to(h.device) if fb.rope_pos3 is not None else fb.positions
        cos, sin = self.rope_tables(device=h.device)
        valid = fb.slots >= 0
        sl = fb.slots[valid].long()
        scale = 1.0 / math.sqrt(D)
        for lw, ve, (k_pool, v_pool) in zip(self.layers, self.vexp, kv_caches):
            x = B.rmsnorm_ref(h, lw.attn.ln, c.rms_eps)[0]
            qkv = self._both(x, lw.attn.qkv, ve.qkv, vrows, lrows)
            q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
            q = A.apply_rope_ref(q.reshape(T, Hq, D), pos, cos, sin, A.ROPE_NEOX, self.rot_dim)
            k = A.apply_rope_ref(k.reshape(T, Hkv, D), pos, cos, sin, A.ROPE_NEOX, self.rot_dim)
            k_pool.view(-1, Hkv, D)[sl] = k[valid].to(k_pool.dtype)
            v_pool.view(-1, Hkv, D)[sl] = v.reshape(T, Hkv, D)[valid].to(v_pool.dtype)
            a = A.paged_attention_general(q.reshape(T, Hq * D).to(h.dtype), k_pool, v_pool, fb.page_table, fb.kv_lens, fb.cu_q, scale,
                                          Hq, Hkv, D)
            h = h + self._both(a, lw.attn.o, ve.o, vrows, lrows).to(h.dtype)
            x = B.rmsnorm_ref(h, lw.mlp.ln, c.rms_eps)[0]
            y = torch.empty_like(h)
            if lrows.numel():
                xl = x.index_select(0, lrows)
                y[lrows] = lw.mlp.down(B.glu_act(lw.mlp.gate_up(xl), "silu", lw.mlp.gate_up.interleaved)).to(h.dtype)
            xv = x.index_select(0, vrows)
            y[vrows] = ve.down(B.glu_act(ve.gate_up(xv), "silu", ve.gate_up.interleaved)).to(h.dtype)
            h = h + y
        x = B.rmsnorm_ref(h, self.final_norm, c.rms_eps)[0]
        if fb.keep_hidden:
            self.last_hidden = x
        if fb.logit_rows is not None:
            x = x.index_select(0, fb.logit_rows)
        return self.lm_head(x, out_f32=True)


def attach(m: CogVLMModel, ck, cfg: ModelConfig, wdtype: str = "dense") -> None:
    """Load the visual experts and the vision tower of a CogVLM checkpoint into a model whose language expert is in place."""
    from ..loader.shard import _gate_up, _lin

    kind = wdtype if wdtype not in ("auto", None) else "dense"
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        ve = VisualExpert()
        ve.qkv = _lin(m, ck.raw(p + "self_attn.vision_expert_query_key_value.weight"), kind,
                      ck.raw(p + "self_attn.vision_expert_query_key_value.bias") if ck.has(p + "self_attn.vision_expert_query_key_value.bias") else None)
        ve.o = _lin(m, ck.raw(p + "self_attn.vision_expert_dense.weight"), kind)
        ve.gate_up = _gate_up(m, ck.raw(p + "mlp.vision_mlp.gate_proj.weight"), ck.raw(p + "mlp.vision_mlp.up_proj.weight"), kind)
        ve.down = _lin(m, ck.raw(p + "mlp.vision_mlp.down_proj.weight"), kind)
        m.vexp.append(ve)
    vc = cfg.raw.get("vision_config")
    names = [n for n in ck.names if n.startswith("model.vision.")]
    if isinstance(vc, dict) and names:
        m.vision = CogVLMVision(vc, {n[len("model.vision."):]: ck.raw(n) for n in names}, m.device, m.dtype)


def preprocess(image, size: int) -> torch.Tensor:
    """An image (path, bytes, ``data:`` URL, PIL image or ``[3, H, W]`` tensor in 0..1) -> ``[3, size, size]`` normalised pixels
    (bicubic resize to the tower's square input, CLIP mean / deviation)."""
    if isinstance(image, torch.Tensor):
        px = image.float()
    else:
        from .vision import load_image

        im = load_image(image).convert("RGB")
        import numpy as np

        px = torch.from_numpy(np.asarray(im).copy()).permute(2, 0, 1).float() / 255.0
    if px.shape[-2:] != (size, size):
        px = F.interpolate(px[None], size=(size, size), mode="bicubic", align_corners=False)[0].clamp(0.0, 1.0)
    mean = torch.tensor(CLIP_MEAN).reshape(3, 1, 1)
    std = torch.tensor(CLIP_STD).reshape(3, 1, 1)
    return (px - mean) / std


def positions_for(prompt_len: int, image_tokens: int):
    """Rotary positions of ``[bos] [image rows] text...`` and the offset of every later token's position from its index."""
    V = image_tokens
    pos = [0, 1] + [2] * (V - 2) + [3]
    pos += list(range(4, 4 + prompt_len - (V + 1)))
    delta = 3 - V                                      # index V (eoi) has position 3
    return torch.tensor(pos, dtype=torch.long), delta


def build_context(model: CogVLMModel, ids, images):
    """Text token ids (starting with bos) and one image -> (ids with the image rows inserted behind bos, the request's
    ``MultimodalContext``: tower output for those rows, rotary positions, the rows of the visual expert)."""
    from ..engine.engine import MultimodalContext

    if model.vision is None:
        raise ValueError("this checkpoint has no vision tower: image inputs are not supported")
    if len(images) != 1:
        raise ValueError("CogVLM takes exactly one image per conversation")
    tower = model.vision
    emb = tower.forward(preprocess(images[0], tower.image_size)[None])[0]
    V = emb.shape[0]
    ids = list(ids)
    if not ids:
        raise ValueError("empty prompt")
    out = ids[:1] + [model.image_token_id] * V + ids[1:]
    pos, delta = positions_for(len(out), V)
    ctx = MultimodalContext(emb, range(1, V + 1), pos[None].expand(3, -1).contiguous(), delta, expert_positions=range(1, V))
    return out, ctx
