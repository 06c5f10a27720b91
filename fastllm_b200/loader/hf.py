"""Load a Hugging Face model folder (config.json + safetensors) into a ``DecoderModel``.

Covers the reference's ``CreateLLMModelFromHF`` pipeline (src/model.cpp:3205-4188): config parsing, tensor
name mapping per family, pre-quantised checkpoints (block-scaled FP8 ``weight_scale_inv``, AWQ
``qweight/qzeros/scales``, exporter ``fastllm`` blobs), ``--dtype`` / ``--moe_dtype`` quantisation at load,
``dtype_config`` regex rules (last match wins, src/model.cpp:3454-3466), q/k/v and gate/up merging, and
tensor-parallel sharding.  Tensors are streamed one layer at a time so host memory stays bounded.
"""
from __future__ import annotations

import json
import re
from pathlib import Path

import torch

from ..models.config import ModelConfig, load_config
from ..models.decoder import DecoderModel, TPInfo
from . import safetensors as st
from .shard import finalize_model

# AWQ packs eight 4-bit values per int32 in this nibble order (reference: src/model.cpp:1143-1218)
_AWQ_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]


def dequant_fp8_block(w: torch.Tensor, scale_inv: torch.Tensor, dtype=torch.bfloat16, block: int = 128) -> torch.Tensor:
    """``w`` float8_e4m3 [N, K], ``scale_inv`` fp32 [ceil(N/128), ceil(K/128)] -> dense."""
    n, k = w.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return (w.float() * s).to(dtype)


_FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)       # e2m1


def _fp4_unpack(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., n] -> fp32 [..., 2n]: the low nibble is the even element, the high nibble the odd one."""
    lut = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=packed.device)
    lo, hi = (packed & 0x0F).long(), (packed >> 4).long()
    return torch.stack([lut[lo], lut[hi]], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """MXFP4 (gpt-oss checkpoints): ``blocks`` uint8 [..., rows, K/32, 16] with two e2m1 values per byte, ``scales`` uint8
    e8m0 [..., rows, K/32] (value 2^(s - 127)) -> dense [..., rows, K].  Reference: the MXFP4 expert path of
    src/models/gpt_oss.cpp and src/devices/cuda/moe/fastllm-moe-vllm-marlin.cu:293-331 (repacks the same format for Marlin)."""
    vals = _fp4_unpack(blocks)                                             # [..., rows, K/32, 32]
    sc = torch.exp2(scales.float() - 127.0)[..., None]
    return (vals * sc).reshape(*blocks.shape[:-2], blocks.shape[-2] * 32).to(dtype)


def dequant_nvfp4(w: torch.Tensor, block_scale: torch.Tensor, global_scale: torch.Tensor | None, dtype=torch.bfloat16) -> torch.Tensor:
    """NVFP4: ``w`` uint8 [N, K/2] (e2m1 pairs), ``block_scale`` e4m3 (or e8m0 as uint8) [N, K/block] with block 16 or 32,
    optional fp32 ``global_scale`` -> dense [N, K].  Reference formats NVFP4_BLOCK_16 / _E8M0 / NVFP4_BLOCK_32_E8M0
    (include/fastllm.h:308-339; de-quantisers src/devices/cuda/linear/fastllm-linear-fp8.cu:2375-2690)."""
    N, K = w.shape[0], w.shape[1] * 2
    vals = _fp4_unpack(w)
    blk = K // block_scale.shape[1]
    sc = torch.exp2(block_scale.float() - 127.0) if block_scale.dtype == torch.uint8 else block_scale.float()
    out = vals.reshape(N, K // blk, blk) * sc[..., None]
    if global_scale is not None:
        out = out * global_scale.float().reshape(-1)[0]
    return out.reshape(N, K).to(dtype)


def dequant_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """AWQ GEMM layout: qweight int32 [K, N/8], qzeros int32 [K/g, N/8], scales fp16 [K/g, N] -> dense [N, K]."""
    K, n8 = qweight.shape
    N = n8 * 8
    shifts = torch.tensor([4 * i for i in _AWQ_ORDER], dtype=torch.int32)
    w = ((qweight[:, :, None] >> shifts[None, None, :]) & 0xF).reshape(K, N)          # [K, N]
    z = ((qzeros[:, :, None] >> shifts[None, None, :]) & 0xF).reshape(qzeros.shape[0], N)
    g = K // scales.shape[0]
    z = z.repeat_interleave(g, 0)
    sc = scales.float().repeat_interleave(g, 0)
    return ((w.float() - z.float()) * sc).t().contiguous().to(dtype)


# ---------------------------------------------------------------------------------------------------
# name canonicalisation: every family is mapped onto the Llama naming that loader.shard understands
# ---------------------------------------------------------------------------------------------------
_RENAMES = [
    (r"\.mlp\.moe_statics\.e_score_correction_bias", ".mlp.gate.e_score_correction_bias"),          # Ernie-4.5-MoE
    (r"\.block_sparse_moe\.e_score_correction_bias", ".mlp.gate.e_score_correction_bias"),          # MiniMax-M2
    (r"\.mlp\.e_score_correction_bias", ".mlp.gate.e_score_correction_bias"),
    (r"\.self_attn\.W_pack\.", ".self_attn.qkv_proj."),                                            # Baichuan: fused [q; k; v]
    # CogVLM: the language expert is the decoder proper (the visual expert is loaded by models/cogvlm.py::attach)
    (r"\.self_attn\.language_expert_query_key_value\.", ".self_attn.qkv_proj."), (r"\.self_attn\.language_expert_dense\.", ".self_attn.o_proj."),
    (r"\.mlp\.language_mlp\.", ".mlp."),
    (r"\.mlp\.gate\.wg\.", ".mlp.gate."), (r"\.mlp\.shared_mlp\.", ".mlp.shared_experts."),         # Hunyuan-MoE
    # Step-3.5 (router, selection bias, shared expert, experts stacked along dim 0) and Laguna
    (r"\.moe\.gate\.", ".mlp.gate."), (r"\.moe\.router_bias$", ".mlp.gate.e_score_correction_bias"),
    (r"\.moe\.(gate|up|down)_proj\.weight$", r".mlp.experts.stacked_\1"), (r"\.moe\.experts\.", ".mlp.experts."),
    (r"\.share_expert\.", ".mlp.shared_experts."), (r"\.mlp\.experts\.e_score_correction_bias$", ".mlp.gate.e_score_correction_bias"),
    (r"\.mlp\.router\.gate\.", ".mlp.gate."), (r"\.mlp\.expert_bias$", ".mlp.gate.e_score_correction_bias"),   # Hunyuan v3
    # TeleChat
    (r"^transformer\.word_embeddings\.", "model.embed_tokens."), (r"^transformer\.lm_head\.", "lm_head."),
    (r"\.self_attention\.query\.", ".self_attn.q_proj."), (r"\.self_attention\.key_value\.", ".self_attn.kv_proj."),
    # ChatGLM2/3 and original GLM-4 checkpoints
    (r"^transformer\.embedding\.word_embeddings\.", "model.embed_tokens."), (r"^transformer\.encoder\.layers\.", "model.layers."),
    (r"^transformer\.encoder\.final_layernorm\.", "model.norm."), (r"^transformer\.output_layer\.", "lm_head."),
    (r"\.self_attention\.query_key_value\.", ".self_attn.qkv_proj."), (r"\.self_attention\.dense\.", ".self_attn.o_proj."),
    (r"\.mlp\.dense_h_to_4h\.", ".mlp.gate_up_proj."), (r"\.mlp\.dense_4h_to_h\.", ".mlp.down_proj."),
    (r"^transformer\.h\.", "model.layers."), (r"^transformer\.wte\.", "model.embed_tokens."),
    (r"^transformer\.ln_f\.", "model.norm."), (r"^language_model\.model\.", "model."), (r"^language_model\.lm_head\.", "lm_head."),
    (r"^model\.(language_model\.)+", "model."),
    (r"\.attention\.wqkv\.", ".self_attn.qkv_proj."), (r"\.attention\.wo\.", ".self_attn.o_proj."),
    (r"\.feed_forward\.w1\.", ".mlp.gate_proj."), (r"\.feed_forward\.w3\.", ".mlp.up_proj."),
    (r"\.feed_forward\.w2\.", ".mlp.down_proj."), (r"\.attention_norm\.", ".input_layernorm."),
    (r"\.ffn_norm\.", ".post_attention_layernorm."), (r"^model\.tok_embeddings\.", "model.embed_tokens."),
    (r"^output\.", "lm_head."),
    (r"\.self_attn\.W_pack\.", ".self_attn.qkv_proj."),
    (r"\.block_sparse_moe\.gate\.", ".mlp.gate."), (r"\.block_sparse_moe\.experts\.(\d+)\.w1\.", r".mlp.experts.\1.gate_proj."),
    (r"\.block_sparse_moe\.experts\.(\d+)\.w3\.", r".mlp.experts.\1.up_proj."),
    (r"\.block_sparse_moe\.experts\.(\d+)\.w2\.", r".mlp.experts.\1.down_proj."),
    (r"\.attn\.c_attn\.", ".self_attn.qkv_proj."), (r"\.attn\.c_proj\.", ".self_attn.o_proj."),
    (r"\.attn\.qkv_proj\.", ".self_attn.qkv_proj."), (r"\.attn\.out_proj\.", ".self_attn.o_proj."),      # CodeGen / MOSS, GPT-J
    (r"\.attn\.([qkv])_proj\.", r".self_attn.\1_proj."),
    (r"\.mlp\.fc_in\.", ".mlp.up_proj."), (r"\.mlp\.fc_out\.", ".mlp.down_proj."),
    (r"\.ln_1\.", ".input_layernorm."), (r"\.ln_2\.", ".post_attention_layernorm."),
    (r"\.mlp\.w2\.", ".mlp.gate_proj."), (r"\.mlp\.w1\.", ".mlp.up_proj."), (r"\.mlp\.c_proj\.", ".mlp.down_proj."),
]


def canonical_name(name: str) -> str:
    for pat, rep in _RENAMES:
        name = re.sub(pat, rep, name)
    return name


class HFCheckpoint:
    """Index of all tensors in a folder with lazy, per-layer access and on-the-fly de-quantisation."""

    def __init__(self, path: str | Path, cfg: ModelConfig, dtype=torch.bfloat16):
        self.files, where = st.open_model_dir(path)
        self.cfg, self.dtype = cfg, dtype
        self.where = {}
        for raw, fi in where.items():
            self.where[canonical_name(raw)] = (fi, raw)
        self.names = list(self.where.keys())
        sh = Path(path) / "fastllm_shapes.json"
        self.blob_shapes = json.loads(sh.read_text()) if sh.exists() else {}

    def raw(self, name):
        fi, rawname = self.where[name]
        return self.files[fi].get(rawname)

    def has(self, name):
        return name in self.where

    def weight(self, prefix: str):
        """Dense 16-bit weight for ``prefix`` ('....q_proj'), de-quantising pre-quantised formats."""
        if self.has(prefix + ".weight"):
            fi, rawname = self.where[prefix + ".weight"]
            if self.files[fi].info(rawname)["dtype"] == "fastllm":
                from .export import decode_blob

                return decode_blob(self.files[fi].get(rawname), self.blob_shapes[rawname], self.dtype)
            w = self.raw(prefix + ".weight")
            if w.dtype == torch.float8_e4m3fn:
                sname = prefix + ".weight_scale_inv" if self.has(prefix + ".weight_scale_inv") else prefix + ".weight_scale"
                if self.has(sname):
                    sc = self.raw(sname)
                    if sc.numel() == 1:
                        return (w.float() * sc.float().item()).to(self.dtype)
                    return dequant_fp8_block(w, sc, self.dtype)
                return w.float().to(self.dtype)
            if w.dtype == torch.uint8 and self.has(prefix + ".weight_scale"):          # NVFP4 (two e2m1 values per byte)
                g2 = self.raw(prefix + ".weight_scale_2") if self.has(prefix + ".weight_scale_2") else None
                return dequant_nvfp4(w, self.raw(prefix + ".weight_scale"), g2, self.dtype)
            return w
        if self.has(prefix + ".qweight"):
            # (fp32 when the run-time format is 4-bit group-wise: the quantiser then recovers the checkpoint's own grid)
            return dequant_awq(self.raw(prefix + ".qweight"), self.raw(prefix + ".qzeros"), self.raw(prefix + ".scales"),
                               torch.float32 if getattr(self, "keep_f32_4bit", False) else self.dtype)
        return None

    def attach_lora(self, adapter_dir: str | Path) -> int:
        """Register a PEFT LoRA adapter folder (``adapter_config.json`` + ``adapter_model.safetensors``): every targeted
        weight is returned merged, ``W + (alpha / r) * B @ A``.  Returns the number of adapted matrices.
        (Reference: the ``lora`` argument of ``llm.model``, tools/fastllm_pytools/llm.py:1083.)"""
        ad = Path(adapter_dir)
        conf = json.loads((ad / "adapter_config.json").read_text())
        scale = float(conf.get("lora_alpha", conf.get("r", 1))) / float(conf.get("r", 1))
        f = st.SafeTensorFile(ad / "adapter_model.safetensors")
        self.lora = {}
        for k in f.keys():
            if ".lora_A" not in k:
                continue
            base = k.split(".lora_A")[0]
            kb = k.replace(".lora_A", ".lora_B")
            name = canonical_name(re.sub(r"^base_model\.model\.", "", base))
            self.lora[name] = (f.get(k).float().clone(), f.get(kb).float().clone(), scale)
        f.close()
        return len(self.lora)

    def _merged(self, base: str, w):
        lo = getattr(self, "lora", None)
        if not lo or base not in lo or w is None:
            return w
        a, b, scale = lo[base]
        return (w.float() + scale * (b @ a)).to(w.dtype)

    def collect(self, prefix: str) -> dict:
        """All tensors under ``prefix`` as canonical name -> dense tensor (quantised triples collapsed to .weight)."""
        out = {}
        done = set()
        for n in self.names:
            if not n.startswith(prefix):
                continue
            base, _, leaf = n.rpartition(".")
            if getattr(self, "want_spans", False) and n.endswith(".gate_proj.weight") and ".experts." in n \
                    and not getattr(self, "lora", None):
                up = n[:-len("gate_proj.weight")] + "up_proj.weight"
                if up in self.where and self.where[up][0] == self.where[n][0]:
                    fi = self.where[n][0]
                    sp = self.files[fi].span(self.where[n][1], self.where[up][1])
                    if sp is not None:          # [gate; up] of one expert as a single view of the file mapping
                        out[n[:-len("gate_proj.weight")] + "gate_up_span"] = sp
            if leaf in ("weight_scale_inv", "weight_scale", "weight_scale_2", "input_scale", "qzeros", "scales", "g_idx"):
                continue
            if leaf.endswith("_scales") and self.has(n[:-7] + "_blocks"):
                continue
            if leaf.endswith("_blocks") and self.has(n[:-7] + "_scales"):
                # MXFP4 stacked experts [E, rows, K/32, 16] -> the 16-bit checkpoint layout [E, K, rows]
                out[n[:-7]] = dequant_mxfp4(self.raw(n), self.raw(n[:-7] + "_scales"), self.dtype).transpose(-1, -2).contiguous()
                continue
            if leaf in ("weight", "qweight"):
                if base in done:
                    continue
                done.add(base)
                out[base + ".weight"] = self._merged(base, self.weight(base))
            else:
                out[n] = self.raw(n)
        return out

    def close(self):
        for f in self.files:
            f.close()


def staged_devices(m) -> bool:
    return getattr(m, "layer_devices", None) is not None


def resolve_wdtype(name: str, default: str, rules: list | None) -> str:
    """Apply ``dtype_config`` rules ``[{"key": regex, "dtype": name}, ...]``; the last matching rule wins."""
    out = default
    for r in rules or []:
        if re.search(r["key"], name):
            out = r["dtype"]
    return out


def load_model(path: str | Path, device="cuda", dtype=None, wdtype: str = "auto", moe_wdtype: str | None = None,
               tp: TPInfo | None = None, ep=None, dtype_config: list | str | None = None, moe_device: str | None = None,
               moe_device_layers: int = -1, lora: str | None = None, device_map: dict | None = None) -> DecoderModel:
    """Build a ready-to-run ``DecoderModel`` from an HF folder.

    ``moe_device="cpu"`` keeps the routed experts (of the first ``moe_device_layers`` layers, all when negative) in host
    memory and runs them on the native CPU backend -- the reference's ``--moe_device cpu`` hybrid placement.
    ``moe_device="numa"`` is the host placement with every expert cut across the memory nodes, each slice in memory its
    node's pinned threads allocated (``csrc/cpu/numa_moe.cpp``).
    ``moe_device="disk"`` is the same placement with the expert matrices left in the checkpoint's file mapping (no copy into
    anonymous memory: pages come from the SSD through the page cache as the router touches an expert), for models larger than
    RAM -- the reference's disk device (src/devices/disk/diskdevice.cpp:45-49).  It applies to 16/32-bit checkpoints whose
    dtype is the run-time dtype; anything else is read into memory as for ``"cpu"``."""
    cfg = load_config(path)
    if dtype is None:
        dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}.get(cfg.torch_dtype, torch.bfloat16)
        if str(device).startswith("cuda") and dtype == torch.float32:
            dtype = torch.bfloat16
    if wdtype in ("float16", "fp16", "half"):
        dtype = torch.float16
    if wdtype in ("bfloat16", "bf16"):
        dtype = torch.bfloat16
    if isinstance(dtype_config, str) and dtype_config:
        dtype_config = json.loads(Path(dtype_config).read_text()) if Path(dtype_config).exists() else json.loads(dtype_config)
    ck = HFCheckpoint(path, cfg, dtype if dtype != torch.float32 else torch.float32)
    if lora:
        ck.attach_lora(lora)
    if wdtype == "auto" and cfg.quantization_config:
        q = cfg.quantization_config
        method = str(q.get("quant_method", "")).lower()
        if method == "fp8":
            wdtype = "fp8"
        elif method in ("awq", "gptq", "compressed-tensors"):
            wdtype = f"int4g{q.get('group_size', 128)}"
    ck.keep_f32_4bit = str(wdtype).startswith("int4")
    if device_map:
        from .shard import split_layers_by_map

        staged = split_layers_by_map(cfg.num_layers, device_map)
        device = staged[0]
    if cfg.model_type in ("gemma4", "gemma4_text"):
        from ..models import gemma4

        if tp is not None and tp.size > 1:
            raise NotImplementedError("gemma4 runs on one rank")
        m = gemma4.build(ck, cfg, device, dtype, wdtype if wdtype != "auto" else "dense", moe_wdtype)
        ck.close()
        return m
    if cfg.model_type == "cogvlm":
        from ..models.cogvlm import CogVLMModel

        if tp is not None and tp.size > 1:
            raise NotImplementedError("cogvlm runs on one rank")
        m = CogVLMModel(cfg, device, dtype, tp, ep)
    else:
        m = DecoderModel(cfg, device, dtype, tp, ep)
    m.moe_disk = moe_device == "disk"
    ck.want_spans = m.moe_disk
    m.moe_numa = moe_device == "numa"          # host placement with every expert cut across the memory nodes
    m.moe_device, m.moe_device_layers = ("cpu" if (m.moe_disk or m.moe_numa) else moe_device), moe_device_layers
    if device_map and len(set(map(str, staged))) > 1:
        m.layer_devices = staged

    def top_fn():
        t = {}
        for k in ("model.embed_tokens.weight", "model.norm.weight", "model.norm.bias", "lm_head.weight", "lm_head.bias"):
            if ck.has(k):
                t[k] = ck.raw(k)
        return t

    def layer_fn(i):
        return ck.collect(f"model.layers.{i}.")

    # dtype_config rules are evaluated per layer-level prefix (attention / mlp / experts)
    if dtype_config:
        base_w, base_m = wdtype, moe_wdtype

        class _Rules:
            pass

        # resolved lazily inside shard.build_layer through these callables
        m.wdtype_for = lambda name: resolve_wdtype(name, base_w, dtype_config)
        m.moe_wdtype_for = lambda name: resolve_wdtype(name, base_m or base_w, dtype_config)
    finalize_model(m, top_fn, layer_fn, wdtype=wdtype, moe_wdtype=moe_wdtype)
    if cfg.mtp_layers and not staged_devices(m):
        from .shard import build_mtp

        L = cfg.num_layers
        t = ck.collect(f"model.layers.{L}.")
        if not t and any(n.startswith("mtp.") for n in ck.names):
            # Qwen3.5 naming: mtp.fc / pre_fc_norm_embedding / pre_fc_norm_hidden / norm / layers.0.*
            ren = {"mtp.fc.weight": "eh_proj.weight", "mtp.pre_fc_norm_embedding.weight": "enorm.weight",
                   "mtp.pre_fc_norm_hidden.weight": "hnorm.weight", "mtp.norm.weight": "shared_head.norm.weight"}
            for k, v in ck.collect("mtp.").items():
                k2 = ren.get(k) or (k[len("mtp.layers.0."):] if k.startswith("mtp.layers.0.") else None)
                if k2 is not None:
                    t[f"model.layers.{L}." + k2] = v
        if t.get(f"model.layers.{L}.eh_proj.weight") is not None:
            build_mtp(m, t, wdtype, moe_wdtype)
    if cfg.model_type == "cogvlm":
        from ..models import cogvlm

        cogvlm.attach(m, ck, cfg, wdtype)
    vc = cfg.raw.get("vision_config")
    vis = [n for n in ck.names if n.startswith("model.visual.") or n.startswith("visual.")]
    if isinstance(vc, dict) and vis and (tp is None or tp.rank == 0):
        # image inputs: the vision tower of the checkpoint (it runs once per image, in the activation dtype, on the scheduling
        # rank; the other ranks receive the image tokens' embeddings)
        from ..models.vision import VisionConfig, VisionTower

        w = {n.split("visual.", 1)[1]: ck.raw(n) for n in vis}
        m.vision = VisionTower(VisionConfig(vc), w, m.device, dtype)
        m.image_token_id = cfg.raw.get("image_token_id")
        m.video_token_id = cfg.raw.get("video_token_id")
    ck.close()
    return m
