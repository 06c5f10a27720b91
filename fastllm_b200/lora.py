"""Run-time LoRA adapters: load several PEFT adapter folders next to the base weights and switch between them (or back to the
base model) without reloading.

``llm.model(path, lora=dir)`` merges one adapter into the weights at load time (``loader/hf.py::attach_lora``); this module is
the other mode: the base weights stay as they are, every adapted projection keeps its low-rank pair and adds ``B (A x)`` while
the adapter is active.  Fused projections get one pair: the ``A`` matrices of q / k / v (gate / up) are stacked and ``B`` is the
matching block matrix in the fused row layout, so one extra pair of skinny GEMMs serves the fused weight.

Reference: ``set_adapter`` / ``disable_adapter`` (tools/fastllm_pytools/llm.py:2709-2713, src/models/basellm.cpp:3484-3493); the
reference applies adapters at run time in its ChatGLM model only (src/models/chatglm.cpp:176-185, LoraLayer), here every dense
(non-MLA) decoder family is covered on one tensor-parallel rank.
"""
from __future__ import annotations

import json
import re
from pathlib import Path

import torch

from .loader import safetensors as st
from .loader.hf import canonical_name
from .ops import basic as B
from .ops.quant import LinearWeight


def _read(adapter_dir) -> dict:
    ad = Path(adapter_dir)
    conf = json.loads((ad / "adapter_config.json").read_text())
    r = float(conf.get("r", 1))
    scale = float(conf.get("lora_alpha", r)) / r
    f = st.SafeTensorFile(ad / "adapter_model.safetensors")
    out = {}
    for k in f.keys():
        if ".lora_A" not in k:
            continue
        base = canonical_name(re.sub(r"^base_model\.model\.", "", k.split(".lora_A")[0]))
        out[base] = (f.get(k).float().clone(), f.get(k.replace(".lora_A", ".lora_B")).float().clone() * scale)
    f.close()
    return out


def _block(pairs, rows):
    """``pairs[i]`` = (A_i, B_i) or None for the i-th row block of ``rows[i]`` rows -> (A stacked, B block matrix) or None."""
    have = [p for p in pairs if p is not None]
    if not have:
        return None
    a = torch.cat([p[0] for p in have], dim=0)
    bs, c0 = [], 0
    for p, n in zip(pairs, rows):
        blk = torch.zeros(n, a.shape[0])
        if p is not None:
            blk[:, c0:c0 + p[0].shape[0]] = p[1]
            c0 += p[0].shape[0]
        bs.append(blk)
    return a, bs


def load_adapter(model, name: str, adapter_dir) -> int:
    """Attach the adapter in ``adapter_dir`` to ``model`` under ``name``; returns the number of adapted projections."""
    cfg = model.cfg
    if model.tp.size != 1 or cfg.use_mla:
        raise NotImplementedError("run-time adapters cover dense-attention models on one tensor-parallel rank; "
                                  "use llm.model(path, lora=adapter_dir) to merge the adapter at load")
    lo = _read(adapter_dir)
    D, rs = cfg.head_dim, float(cfg.residual_scale)
    nq, nkv = cfg.num_heads * D, cfg.num_kv_heads * D
    n = 0

    def put(w: LinearWeight | None, a, b):
        nonlocal n
        if w is None:
            return
        if w.adapters is None:
            w.adapters = {}
        w.adapters[name] = (a.to(model.device, model.dtype).contiguous(), b.to(model.device, model.dtype).contiguous())
        n += 1

    for i, lw in enumerate(model.layers):
        p = f"model.layers.{i}."
        g = lambda s: lo.get(p + s)
        if g("self_attn.qkv_proj") is not None:
            put(lw.attn.qkv, *g("self_attn.qkv_proj"))
        else:
            blk = _block([g("self_attn.q_proj"), g("self_attn.k_proj"), g("self_attn.v_proj")], [nq, nkv, nkv])
            if blk is not None:
                put(lw.attn.qkv, blk[0], torch.cat(blk[1], dim=0))
        if g("self_attn.o_proj") is not None:
            a, b = g("self_attn.o_proj")
            put(lw.attn.o, a, b * rs)
        gu = lw.mlp.gate_up
        if gu is not None:
            if g("mlp.gate_up_proj") is not None:            # stored merged [gate | up]
                a, b = g("mlp.gate_up_proj")
                bg, bu = b.chunk(2, dim=0)
                put(gu, a, B.interleave_gate_up(bg, bu) if gu.interleaved else b)
            else:
                inter = gu.n // 2
                blk = _block([g("mlp.gate_proj"), g("mlp.up_proj")], [inter, inter])
                if blk is not None:
                    put(gu, blk[0], B.interleave_gate_up(blk[1][0], blk[1][1]) if gu.interleaved else torch.cat(blk[1], dim=0))
        if g("mlp.down_proj") is not None:
            a, b = g("mlp.down_proj")
            put(lw.mlp.down, a, b * rs)
    if n == 0:
        raise ValueError(f"no tensor of the adapter in {adapter_dir} matches a projection of this model")
    return n


def set_adapter(name: str | None) -> None:
    """Activate the adapter ``name`` (None: the base model) for every model of this process."""
    LinearWeight.active_adapter = name
