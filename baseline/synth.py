"""Write a random-init Hugging Face model folder (config.json, sharded safetensors, minimal tokenizer) for one of
the benchmark architectures, so that the reference can load the same architecture through its normal loader."""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch

from fastllm_b200.loader.safetensors import save_file
from fastllm_b200.models.config import preset


def _bytes_to_unicode():
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


def write_tokenizer(path: Path, eos_id: int):
    vocab = {ch: i for i, ch in enumerate(_bytes_to_unicode().values())}
    tok = {
        "version": "1.0", "truncation": None, "padding": None,
        "added_tokens": [{"id": 256, "content": "<|endoftext|>", "single_word": False, "lstrip": False, "rstrip": False,
                          "normalized": False, "special": True}],
        "normalizer": None,
        "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": True},
        "post_processor": None,
        "decoder": {"type": "ByteLevel", "add_prefix_space": True, "trim_offsets": True, "use_regex": True},
        "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": None,
                  "end_of_word_suffix": None, "fuse_unk": False, "byte_fallback": False, "vocab": vocab, "merges": []},
    }
    (path / "tokenizer.json").write_text(json.dumps(tok))
    (path / "tokenizer_config.json").write_text(json.dumps({
        "tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<|endoftext|>", "model_max_length": 131072,
        "clean_up_tokenization_spaces": False}))


def fp8_block_quant(w: torch.Tensor, block: int = 128):
    """fp32/bf16 ``[N, K]`` -> (float8_e4m3 ``[N, K]``, fp32 ``weight_scale_inv`` ``[ceil(N/b), ceil(K/b)]``): one scale per
    128 x 128 block, ``w ~ q * scale`` (the layout of DeepSeek-V3 / Qwen3-FP8 checkpoints)."""
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, block, kb, block)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    q = (blocks / scale[:, None, :, None]).view(nb * block, kb * block)[:N, :K]
    return q.to(torch.float8_e4m3fn), scale.contiguous()


def write_model(name: str, out_dir: str, dtype=torch.bfloat16, seed: int = 0, std: float = 0.02, fp8: bool = False) -> str:
    """``fp8``: the projection matrices (attention, MLP, experts) are stored block-scaled e4m3 with ``weight_scale_inv``
    tensors and the config carries the matching ``quantization_config``; embeddings, norms, the router and the head stay 16-bit.
    Mixture-of-experts presets get ``mlp.gate`` and per-expert projections.  Tensors are drawn on the GPU when one is visible."""
    cfg = preset(name)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    if (out / "DONE").exists():
        return str(out)
    raw = dict(cfg.raw)
    if fp8:
        raw["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic", "weight_block_size": [128, 128]}
    raw.setdefault("architectures", ["LlamaForCausalLM"] if cfg.model_type == "llama" else [])
    raw["torch_dtype"] = "bfloat16" if dtype == torch.bfloat16 else "float16"
    raw["eos_token_id"] = cfg.vocab_size - 1          # a greedy run on random weights practically never emits it
    raw["bos_token_id"] = 0
    raw.setdefault("hidden_act", "silu")
    (out / "config.json").write_text(json.dumps(raw, indent=1))
    (out / "generation_config.json").write_text(json.dumps({"eos_token_id": cfg.vocab_size - 1, "do_sample": False}))
    write_tokenizer(out, cfg.vocab_size - 1)
    gdev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=gdev).manual_seed(seed)
    H, D = cfg.hidden_size, cfg.head_dim

    def rn(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32, device=gdev) * std).to(dtype).cpu()

    def proj(t: dict, key: str, *shape):
        """A projection matrix: 16-bit, or block-scaled e4m3 + its scale tensor."""
        w = torch.randn(*shape, generator=g, dtype=torch.float32, device=gdev) * std
        if fp8:
            q, sc = fp8_block_quant(w)
            t[key] = q.cpu()
            t[key + "_scale_inv"] = sc.cpu()
        else:
            t[key] = w.to(dtype).cpu()

    weight_map = {}
    shard = 0

    def flush(tensors):
        nonlocal shard
        shard += 1
        fn = f"model-{shard:05d}.safetensors"
        save_file(tensors, out / fn, metadata={"format": "pt"})
        for k in tensors:
            weight_map[k] = fn

    top = {"model.embed_tokens.weight": rn(cfg.vocab_size, H), "model.norm.weight": torch.ones(H, dtype=dtype)}
    if not cfg.tie_embeddings:
        top["lm_head.weight"] = rn(cfg.vocab_size, H)
        # the end-of-sequence row is zero: its logit is exactly 0 for every hidden state and never wins an arg-max over
        # ~10^5 random logits, so a greedy benchmark run cannot stop early
        top["lm_head.weight"][cfg.vocab_size - 1].zero_()
    flush(top)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        t = {
            p + "input_layernorm.weight": torch.ones(H, dtype=dtype),
            p + "post_attention_layernorm.weight": torch.ones(H, dtype=dtype),
        }
        proj(t, p + "self_attn.q_proj.weight", cfg.num_heads * D, H)
        proj(t, p + "self_attn.k_proj.weight", cfg.num_kv_heads * D, H)
        proj(t, p + "self_attn.v_proj.weight", cfg.num_kv_heads * D, H)
        proj(t, p + "self_attn.o_proj.weight", H, cfg.num_heads * D)
        if cfg.layer_is_moe(i):
            t[p + "mlp.gate.weight"] = rn(cfg.num_experts, H)
            I = cfg.moe_intermediate_size
            for e in range(cfg.num_experts):
                proj(t, p + f"mlp.experts.{e}.gate_proj.weight", I, H)
                proj(t, p + f"mlp.experts.{e}.up_proj.weight", I, H)
                proj(t, p + f"mlp.experts.{e}.down_proj.weight", H, I)
        else:
            proj(t, p + "mlp.gate_proj.weight", cfg.intermediate_size, H)
            proj(t, p + "mlp.up_proj.weight", cfg.intermediate_size, H)
            proj(t, p + "mlp.down_proj.weight", H, cfg.intermediate_size)
        if cfg.qk_norm:
            t[p + "self_attn.q_norm.weight"] = torch.ones(D, dtype=dtype)
            t[p + "self_attn.k_norm.weight"] = torch.ones(D, dtype=dtype)
        flush(t)
    (out / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    (out / "DONE").write_text("ok")
    return str(out)


if __name__ == "__main__":
    import sys

    print(write_model(sys.argv[1], sys.argv[2]))
