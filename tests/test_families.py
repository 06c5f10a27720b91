"""Model-family parity: for every supported architecture a tiny random model is instantiated with Hugging Face
transformers, saved as a checkpoint folder, loaded by this framework's HF loader and compared on last-token logits
(the reference checks whole models the same way against transformers, test/basic/forward_check.py, logits_test.py)."""
import pytest
import torch

from fastllm_b200.engine import EngineConfig, LLMEngine
from fastllm_b200.loader import hf
from fastllm_b200.models.decoder import ForwardBatch

transformers = pytest.importorskip("transformers")

_C = dict(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=512,
          max_position_embeddings=512, head_dim=64)
_NH = {k: v for k, v in _C.items() if k != "head_dim"}
_MLA = dict(vocab_size=512, hidden_size=256, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, intermediate_size=512,
            moe_intermediate_size=128, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, first_k_dense_replace=1,
            kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, max_position_embeddings=512)

FAMILIES = {
    "mistral": dict(model_type="mistral", **_C, sliding_window=None),
    "mistral-sliding-window": dict(model_type="mistral", **_C, sliding_window=16),
    "qwen2": dict(model_type="qwen2", **_NH),
    "phi3": dict(model_type="phi3", **_NH, pad_token_id=0),
    "glm": dict(model_type="glm", **_C, partial_rotary_factor=0.5, pad_token_id=0),
    "glm4": dict(model_type="glm4", **_C, partial_rotary_factor=0.5, pad_token_id=0),
    "gemma": dict(model_type="gemma", **_C),
    "gemma2": dict(model_type="gemma2", **_C, sliding_window=16, query_pre_attn_scalar=64),
    "mixtral": dict(model_type="mixtral", **_NH, num_local_experts=4, num_experts_per_tok=2),
    "qwen2_moe": dict(model_type="qwen2_moe", **_NH, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                      shared_expert_intermediate_size=256, decoder_sparse_step=1, norm_topk_prob=False),
    "qwen3_moe": dict(model_type="qwen3_moe", **_C, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                      decoder_sparse_step=1, norm_topk_prob=True),
    "deepseek_v2": dict(model_type="deepseek_v2", **_MLA, n_group=1, topk_group=1, q_lora_rank=None),
    "deepseek_v3": dict(model_type="deepseek_v3", **_MLA, n_group=2, topk_group=1, routed_scaling_factor=2.5, norm_topk_prob=True,
                        q_lora_rank=128),
    "glm_moe_dsa": dict(model_type="glm_moe_dsa", **_MLA, n_group=1, topk_group=1, q_lora_rank=128,
                        mlp_layer_types=["dense", "sparse", "sparse"]),
    "glm4_moe": dict(model_type="glm4_moe", **_C, moe_intermediate_size=128, n_routed_experts=8, num_experts_per_tok=2,
                     n_shared_experts=1, first_k_dense_replace=1, n_group=1, topk_group=1, partial_rotary_factor=0.5, use_qk_norm=True),
    "ernie4_5": dict(model_type="ernie4_5", **_C),
    "ernie4_5_moe": dict(model_type="ernie4_5_moe", **_C, moe_intermediate_size=128, moe_num_experts=8, moe_k=2, moe_num_shared_experts=1,
                         moe_layer_start_index=1, moe_layer_interval=1),
    "hunyuan_v1_moe": dict(model_type="hunyuan_v1_moe", **_C, num_experts=4, moe_topk=2, num_shared_expert=1, moe_intermediate_size=128),
    "hunyuan_v1_dense": dict(model_type="hunyuan_v1_dense", **_C),
    "gpt_oss": dict(model_type="gpt_oss", **_C, num_local_experts=4, num_experts_per_tok=2, sliding_window=16),
    "gemma3_text": dict(model_type="gemma3_text", **_C, sliding_window=16, query_pre_attn_scalar=64,
                        layer_types=["sliding_attention", "full_attention"]),
    "minimax_m2": dict(model_type="minimax_m2", **_C, num_local_experts=4, num_experts_per_tok=2,
                       rope_parameters={"rope_type": "default", "rope_theta": 1e6, "partial_rotary_factor": 0.5}),
    "minimax": dict(model_type="minimax", **_C, num_local_experts=4, num_experts_per_tok=2, block_size=16,
                    layer_types=["linear_attention", "full_attention"], full_attn_alpha_factor=1.5, full_attn_beta_factor=0.8,
                    linear_attn_alpha_factor=1.25, linear_attn_beta_factor=0.9, mlp_alpha_factor=1.1, mlp_beta_factor=0.7),
    "qwen3_next": dict(model_type="qwen3_next", **_C, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                       shared_expert_intermediate_size=256, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
                       linear_value_head_dim=32, layer_types=["linear_attention", "full_attention"]),
    "qwen3_5_text": dict(model_type="qwen3_5_text", **_C, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
                         linear_value_head_dim=32, layer_types=["linear_attention", "full_attention"]),
    "qwen3_5_moe_text": dict(model_type="qwen3_5_moe_text", **_C, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                             shared_expert_intermediate_size=256, linear_num_key_heads=2, linear_num_value_heads=4,
                             linear_key_head_dim=32, linear_value_head_dim=32, layer_types=["linear_attention", "full_attention"]),
    "granite": dict(model_type="granite", **_NH, attention_multiplier=0.2, embedding_multiplier=3.0, residual_multiplier=0.5,
                    logits_scaling=2.0),
}


@pytest.mark.parametrize("name", sorted(FAMILIES))
def test_family_matches_transformers(name, tmp_path):
    torch.manual_seed(0)
    try:
        cfg = transformers.AutoConfig.for_model(**FAMILIES[name])
        # glm_moe_dsa: with the fused attention back end the oracle hands over the indexer mask alone (every position is
        # selected at this length) and loses the causal mask; the eager back end combines the two
        extra = {"attn_implementation": "eager"} if name == "glm_moe_dsa" else {}
        ref = transformers.AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.float32, **extra)
    except Exception as e:      # architecture not present in the installed transformers
        pytest.skip(f"transformers cannot build {name}: {e}")
    for p in ref.parameters():
        if p.dim() >= 2:
            torch.nn.init.normal_(p, std=0.05)
        elif "sinks" in str(p.shape) or p.dim() == 1:
            pass
    ref.eval()
    d = str(tmp_path / name)
    ref.save_pretrained(d, safe_serialization=True)
    prompt = list(range(5, 90, 3))
    T = len(prompt)
    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512), num_pages=8)
    fb = ForwardBatch(ids=torch.tensor(prompt, dtype=torch.int32), positions=torch.arange(T, dtype=torch.int32),
                      slots=torch.arange(T, dtype=torch.int32), page_table=torch.tensor([[0, 1, 2, 3]], dtype=torch.int32),
                      kv_lens=torch.tensor([T], dtype=torch.int32), cu_q=torch.tensor([0, T], dtype=torch.int32),
                      logit_rows=torch.tensor([T - 1]), cu_q_host=[0, T],
                      state_slots=torch.tensor([0], dtype=torch.int32), state_slots_host=[0])
    got = m.forward(fb, eng.runner.kv.pools)[0].float()[:want.numel()]
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    assert (got - want).abs().max().item() < 2e-3
    assert int(got.argmax()) == int(want.argmax())


def _save_renamed(ref, cfg_dict, rename, d, merge=None):
    """Write ``ref``'s weights under another family's tensor names / layout with that family's config.json."""
    import json
    import os

    from fastllm_b200.loader.safetensors import save_file

    os.makedirs(d, exist_ok=True)
    sd = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    if merge is not None:
        sd = merge(sd)
    out = {rename(k): v.contiguous() for k, v in sd.items()}
    save_file(out, os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg_dict, f)


def _last_logits(m, prompt):
    T = len(prompt)
    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512), num_pages=8)
    fb = ForwardBatch(ids=torch.tensor(prompt, dtype=torch.int32), positions=torch.arange(T, dtype=torch.int32),
                      slots=torch.arange(T, dtype=torch.int32), page_table=torch.tensor([[0, 1, 2, 3]], dtype=torch.int32),
                      kv_lens=torch.tensor([T], dtype=torch.int32), cu_q=torch.tensor([0, T], dtype=torch.int32),
                      logit_rows=torch.tensor([T - 1]), cu_q_host=[0, T])
    return m.forward(fb, eng.runner.kv.pools)[0].float()


def _tiny(model_type, **extra):
    torch.manual_seed(0)
    cfg = transformers.AutoConfig.for_model(model_type=model_type, **extra)
    ref = transformers.AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.float32)
    for p in ref.parameters():
        if p.dim() >= 2:
            torch.nn.init.normal_(p, std=0.05)
    return ref.eval()


def test_chatglm_layout(tmp_path):
    """ChatGLM2/3 / original GLM-4 checkpoints: own tensor names, packed QKV and [gate | up], own config keys."""
    ref = _tiny("glm", **_C, partial_rotary_factor=0.5, pad_token_id=0)
    prompt = list(range(7, 70, 2))
    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()

    def merge(sd):
        out = {}
        for k, v in sd.items():
            if ".q_proj." in k:
                kk, vv = k.replace(".q_proj.", ".k_proj."), k.replace(".q_proj.", ".v_proj.")
                out[k.replace(".self_attn.q_proj.", ".self_attention.query_key_value.")] = torch.cat([v, sd[kk], sd[vv]], dim=0)
            elif ".k_proj." in k or ".v_proj." in k:
                continue
            else:
                out[k] = v
        return out

    def rename(k):
        k = k.replace("model.embed_tokens.", "transformer.embedding.word_embeddings.").replace("model.layers.", "transformer.encoder.layers.")
        k = k.replace("model.norm.", "transformer.encoder.final_layernorm.").replace("lm_head.", "transformer.output_layer.")
        return k.replace(".self_attn.o_proj.", ".self_attention.dense.").replace(".mlp.gate_up_proj.", ".mlp.dense_h_to_4h.").replace(
            ".mlp.down_proj.", ".mlp.dense_4h_to_h.")

    cfgd = dict(model_type="chatglm", padded_vocab_size=512, hidden_size=256, num_layers=2, num_attention_heads=4, multi_query_attention=True,
                multi_query_group_num=2, kv_channels=64, ffn_hidden_size=512, layernorm_epsilon=ref.config.rms_norm_eps, add_qkv_bias=True,
                seq_length=512, rope_ratio=1.0, eos_token_id=2)
    d = str(tmp_path / "chatglm")
    _save_renamed(ref, cfgd, rename, d, merge)
    got = _last_logits(hf.load_model(d, device="cpu", dtype=torch.float32), prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999


def test_internlm2_and_minicpm_layouts(tmp_path):
    """InternLM2 (grouped wqkv, w1/w3/w2 names) and MiniCPM (embedding / residual / logit scaling) from a llama oracle."""
    ref = _tiny("llama", **_C)
    prompt = list(range(9, 80, 2))
    c = ref.config
    G = c.num_attention_heads // c.num_key_value_heads

    def merge(sd):
        out = {}
        for k, v in sd.items():
            if ".q_proj." in k:
                q = v.reshape(c.num_key_value_heads, G, 64, -1)
                kk = sd[k.replace(".q_proj.", ".k_proj.")].reshape(c.num_key_value_heads, 1, 64, -1)
                vv = sd[k.replace(".q_proj.", ".v_proj.")].reshape(c.num_key_value_heads, 1, 64, -1)
                out[k.replace(".self_attn.q_proj.", ".attention.wqkv.")] = torch.cat([q, kk, vv], dim=1).reshape(-1, v.shape[-1])
            elif ".k_proj." in k or ".v_proj." in k:
                continue
            else:
                out[k] = v
        return out

    def rename(k):
        k = k.replace("model.embed_tokens.", "model.tok_embeddings.").replace("lm_head.", "output.")
        k = k.replace(".self_attn.o_proj.", ".attention.wo.").replace(".mlp.gate_proj.", ".feed_forward.w1.").replace(".mlp.up_proj.", ".feed_forward.w3.")
        return k.replace(".mlp.down_proj.", ".feed_forward.w2.").replace(".input_layernorm.", ".attention_norm.").replace(".post_attention_layernorm.", ".ffn_norm.")

    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()
    cfgd = dict(c.to_dict(), model_type="internlm2")
    d = str(tmp_path / "internlm2")
    _save_renamed(ref, cfgd, rename, d, merge)
    got = _last_logits(hf.load_model(d, device="cpu", dtype=torch.float32), prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999

    # MiniCPM = llama with scale_emb, scale_depth / sqrt(layers) on every sub-layer output, logits / (hidden / dim_model_base):
    # the same numbers come out of a Granite oracle with the equivalent multipliers.
    ref2 = _tiny("granite", **_NH, attention_multiplier=(256 // 4) ** -0.5, embedding_multiplier=12.0, residual_multiplier=1.4 / (2 ** 0.5),
                 logits_scaling=256 / 64)
    with torch.no_grad():
        want2 = ref2(torch.tensor([prompt])).logits[0, -1].float()
    cfgd2 = dict(ref2.config.to_dict(), model_type="minicpm", scale_emb=12.0, scale_depth=1.4, dim_model_base=64)
    d2 = str(tmp_path / "minicpm")
    _save_renamed(ref2, cfgd2, lambda k: k, d2)
    got2 = _last_logits(hf.load_model(d2, device="cpu", dtype=torch.float32), prompt)
    assert torch.nn.functional.cosine_similarity(got2, want2, dim=0).item() > 0.99999


def test_qwen_v1_layout(tmp_path):
    """Qwen (v1): transformer.h.N.attn.c_attn / c_proj, mlp.w1 (up) / w2 (gate) / c_proj, ln_1 / ln_2, QKV bias."""
    ref = _tiny("qwen2", **{**_NH, "num_key_value_heads": 4})
    prompt = list(range(11, 90, 3))
    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()

    def merge(sd):
        out = {}
        for k, v in sd.items():
            if ".q_proj." in k:
                out[k.replace(".self_attn.q_proj.", ".attn.c_attn.")] = torch.cat([v, sd[k.replace(".q_proj.", ".k_proj.")], sd[k.replace(".q_proj.", ".v_proj.")]], dim=0)
            elif ".k_proj." in k or ".v_proj." in k:
                continue
            else:
                out[k] = v
        return out

    def rename(k):
        k = k.replace("model.embed_tokens.", "transformer.wte.").replace("model.layers.", "transformer.h.").replace("model.norm.", "transformer.ln_f.")
        k = k.replace(".self_attn.o_proj.", ".attn.c_proj.").replace(".mlp.gate_proj.", ".mlp.w2.").replace(".mlp.up_proj.", ".mlp.w1.")
        return k.replace(".mlp.down_proj.", ".mlp.c_proj.").replace(".input_layernorm.", ".ln_1.").replace(".post_attention_layernorm.", ".ln_2.")

    cfgd = dict(model_type="qwen", vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, kv_channels=64,
                intermediate_size=1024, layer_norm_epsilon=ref.config.rms_norm_eps, seq_length=512, rotary_emb_base=ref.config.rope_parameters["rope_theta"])
    d = str(tmp_path / "qwen")
    _save_renamed(ref, cfgd, rename, d, merge)
    got = _last_logits(hf.load_model(d, device="cpu", dtype=torch.float32), prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999


def _to_fp4(x):
    """Nearest e2m1 code (0..15) of every element of ``x`` (already divided by its block scale)."""
    lut = torch.tensor(hf._FP4_VALUES)
    return (x[..., None] - lut).abs().argmin(-1).to(torch.uint8)


def test_gpt_oss_mxfp4_checkpoint(tmp_path):
    """gpt-oss as published: experts stored as MXFP4 ``*_blocks`` / ``*_scales``.  The loader must give the same logits as the
    16-bit checkpoint that holds the de-quantised values."""
    import json
    import os

    from fastllm_b200.loader.safetensors import save_file

    ref = _tiny("gpt_oss", **_C, num_local_experts=4, num_experts_per_tok=2, sliding_window=16)
    sd = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    packed, dense = {}, {}
    for k, v in sd.items():
        if k.endswith("mlp.experts.gate_up_proj") or k.endswith("mlp.experts.down_proj"):
            w = v.transpose(1, 2).contiguous()                                 # [E, rows, K]
            E, R, K = w.shape
            wb = w.reshape(E, R, K // 32, 32)
            e = torch.ceil(torch.log2(wb.abs().amax(-1).clamp(min=1e-20) / 6.0)).clamp(-127, 127)
            codes = _to_fp4(wb / torch.exp2(e)[..., None])                     # [E, R, K/32, 32]
            packed[k + "_blocks"] = (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()
            packed[k + "_scales"] = (e + 127).to(torch.uint8).contiguous()
            deq = (torch.tensor(hf._FP4_VALUES)[codes.long()] * torch.exp2(e)[..., None]).reshape(E, R, K)
            dense[k] = deq.transpose(1, 2).contiguous()
            assert torch.equal(hf.dequant_mxfp4(packed[k + "_blocks"], packed[k + "_scales"], torch.float32), deq)
        else:
            packed[k] = v.contiguous()
            dense[k] = v.contiguous()
    logits = []
    for name, tensors in (("mx", packed), ("dense", dense)):
        d = str(tmp_path / name)
        os.makedirs(d)
        save_file(tensors, os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(ref.config.to_dict(), f)
        logits.append(_last_logits(hf.load_model(d, device="cpu", dtype=torch.float32), list(range(5, 60, 3))))
    assert torch.allclose(logits[0], logits[1], atol=1e-5)


def test_nvfp4_checkpoint(tmp_path):
    """NVFP4 linear weights (uint8 pairs + e4m3 block-16 scales + fp32 global scale) load as their de-quantised values."""
    import json
    import os

    from fastllm_b200.loader.safetensors import save_file

    ref = _tiny("llama", **_C)
    sd = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    packed, dense = {}, {}
    for k, v in sd.items():
        if k.endswith("_proj.weight"):
            N, K = v.shape
            g = v.abs().max() / (6.0 * 448.0)
            wb = v.reshape(N, K // 16, 16)
            bs = (wb.abs().amax(-1) / 6.0 / g).to(torch.float8_e4m3fn)
            codes = _to_fp4(wb / (bs.float() * g).clamp(min=1e-20)[..., None]).reshape(N, K)
            base = k[:-len(".weight")]
            packed[k] = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
            packed[base + ".weight_scale"] = bs.contiguous()
            packed[base + ".weight_scale_2"] = g.reshape(1).float()
            packed[base + ".input_scale"] = torch.ones(1)
            dense[k] = (torch.tensor(hf._FP4_VALUES)[codes.long()].reshape(N, K // 16, 16) * (bs.float() * g)[..., None]).reshape(N, K)
        else:
            packed[k] = v.contiguous()
            dense[k] = v.contiguous()
    logits = []
    for name, tensors in (("nv", packed), ("dense", dense)):
        d = str(tmp_path / name)
        os.makedirs(d)
        save_file(tensors, os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(ref.config.to_dict(), f)
        logits.append(_last_logits(hf.load_model(d, device="cpu", dtype=torch.float32), list(range(5, 60, 3))))
    assert torch.allclose(logits[0], logits[1], atol=1e-4)


def test_baichuan_and_internlm3_layouts(tmp_path):
    """Baichuan (rotary variants: ``W_pack`` = [q; k; v]) and InternLM3 (Llama names, ``qkv_bias`` / ``bias`` flags) from oracles."""
    ref = _tiny("llama", **{**_NH, "num_key_value_heads": 4})
    prompt = list(range(7, 70, 2))

    def merge(sd):
        out = {}
        for k, v in sd.items():
            if ".q_proj." in k:
                out[k.replace(".q_proj.", ".W_pack.")] = torch.cat([v, sd[k.replace(".q_proj.", ".k_proj.")], sd[k.replace(".q_proj.", ".v_proj.")]], dim=0)
            elif ".k_proj." not in k and ".v_proj." not in k:
                out[k] = v
        return out

    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()
    d = str(tmp_path / "baichuan")
    _save_renamed(ref, dict(ref.config.to_dict(), model_type="baichuan"), lambda k: k, d, merge)
    got = _last_logits(hf.load_model(d, device="cpu", dtype=torch.float32), prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999

    ref3 = _tiny("qwen2", **_NH)                                   # q/k/v bias, no o / mlp bias = InternLM3 with qkv_bias
    for n_, p_ in ref3.named_parameters():
        if n_.endswith("_proj.bias"):
            torch.nn.init.normal_(p_, std=0.1)
    with torch.no_grad():
        want3 = ref3(torch.tensor([prompt])).logits[0, -1].float()
    d3 = str(tmp_path / "internlm3")
    cfg3 = {k: v for k, v in ref3.config.to_dict().items() if k not in ("use_sliding_window", "sliding_window", "layer_types", "max_window_layers")}
    _save_renamed(ref3, dict(cfg3, model_type="internlm3", qkv_bias=True, bias=False), lambda k: k, d3)
    got3 = _last_logits(hf.load_model(d3, device="cpu", dtype=torch.float32), prompt)
    assert torch.nn.functional.cosine_similarity(got3, want3, dim=0).item() > 0.99999
    # InternLM (v1): the same tensors under model_type "internlm" with its single "bias" flag
    d1 = str(tmp_path / "internlm")
    _save_renamed(ref3, dict(cfg3, model_type="internlm", bias=True), lambda k: k, d1)
    got1 = _last_logits(hf.load_model(d1, device="cpu", dtype=torch.float32), prompt)
    assert torch.nn.functional.cosine_similarity(got1, want3, dim=0).item() > 0.99999


def test_minicpm3_and_hy_v3_layouts(tmp_path):
    """MiniCPM3 (latent attention with rotate-half rotary, dense MLPs, MiniCPM multipliers) from a DeepSeek-V3 oracle whose
    weights are pre-divided by the multipliers; Hunyuan v3 (router.gate / expert_bias / shared_mlp names, sigmoid router) from a
    GLM-4-MoE oracle."""
    prompt = list(range(7, 90, 3))
    try:
        ref = _tiny("deepseek_v3", **dict(_MLA, num_hidden_layers=2, first_k_dense_replace=2), n_group=1, topk_group=1, q_lora_rank=128,
                    rope_interleave=False)
    except Exception as e:
        pytest.skip(f"transformers cannot build the oracle: {e}")
    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()
    scale_emb, scale_depth, base = 12.0, 1.4, 64
    rs = scale_depth / (2 ** 0.5)

    def merge(sd):
        out = {}
        for k, v in sd.items():
            if k.endswith("embed_tokens.weight"):
                v = v / scale_emb
            elif k.endswith("self_attn.o_proj.weight") or k.endswith("mlp.down_proj.weight"):
                v = v / rs
            elif k == "lm_head.weight":
                v = v * (256 / base)
            out[k] = v
        return out

    cfgd = dict(ref.config.to_dict(), model_type="minicpm3", scale_emb=scale_emb, scale_depth=scale_depth, dim_model_base=base,
                tie_word_embeddings=False)
    for k in ("n_routed_experts", "num_experts_per_tok", "n_shared_experts", "first_k_dense_replace", "moe_intermediate_size"):
        cfgd.pop(k, None)
    d = str(tmp_path / "minicpm3")
    _save_renamed(ref, cfgd, lambda k: k, d, merge)
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    assert m.cfg.use_mla and not m.cfg.is_moe and m.cfg.rope_mode == "neox"
    got = _last_logits(m, prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    assert (got - want).abs().max().item() < 2e-3

    ref2 = _tiny("glm4_moe", **_C, moe_intermediate_size=128, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1,
                 first_k_dense_replace=1, n_group=1, topk_group=1, partial_rotary_factor=1.0, use_qk_norm=True,
                 routed_scaling_factor=2.0, norm_topk_prob=True)
    with torch.no_grad():
        for n_, p_ in ref2.named_parameters():
            if n_.endswith("e_score_correction_bias"):
                p_.copy_(torch.randn_like(p_) * 0.1)
        want2 = ref2(torch.tensor([prompt])).logits[0, -1].float()

    def rename(k):
        return (k.replace(".mlp.gate.weight", ".mlp.router.gate.weight").replace(".mlp.gate.e_score_correction_bias", ".mlp.expert_bias")
                .replace(".mlp.shared_experts.", ".mlp.shared_mlp."))

    c2 = ref2.config
    cfgd2 = dict(model_type="hy_v3", architectures=["HYV3ForCausalLM"], vocab_size=c2.vocab_size, hidden_size=c2.hidden_size,
                 num_hidden_layers=c2.num_hidden_layers, num_attention_heads=c2.num_attention_heads,
                 num_key_value_heads=c2.num_key_value_heads, head_dim=64, intermediate_size=c2.intermediate_size,
                 moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2, num_shared_experts=1, first_k_dense_replace=1,
                 moe_router_use_sigmoid=True, route_norm=True, router_scaling_factor=2.0, rms_norm_eps=c2.rms_norm_eps,
                 rope_theta=ref2.config.to_dict().get("rope_theta", (c2.to_dict().get("rope_parameters") or {}).get("rope_theta", 10000.0)),
                 max_position_embeddings=c2.max_position_embeddings, tie_word_embeddings=False, attention_bias=bool(c2.attention_bias))
    def unstack(sd):                      # the oracle keeps its experts stacked: [E, 2I, H] (gate rows, then up rows) and [E, H, I]
        out = {}
        for k, v in sd.items():
            if k.endswith(".mlp.experts.gate_up_proj"):
                for e in range(v.shape[0]):
                    gw, uw = v[e].chunk(2, dim=0)
                    out[k.replace("gate_up_proj", f"{e}.gate_proj.weight")] = gw
                    out[k.replace("gate_up_proj", f"{e}.up_proj.weight")] = uw
            elif k.endswith(".mlp.experts.down_proj"):
                for e in range(v.shape[0]):
                    out[k.replace("down_proj", f"{e}.down_proj.weight")] = v[e]
            else:
                out[k] = v
        return out

    d2 = str(tmp_path / "hy_v3")
    _save_renamed(ref2, cfgd2, rename, d2, unstack)
    m2 = hf.load_model(d2, device="cpu", dtype=torch.float32)
    assert m2.cfg.scoring_func == "sigmoid" and m2.cfg.num_shared_experts == 1
    got2 = _last_logits(m2, prompt)
    assert torch.nn.functional.cosine_similarity(got2, want2, dim=0).item() > 0.99999
    assert int(got2.argmax()) == int(want2.argmax())


def test_pangu_grouped_routing():
    """Mixture of grouped experts: one expert per group, softmax score times the expert's scale (loop form of
    src/models/pangu_moe.cpp:392-430), and a tiny Pangu Pro MoE model generating through the engine."""
    from fastllm_b200.models import preset, random_init
    from fastllm_b200.ops import moe as MOE

    torch.manual_seed(3)
    M, E, k = 6, 12, 4
    logits = torch.randn(M, E)
    scale = torch.rand(E) + 0.5
    idx, w = MOE.route_group_top1(logits, k, scale)
    sc = torch.softmax(logits, -1)
    per = E // k
    for r in range(M):
        for gi in range(k):
            best = max(range(gi * per, (gi + 1) * per), key=lambda j: sc[r, j].item())
            assert int(idx[r, gi]) == best
            assert abs(float(w[r, gi]) - float(sc[r, best] * scale[best])) < 1e-6
    cfg = preset("tiny-pangu-moe")
    assert cfg.route_group_top1 and cfg.attention_bias and cfg.num_shared_experts == 1
    m = random_init(cfg, "cpu", torch.float32, seed=1)
    got = _last_logits(m, list(range(3, 50)))
    assert torch.isfinite(got).all() and got.shape[0] == cfg.vocab_size


def test_moss_codegen_layout(tmp_path):
    """MOSS-moon / CodeGen: LayerNorm with bias, attention and GELU MLP in parallel from one norm, pairwise rotary on the first
    rotary_dim dims, the four-block [query | value | key] projection layout, biased head -- against transformers' CodeGen."""
    try:
        ref = _tiny("codegen", vocab_size=512, n_embd=256, n_layer=2, n_head=4, rotary_dim=32, n_positions=512, n_ctx=512,
                    tie_word_embeddings=False)
    except Exception as e:
        pytest.skip(f"transformers cannot build the oracle: {e}")
    with torch.no_grad():
        for n_, p_ in ref.named_parameters():
            if n_.endswith(".bias"):
                p_.copy_(torch.randn_like(p_) * 0.05)
    prompt = list(range(11, 95, 3))
    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()
    cfgd = dict(ref.config.to_dict(), model_type="moss")
    d = str(tmp_path / "moss")
    keep = lambda sd: {k: v for k, v in sd.items() if "causal_mask" not in k and "embed_positions" not in k and not k.endswith(".attn.bias")}
    _save_renamed(ref, cfgd, lambda k: k, d, keep)
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    assert m.cfg.parallel_block and m.cfg.norm_kind == "layernorm" and not m.cfg.mlp_gated and m.cfg.rotary_dim == 32
    got = _last_logits(m, prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    assert (got - want).abs().max().item() < 2e-3


def _step3p5_reference(sd, cfg, ids):
    """Plain full-sequence evaluation of the Step-3.5 text decoder from a state dict in the checkpoint's own naming
    (reference semantics: src/models/step3p5.cpp:6320-6670)."""
    import math

    F = torch.nn.functional
    D, L, eps = cfg["head_dim"], cfg["num_hidden_layers"], cfg["rms_norm_eps"]
    kv = cfg["num_attention_groups"]
    lt = cfg["layer_types"]
    T = len(ids)
    rms = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * (w + 1.0)
    pos = torch.arange(T, dtype=torch.float32)

    def rope(t, theta, rot):
        inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
        ang = pos[:, None] * inv[None, :]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b, rest = t[..., :rot // 2], t[..., rot // 2:rot], t[..., rot:]
        return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)

    def glu(g, u, lim):
        a = F.silu(g)
        if lim:
            a, u = a.clamp(max=lim), u.clamp(min=-lim, max=lim)
        return a * u

    x = sd["model.embed_tokens.weight"][ids]
    for i in range(L):
        p = f"model.layers.{i}."
        full = lt[i] == "full_attention"
        nh = cfg["num_attention_heads"] if full else cfg["attention_other_setting"]["num_attention_heads"]
        h = rms(x, sd[p + "input_layernorm.weight"])
        q = (h @ sd[p + "self_attn.q_proj.weight"].t()).view(T, nh, D)
        k = (h @ sd[p + "self_attn.k_proj.weight"].t()).view(T, kv, D)
        v = (h @ sd[p + "self_attn.v_proj.weight"].t()).view(T, kv, D)
        q, k = rms(q, sd[p + "self_attn.q_norm.weight"]), rms(k, sd[p + "self_attn.k_norm.weight"])
        rot = int(D * cfg["partial_rotary_factors"][i])
        q, k = rope(q, cfg["rope_theta"][i], rot), rope(k, cfg["rope_theta"][i], rot)
        k, v = k.repeat_interleave(nh // kv, dim=1), v.repeat_interleave(nh // kv, dim=1)
        sc = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        qi, ki = torch.arange(T)[:, None], torch.arange(T)[None, :]
        mask = ki > qi
        if not full:
            mask = mask | (ki <= qi - cfg["sliding_window"])
        a = torch.einsum("hqk,khd->qhd", torch.softmax(sc.masked_fill(mask[None], float("-inf")), -1), v)
        a = a * torch.sigmoid(h @ sd[p + "self_attn.g_proj.weight"].t())[:, :, None]
        x = x + a.reshape(T, nh * D) @ sd[p + "self_attn.o_proj.weight"].t()
        h = rms(x, sd[p + "post_attention_layernorm.weight"])
        ls, le = cfg["swiglu_limits_shared"][i], cfg["swiglu_limits"][i]
        if i in cfg["moe_layers"]:
            y = glu(h @ sd[p + "share_expert.gate_proj.weight"].t(), h @ sd[p + "share_expert.up_proj.weight"].t(), ls) \
                @ sd[p + "share_expert.down_proj.weight"].t()
            pr = torch.sigmoid(h @ sd[p + "moe.gate.weight"].t())
            idx = (pr + sd[p + "moe.router_bias"]).topk(cfg["moe_top_k"], dim=-1)[1]
            w = pr.gather(1, idx)
            w = w / w.sum(-1, keepdim=True) * cfg["moe_router_scaling_factor"]
            for t in range(T):
                for j in range(idx.shape[1]):
                    e = int(idx[t, j])
                    he = glu(h[t] @ sd[p + "moe.gate_proj.weight"][e].t(), h[t] @ sd[p + "moe.up_proj.weight"][e].t(), le)
                    y[t] += w[t, j] * (he @ sd[p + "moe.down_proj.weight"][e].t())
            x = x + y
        else:
            x = x + glu(h @ sd[p + "mlp.gate_proj.weight"].t(), h @ sd[p + "mlp.up_proj.weight"].t(), ls) @ sd[p + "mlp.down_proj.weight"].t()
    return rms(x, sd["model.norm.weight"]) @ sd["lm_head.weight"].t()


def test_step3p5_checkpoint(tmp_path):
    """Step-3.5 text decoder from a checkpoint in its own naming (stacked experts under ``moe.``, ``share_expert.``,
    ``g_proj`` head gates, norm weights stored as deltas from one): layers with 4 / 6 query heads, their own rotary base and
    width, sliding windows, clamped SwiGLU -- against a plain full-sequence evaluation."""
    import json
    import os

    from fastllm_b200.loader.safetensors import save_file

    torch.manual_seed(5)
    H, D, L, E, I, V = 128, 32, 4, 8, 64, 256
    cfg = dict(model_type="step3p5", vocab_size=V, hidden_size=H, num_hidden_layers=L, num_attention_heads=4, num_attention_groups=2,
               head_dim=D, intermediate_size=128, moe_intermediate_size=I, moe_num_experts=E, moe_top_k=2, share_expert_dim=64,
               moe_router_scaling_factor=2.0, attention_other_setting={"num_attention_heads": 6, "num_attention_groups": 2},
               layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
               rope_theta=[1e6, 1e4, 1e4, 1e6], partial_rotary_factors=[0.5, 1.0, 1.0, 0.5], sliding_window=8,
               swiglu_limits=[0, 0, 0.05, 0.05], swiglu_limits_shared=[0, 0, 0, 0.08], moe_layers_enum="1,2,3",
               max_position_embeddings=512, rms_norm_eps=1e-5, tie_word_embeddings=False)
    r = lambda *s: torch.randn(*s) * 0.08
    sd = {"model.embed_tokens.weight": r(V, H), "model.norm.weight": r(H), "lm_head.weight": r(V, H)}
    for i in range(L):
        p = f"model.layers.{i}."
        nh = 4 if cfg["layer_types"][i] == "full_attention" else 6
        sd.update({p + "input_layernorm.weight": r(H), p + "post_attention_layernorm.weight": r(H),
                   p + "self_attn.q_proj.weight": r(nh * D, H), p + "self_attn.k_proj.weight": r(2 * D, H),
                   p + "self_attn.v_proj.weight": r(2 * D, H), p + "self_attn.o_proj.weight": r(H, nh * D),
                   p + "self_attn.q_norm.weight": r(D), p + "self_attn.k_norm.weight": r(D), p + "self_attn.g_proj.weight": r(nh, H)})
        if i == 0:
            sd.update({p + "mlp.gate_proj.weight": r(128, H), p + "mlp.up_proj.weight": r(128, H), p + "mlp.down_proj.weight": r(H, 128)})
        else:
            sd.update({p + "moe.gate.weight": r(E, H), p + "moe.router_bias": r(E), p + "moe.gate_proj.weight": r(E, I, H),
                       p + "moe.up_proj.weight": r(E, I, H), p + "moe.down_proj.weight": r(E, H, I),
                       p + "share_expert.gate_proj.weight": r(64, H), p + "share_expert.up_proj.weight": r(64, H),
                       p + "share_expert.down_proj.weight": r(H, 64)})
    d = str(tmp_path / "step3p5")
    os.makedirs(d)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    prompt = list(range(3, 75, 2))
    want = _step3p5_reference(sd, dict(cfg, moe_layers={1, 2, 3}), prompt)[-1]
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    assert m.cfg.layer_heads == [4, 6, 6, 4] and m.layers[2].mlp.experts.act == "swiglu_clamp" and m.layers[1].attn.window == 8
    got = _last_logits(m, prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    assert (got - want).abs().max().item() < 2e-3


def test_laguna_preset_runs():
    """Laguna: softplus head gates, yarn rotary over half of each head in the full-attention layers; chunked prefill plus
    decode reproduces the one-shot prefill logits."""
    from fastllm_b200.models import preset, random_init

    cfg = preset("tiny-laguna")
    assert cfg.head_gate == "softplus" and cfg.layer_rope[0]["scaling"]["rope_type"] == "yarn" and cfg.layer_rope[1]["rot_dim"] == 64
    m = random_init(cfg, "cpu", torch.float32, seed=2, std=0.05)
    prompt = list(range(4, 64))
    full = _last_logits(m, prompt)
    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512, chunked_prefill_size=16), num_pages=8)
    from fastllm_b200.engine import GenerationConfig

    toks = eng.generate([prompt], GenerationConfig(max_new_tokens=2, ignore_eos=True))[0]
    assert torch.isfinite(full).all()
    assert int(toks[0]) == int(full.argmax())


def test_telechat_layout(tmp_path):
    """TeleChat: ``transformer.h.N.self_attention.query / key_value / dense`` (keys and values interleaved per head, biases on
    the output projections), fixed NTK rotary base -- from a llama oracle with the same base."""
    D = 64
    theta = 10000.0 * 3.0 ** (D / (D - 2))
    ref = _tiny("llama", **dict(_C, num_key_value_heads=4), rope_theta=theta, attention_bias=True, mlp_bias=True)
    with torch.no_grad():
        for n_, p_ in ref.named_parameters():
            if n_.endswith(".bias"):
                p_.copy_(torch.randn_like(p_) * 0.05)
    prompt = list(range(9, 80, 2))
    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()

    def merge(sd):
        out = {}
        for k, v in sd.items():
            if ".k_proj." in k:
                vv = sd[k.replace(".k_proj.", ".v_proj.")]
                kk = v.reshape(4, 1, D, -1) if v.dim() == 2 else v.reshape(4, 1, D)
                vv = vv.reshape(4, 1, D, -1) if vv.dim() == 2 else vv.reshape(4, 1, D)
                out[k.replace(".self_attn.k_proj.", ".self_attention.key_value.")] = torch.cat([kk, vv], dim=1).reshape(-1, *v.shape[1:])
            elif ".v_proj." in k:
                continue
            else:
                out[k] = v
        return out

    def rename(k):
        k = k.replace("model.embed_tokens.", "transformer.word_embeddings.").replace("model.layers.", "transformer.h.")
        k = k.replace("model.norm.", "transformer.ln_f.").replace("lm_head.", "transformer.lm_head.")
        return k.replace(".self_attn.q_proj.", ".self_attention.query.").replace(".self_attn.o_proj.", ".self_attention.dense.")

    c = ref.config
    cfgd = dict(model_type="telechat", architectures=["TelechatForCausalLM"], vocab_size=c.vocab_size, hidden_size=c.hidden_size,
                n_layer=c.num_hidden_layers, n_head=c.num_attention_heads, ffn_hidden_size=c.intermediate_size, seq_length=512,
                layer_norm_epsilon=c.rms_norm_eps, tie_word_embeddings=False, attention_bias=True)
    d = str(tmp_path / "telechat")
    _save_renamed(ref, cfgd, rename, d, merge)
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    assert abs(m.cfg.rope_theta - theta) < 1e-3
    got = _last_logits(m, prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    assert (got - want).abs().max().item() < 2e-3


_G4 = dict(model_type="gemma4_text", vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
           num_key_value_heads=2, head_dim=32, global_head_dim=64, max_position_embeddings=512, sliding_window=16,
           layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"], final_logit_softcapping=30.0,
           vocab_size_per_layer_input=512, pad_token_id=0)


@pytest.mark.parametrize("variant", ["per_layer_inputs_shared_kv", "moe_k_eq_v"])
def test_gemma4_text_matches_transformers(variant, tmp_path):
    """Gemma-4 text: layers with their own head width and page pools, keys / values shared by the last layers, values from
    the key projection, per-layer token inputs, proportional rotary, the expert block beside the dense MLP."""
    extra = (dict(hidden_size_per_layer_input=16, num_kv_shared_layers=2, use_double_wide_mlp=True) if variant.startswith("per_layer")
             else dict(hidden_size_per_layer_input=0, attention_k_eq_v=True, num_global_key_value_heads=1, enable_moe_block=True,
                       num_experts=4, top_k_experts=2, moe_intermediate_size=64))
    torch.manual_seed(0)
    try:
        cfg = transformers.AutoConfig.for_model(**dict(_G4, **extra))
        ref = transformers.AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.float32, attn_implementation="eager")
    except Exception as e:
        pytest.skip(f"transformers cannot build gemma4_text: {e}")
    with torch.no_grad():
        for n_, p_ in ref.named_parameters():
            if p_.dim() >= 2:
                torch.nn.init.normal_(p_, std=0.05)
            else:
                p_.copy_(1.0 + torch.randn_like(p_) * 0.1)
        for n_, b_ in ref.named_buffers():
            if n_.endswith("layer_scalar"):
                b_.fill_(0.9)
    ref.eval()
    d = str(tmp_path / "g4")
    ref.save_pretrained(d, safe_serialization=True)
    prompt = list(range(5, 90, 3))
    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    got = _last_logits(m, prompt)[:want.numel()]
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    assert (got - want).abs().max().item() < 2e-3
    # chunked prefill then decode steps through the engine (shared pools, per-layer page shapes) agree with one-shot logits
    from fastllm_b200.engine import GenerationConfig

    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512, chunked_prefill_size=16), num_pages=8)
    toks = eng.generate([prompt], GenerationConfig(max_new_tokens=3, ignore_eos=True))[0]
    assert int(toks[0]) == int(want.argmax())
    with torch.no_grad():
        want2 = ref(torch.tensor([prompt + [int(toks[0])]])).logits[0, -1].float()
    assert int(toks[1]) == int(want2.argmax())


@pytest.mark.parametrize("naming", ["qwen3_5", "deepseek_v3"])
def test_mtp_weights_are_loaded(naming, tmp_path):
    """The multi-token-prediction module of a checkpoint (``mtp.*`` in the Qwen3.5 naming, ``model.layers.<L>.*`` with enorm /
    hnorm / eh_proj / shared_head in the DeepSeek-V3 naming) becomes the model's draft head; the decoder's logits are untouched."""
    ref = _tiny("llama", **_C)
    H, L = 256, 2
    prompt = list(range(9, 60, 2))
    with torch.no_grad():
        want = ref(torch.tensor([prompt])).logits[0, -1].float()
    torch.manual_seed(4)
    layer = {k.replace("model.layers.0.", ""): torch.randn_like(v) * 0.05 for k, v in ref.state_dict().items() if k.startswith("model.layers.0.")}
    fc, ne, nh, nf = torch.randn(H, 2 * H) * 0.05, torch.rand(H) + 0.5, torch.rand(H) + 0.5, torch.rand(H) + 0.5

    def merge(sd):
        out = dict(sd)
        if naming == "qwen3_5":
            out.update({"mtp.fc.weight": fc, "mtp.pre_fc_norm_embedding.weight": ne, "mtp.pre_fc_norm_hidden.weight": nh, "mtp.norm.weight": nf})
            out.update({"mtp.layers.0." + k: v for k, v in layer.items()})
        else:
            p = f"model.layers.{L}."
            out.update({p + "eh_proj.weight": fc, p + "enorm.weight": ne, p + "hnorm.weight": nh, p + "shared_head.norm.weight": nf,
                        p + "shared_head.head.weight": sd["lm_head.weight"], p + "embed_tokens.weight": sd["model.embed_tokens.weight"]})
            out.update({p + k: v for k, v in layer.items()})
        return out

    key = "mtp_num_hidden_layers" if naming == "qwen3_5" else "num_nextn_predict_layers"
    d = str(tmp_path / naming)
    _save_renamed(ref, dict(ref.config.to_dict(), **{key: 1}), lambda k: k, d, merge)
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    assert m.mtp is not None and len(m.layers) == L and m.mtp.head is None
    assert torch.equal(m.mtp.fc.w, fc) and torch.equal(m.mtp.norm_e, ne) and torch.equal(m.mtp.norm_h, nh) and torch.equal(m.mtp.final_norm, nf)
    assert torch.equal(m.mtp.layer.attn.o.w, layer["self_attn.o_proj.weight"])
    got = _last_logits(m, prompt)
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512, speculative="mtp", speculative_tokens=2), num_pages=8)
    from fastllm_b200.engine import GenerationConfig

    a = eng.generate([prompt], GenerationConfig(max_new_tokens=8, ignore_eos=True))[0]
    b = LLMEngine(m, EngineConfig(max_batch=2, max_context=512), num_pages=8).generate([prompt], GenerationConfig(max_new_tokens=8, ignore_eos=True))[0]
    assert a == b and eng.spec_proposed > 0


def test_glm_moe_dsa_sparse_attention_indexer(tmp_path):
    """GLM-MoE-DSA / DeepSeek-V3.2 sparse attention: with a selection size below the context every query attends only to its
    best-scoring keys (index keys kept in their own paged pool); one-shot prefill logits and chunked prefill + decode through
    the engine agree with transformers."""
    from fastllm_b200.engine import GenerationConfig

    torch.manual_seed(0)
    cfgd = dict(model_type="glm_moe_dsa", **_MLA, n_group=1, topk_group=1, q_lora_rank=128, mlp_layer_types=["dense", "sparse", "sparse"],
                index_topk=16, index_n_heads=4, index_head_dim=32)
    try:
        cfg = transformers.AutoConfig.for_model(**cfgd)
        ref = transformers.AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.float32, attn_implementation="eager")
    except Exception as e:
        pytest.skip(f"transformers cannot build glm_moe_dsa: {e}")
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() >= 2:
                torch.nn.init.normal_(p, std=0.05)
    ref.eval()
    d = str(tmp_path / "dsa")
    ref.save_pretrained(d, safe_serialization=True)
    prompt = list(range(5, 90, 3))                 # 29 tokens: every later query selects 16 of its keys
    with torch.no_grad():
        want = ref(torch.tensor([prompt]), use_cache=False).logits[0, -1].float()
        dense = None
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    assert getattr(m, "has_indexer", False) and m.cfg.index_topk == 16 and m.layers[0].attn.idx_wq is not None
    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512), num_pages=8)
    assert eng.runner.kv.pools[0][1] is not None and eng.runner.kv.pools[0][1].shape[-1] == 32
    got = eng.runner.prefill([(prompt, 0, [0, 1], True, 0)])[0].float()[:want.numel()]
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    assert (got - want).abs().max().item() < 2e-3
    # the selection matters: attending to every key gives different logits
    m.has_indexer, saved = False, [lw.attn.idx_wq for lw in m.layers]
    for lw in m.layers:
        lw.attn.idx_wq = None
    full = LLMEngine(m, EngineConfig(max_batch=2, max_context=512), num_pages=8).runner.prefill([(prompt, 0, [0, 1], True, 0)])[0].float()
    assert (full[:want.numel()] - want).abs().max().item() > 1e-3
    m.has_indexer = True
    for lw, w in zip(m.layers, saved):
        lw.attn.idx_wq = w
    # chunked prefill and decode steps: greedy tokens against transformers' own greedy loop (full re-evaluation per step)
    eng2 = LLMEngine(m, EngineConfig(max_batch=2, max_context=512, chunked_prefill_size=8), num_pages=8)
    toks = eng2.generate([prompt], GenerationConfig(max_new_tokens=4, ignore_eos=True))[0]
    cur = list(prompt)
    for t in toks:
        with torch.no_grad():
            nxt = int(ref(torch.tensor([cur]), use_cache=False).logits[0, -1].argmax())
        assert int(t) == nxt
        cur.append(nxt)
