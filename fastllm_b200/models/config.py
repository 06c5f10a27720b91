"""Typed model configuration parsed from a Hugging Face ``config.json``.

The reference flattens ``config.json`` into a string dictionary and queries it by key at use sites
(src/model.cpp:2450+, e.g. ``rope_scaling.type`` in src/models/llama.cpp:82); here every field the
decoder needs is resolved once into a dataclass, per model family.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path


@dataclass
class ModelConfig:
    model_type: str = "llama"
    architectures: list = field(default_factory=list)
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    intermediate_size: int = 11008
    rms_eps: float = 1e-6
    norm_unit_offset: float = 0.0          # Gemma-style (1 + w)
    rope_theta: float = 10000.0
    rope_scaling: dict | None = None
    rope_mode: str = "neox"                # neox | interleaved | none
    rotary_dim: int | None = None          # partial rotary
    max_position: int = 8192
    tie_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    qk_norm: bool = False
    hidden_act: str = "silu"
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    sliding_window: int | None = None
    layer_windows: list | None = None      # per-layer sliding window (0 = full attention) for alternating patterns
    attn_softcap: float = 0.0              # tanh soft-capping of attention logits (Gemma-2)
    final_softcap: float = 0.0             # tanh soft-capping of the output logits
    attn_scale_override: float | None = None   # softmax scale when it is not 1/sqrt(head_dim)
    residual_scale: float = 1.0            # multiplier of every sub-layer output before the residual add (folded into weights)
    post_norms: bool = False               # sandwich norms: the sub-layer output is normalised before the residual add
    latent_norm_eps: float = 0.0           # MLA q_a / kv_a norms when they do not follow rms_norm_eps (GLM-MoE-DSA: 1e-6)
    rope_local_theta: float = 0.0          # Gemma-3: sliding-window layers rotate with this base (and no scaling)
    qk_norm_full: bool = False             # MiniMax-M2: one RMSNorm over all heads of q (and of k) instead of per head
    qk_norm_after_rope: bool = False       # Hunyuan: per-head norm applied after the rotary embedding
    attn_sinks: bool = False               # learned per-head sink logit in the softmax denominator (gpt-oss)
    moe_act: str = "swiglu"                # swiglu | gptoss (clamped, alpha 1.702, (up + 1))
    norm_kind: str = "rms"                 # rms | layernorm (mean-centred, weight + bias: CodeGen / MOSS, GPT-J)
    parallel_block: bool = False           # attention and MLP both read the one pre-norm of the layer; one residual add
    mlp_gated: bool = True                 # False: up projection -> activation -> down projection
    # per-layer attention geometry (Step-3.5 / Laguna: full-attention and sliding-window layers differ)
    layer_heads: list | None = None        # query heads per layer (None: num_heads everywhere)
    layer_rope: list | None = None         # per layer {"theta", "rot_dim", "scaling"} (None: the model-wide rotary tables)
    head_gate: str = ""                    # "sigmoid" | "softplus": g_proj gives one gate per query head on the attention output
    swiglu_limits: list | None = None      # per layer clamp of the routed experts' SwiGLU (0: none): silu(gate) <= l, |up| <= l
    swiglu_limits_shared: list | None = None   # same for the dense MLP / shared expert of the layer
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    num_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0
    shared_expert_gate: bool = False       # qwen2_moe gates the shared expert with a sigmoid
    first_k_dense: int = 0
    moe_layer_freq: int = 1
    scoring_func: str = "softmax"          # softmax | sigmoid
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    router_bias: bool = False              # e_score_correction_bias
    route_group_top1: bool = False         # Pangu Pro MoE: the experts form num_experts_per_tok groups; the best of each group is taken
    # MLA
    use_mla: bool = False
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # sparse attention indexer (DeepSeek-V3.2 / GLM-MoE-DSA): every query attends to its index_topk best-scoring keys
    index_topk: int = 0
    index_n_heads: int = 0
    index_head_dim: int = 0
    # hybrid linear attention (Gated DeltaNet: Qwen3-Next, Qwen3.5)
    layer_types: list | None = None        # per layer "linear_attention" | "full_attention" (None: all full attention)
    lin_num_k_heads: int = 0
    lin_num_v_heads: int = 0
    lin_k_dim: int = 0
    lin_v_dim: int = 0
    lin_conv_kernel: int = 4
    lin_kind: str = "gdn"                  # "gdn" Gated DeltaNet | "lightning" decayed linear attention (MiniMax-Text-01 / M1)
    lin_block: int = 256                   # lightning attention: block length of the chunked evaluation
    # DeepNorm-style residual (MiniMax-Text-01 / M1): the block input is normalised first and the NORMALISED rows are the
    # residual: y = alpha * norm(x) + beta * f(norm(x)).  (alpha, beta) for full-attention layers, linear layers, MLPs.
    postnorm_residual: bool = False
    resid_factors: tuple = (1.0, 1.0, 1.0, 1.0, 1.0, 1.0)
    attn_output_gate: bool = False         # q_proj also produces a per-head gate; the attention output is multiplied by its sigmoid
    mlp_only_layers: list = field(default_factory=list)   # layers that keep a dense MLP in an otherwise sparse model
    mtp_layers: int = 0                    # multi-token-prediction modules stored with the checkpoint (draft heads)
    # bookkeeping
    eos_token_ids: list = field(default_factory=list)
    bos_token_id: int | None = None
    quantization_config: dict | None = None
    torch_dtype: str = "bfloat16"
    raw: dict = field(default_factory=dict)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_is_moe(self, i: int) -> bool:
        if i in self.mlp_only_layers:
            return False
        if self.model_type in ("qwen3_next", "qwen3_5_moe", "qwen3_5_moe_text") and self.moe_layer_freq > 1:
            return self.is_moe and (i + 1) % self.moe_layer_freq == 0
        return self.is_moe and i >= self.first_k_dense and (i % self.moe_layer_freq == 0 or self.moe_layer_freq == 1)

    def layer_is_linear(self, i: int) -> bool:
        return bool(self.layer_types) and i < len(self.layer_types) and self.layer_types[i] == "linear_attention"

    @property
    def has_linear_attn(self) -> bool:
        return bool(self.layer_types) and "linear_attention" in self.layer_types

    @property
    def q_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim if self.use_mla else self.head_dim


LLAMA_LIKE = {"llama", "mistral", "internlm", "internlm3", "baichuan", "yi", "deepseek", "qwen2", "qwen3", "minicpm", "minicpm3",
              "phi3", "glm4", "glm", "gemma", "gemma2", "ernie4_5", "hunyuan", "telechat", "internlm2", "qwen", "cogvlm"}
MOE_LIKE = {"qwen3_moe", "qwen2_moe", "moe", "mixtral", "deepseek_v2", "deepseek_v3", "kimi_k2", "deepseek_v32",
            "glm4_moe", "ernie4_5_moe", "minimax_m2", "minimax", "hunyuan_moe", "gpt_oss", "PanguProMoE", "hy_v3", "step3p5", "step3p7",
            "laguna"}


def _eos_list(v) -> list:
    if v is None:
        return []
    return list(v) if isinstance(v, (list, tuple)) else [v]


def from_hf_dict(d: dict) -> ModelConfig:
    """Build a ModelConfig from the ``config.json`` dictionary of any supported family."""
    if "text_config" in d and isinstance(d["text_config"], dict):   # multimodal wrappers keep the LLM config nested
        inner = dict(d["text_config"])
        inner.setdefault("model_type", d.get("model_type", "llama"))
        for k in ("eos_token_id", "bos_token_id", "tie_word_embeddings", "quantization_config", "vision_config", "image_token_id",
                  "video_token_id", "vision_start_token_id", "vision_end_token_id", "torch_dtype", "dtype"):
            if k in d and k not in inner:
                inner[k] = d[k]
        d = inner
    mt = d.get("model_type", "llama")
    if "CogVLMForCausalLM" in (d.get("architectures") or []) or mt == "CogVLMForCausalLM":
        mt = "cogvlm"                                   # the checkpoint's config names no model_type
    c = ModelConfig(model_type=mt, raw=d, architectures=d.get("architectures", []))
    g = d.get
    c.vocab_size = g("vocab_size", c.vocab_size)
    c.hidden_size = g("hidden_size", g("n_embd", c.hidden_size))
    c.num_layers = g("num_hidden_layers", g("n_layer", g("num_layers", c.num_layers)))
    c.num_heads = g("num_attention_heads", g("n_head", c.num_heads))
    c.num_kv_heads = g("num_key_value_heads", g("multi_query_group_num", c.num_heads)) or c.num_heads
    c.head_dim = g("head_dim") or g("kv_channels") or c.hidden_size // c.num_heads
    c.intermediate_size = g("intermediate_size", g("ffn_hidden_size", c.intermediate_size))
    c.rms_eps = g("rms_norm_eps", g("layernorm_epsilon", g("layer_norm_eps", c.rms_eps)))
    rt = g("rope_theta", g("rotary_emb_base", 10000.0))
    c.rope_theta = float(rt[0] if isinstance(rt, list) else (rt or 10000.0))       # Step-3.5 lists one base per layer
    rs = g("rope_scaling") or g("rope_parameters")
    if isinstance(rs, dict) and isinstance(rs.get("full_attention"), dict):
        # per-layer-type rope parameters (Gemma-3): global layers use "full_attention", sliding layers their own base
        loc = rs.get("sliding_attention") or {}
        c.rope_local_theta = float(loc.get("rope_theta", 10000.0))
        rs = rs["full_attention"]
    if isinstance(rs, dict):
        if "rope_theta" in rs:
            c.rope_theta = float(rs["rope_theta"])
        kind = rs.get("rope_type", rs.get("type", "default"))
        c.rope_scaling = rs if kind not in ("default", None) else None
    c.max_position = g("max_position_embeddings", g("seq_length", c.max_position))
    c.tie_embeddings = bool(g("tie_word_embeddings", False))
    c.attention_bias = bool(g("attention_bias", g("qkv_bias", g("add_qkv_bias", mt in ("qwen2", "qwen2_moe", "qwen")))))
    if mt == "internlm" and g("bias") is not None:          # InternLM (v1): one flag for the q / k / v / o biases
        c.attention_bias = bool(g("bias"))
    c.mlp_bias = bool(g("mlp_bias", False))
    c.hidden_act = g("hidden_act", g("hidden_activation", "silu"))
    c.sliding_window = g("sliding_window") if g("use_sliding_window", True) else None
    c.eos_token_ids = _eos_list(g("eos_token_id"))
    c.bos_token_id = g("bos_token_id")
    c.quantization_config = g("quantization_config")
    c.torch_dtype = str(g("torch_dtype", g("dtype", "bfloat16"))).replace("torch.", "")
    c.mtp_layers = int(g("mtp_num_hidden_layers", g("num_nextn_predict_layers", 0)) or 0)
    # the value inside rope_parameters is the one the model's rotary embedding reads; the top-level key is its legacy place
    prf = (rs.get("partial_rotary_factor") if isinstance(rs, dict) else None) or g("partial_rotary_factor")
    if prf:
        c.rotary_dim = int(c.head_dim * float(prf))
    if mt in ("qwen3", "qwen3_moe", "gemma3_text"):
        c.qk_norm = True
    if mt == "gemma3_text" and g("rope_local_base_freq") and not c.rope_local_theta:
        c.rope_local_theta = float(g("rope_local_base_freq"))          # config.json of released checkpoints
    if mt in ("gemma", "gemma2", "gemma3_text"):
        c.norm_unit_offset = 1.0
        c.embed_scale = float(c.hidden_size) ** 0.5
    if mt in ("chatglm", "glm", "glm4", "ernie4_5", "ernie4_5_moe"):
        c.rope_mode = "interleaved"            # rotates adjacent pairs (x[2i], x[2i+1])
    if mt == "chatglm":                        # ChatGLM2/3, GLM-4 original checkpoints (their own config keys)
        c.vocab_size = g("padded_vocab_size", c.vocab_size)
        c.rotary_dim = c.head_dim // 2
        c.rope_theta = 10000.0 * float(g("rope_ratio", 1.0))
        if not g("multi_query_attention", True):
            c.num_kv_heads = c.num_heads
    if mt == "qwen":                           # Qwen (v1): intermediate_size counts gate and up together
        c.intermediate_size = g("intermediate_size", 2 * c.intermediate_size) // 2
        c.attention_bias = True
        c.num_kv_heads = c.num_heads
    if mt == "glm4":
        c.post_norms = True
    if mt in ("gemma2", "gemma3_text"):
        c.post_norms = True
        c.attn_softcap = float(g("attn_logit_softcapping") or 0.0)
        c.final_softcap = float(g("final_logit_softcapping") or 0.0)
        if g("query_pre_attn_scalar"):
            c.attn_scale_override = float(g("query_pre_attn_scalar")) ** -0.5
    lt = g("layer_types")
    if lt is None and mt == "gemma3_text" and c.sliding_window:
        pat = int(g("sliding_window_pattern", 6) or 6)          # older configs: every pat-th layer is a global one
        lt = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(c.num_layers)]
    if isinstance(lt, list) and c.sliding_window:
        c.layer_windows = [int(c.sliding_window) if t == "sliding_attention" else 0 for t in lt]
    if mt in ("hunyuan_v1_dense", "hunyuan_v1_moe"):
        c.qk_norm = True
        c.qk_norm_after_rope = True
    if mt == "telechat":
        # TeleChat-7B / 12B and TeleChat2: llama-like; keys and values come out of one projection interleaved per head; the
        # first generation rotates with a fixed NTK base 10000 * 3^(d / (d - 2)) (reference: src/models/graph/telechat.cpp:11-43)
        c.intermediate_size = g("ffn_hidden_size", c.intermediate_size)
        c.max_position = g("seq_length", g("max_position_embeddings", c.max_position))
        if "Telechat2ForCausalLM" not in (c.architectures or []) and not g("rope_theta"):
            c.rope_theta = 10000.0 * 3.0 ** (c.head_dim / (c.head_dim - 2))
    if mt in ("moss", "codegen", "gptj"):
        # CodeGen / MOSS-moon and GPT-J: LayerNorm with bias, attention and a two-matrix GELU MLP in parallel from the one
        # norm of the layer, rotary over the first rotary_dim dims of every head in adjacent pairs
        # (reference: src/models/moss.cpp:66-84, 99-118)
        c.norm_kind = "layernorm"
        c.parallel_block = True
        c.mlp_gated = False
        c.rope_mode = "interleaved"
        c.rotary_dim = int(g("rotary_dim") or c.head_dim)
        c.hidden_act = g("activation_function", "gelu_new")
        c.rms_eps = float(g("layer_norm_epsilon", 1e-5))
        c.intermediate_size = int(g("n_inner") or 4 * c.hidden_size)
        c.max_position = int(g("n_positions", g("n_ctx", c.max_position)))
        c.num_kv_heads = c.num_heads
        c.mlp_bias = True
    if mt in ("granite", "granitemoe"):
        c.attn_scale_override = float(g("attention_multiplier", c.head_dim ** -0.5))
        c.embed_scale = float(g("embedding_multiplier", 1.0))
        c.residual_scale = float(g("residual_multiplier", 1.0))
        c.logit_scale = 1.0 / float(g("logits_scaling", 1.0))
    if mt in ("minicpm", "minicpm3"):
        c.embed_scale = float(g("scale_emb", 1.0))
        c.residual_scale = float(g("scale_depth", 1.0)) / (c.num_layers ** 0.5)
        c.logit_scale = 1.0 / (c.hidden_size / float(g("dim_model_base", c.hidden_size)))
    if mt == "gpt_oss":
        c.attn_sinks = True
        c.moe_act = "gptoss"
        c.num_experts = g("num_local_experts", 0)
        c.num_experts_per_tok = g("num_experts_per_tok", 4)
        c.moe_intermediate_size = c.intermediate_size
        c.norm_topk_prob = True
    if mt in ("qwen3_next", "qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text"):
        # hybrid stack: Gated-DeltaNet layers with a gated full-attention layer every few layers; zero-centred norm weights
        # (reference: src/models/qwen3_next.cpp, qwen3_5.cpp)
        c.qk_norm = True
        c.norm_unit_offset = 1.0
        c.attn_output_gate = True
        lt = g("layer_types")
        if lt is None:
            every = int(g("full_attention_interval", 4) or 4)
            lt = ["full_attention" if (i + 1) % every == 0 else "linear_attention" for i in range(c.num_layers)]
        c.layer_types = list(lt)
        c.lin_num_k_heads = g("linear_num_key_heads", 16)
        c.lin_num_v_heads = g("linear_num_value_heads", 32)
        c.lin_k_dim = g("linear_key_head_dim", 128)
        c.lin_v_dim = g("linear_value_head_dim", 128)
        c.lin_conv_kernel = g("linear_conv_kernel_dim", 4)
        c.mlp_only_layers = list(g("mlp_only_layers", []) or [])
        if not prf and not c.rotary_dim:
            c.rotary_dim = int(c.head_dim * 0.25)
    # --- MoE families ---
    if mt in ("qwen3_moe", "qwen2_moe", "moe", "qwen3_next", "qwen3_5_moe", "qwen3_5_moe_text"):
        c.num_experts = g("num_experts", g("num_local_experts", 0))
        c.num_experts_per_tok = g("num_experts_per_tok", 0)
        c.moe_intermediate_size = g("moe_intermediate_size", 0)
        c.norm_topk_prob = bool(g("norm_topk_prob", mt != "qwen2_moe" and mt != "moe"))
        c.moe_layer_freq = g("decoder_sparse_step", 1) or 1
        sis = g("shared_expert_intermediate_size", 0) or 0
        if sis:
            c.num_shared_experts = 1
            c.shared_expert_intermediate_size = sis
            c.shared_expert_gate = True
    elif mt == "hunyuan_v1_moe":
        c.num_experts = g("num_experts", 0)
        tk = g("moe_topk", 1)
        c.num_experts_per_tok = tk[0] if isinstance(tk, list) else tk
        c.moe_intermediate_size = c.intermediate_size          # experts use the full intermediate size
        c.norm_topk_prob = True
        ns = g("num_shared_expert", 0)
        ns = ns[0] if isinstance(ns, list) else ns
        c.num_shared_experts = int(ns or 0)
        c.shared_expert_intermediate_size = c.intermediate_size * c.num_shared_experts
    elif mt == "mixtral":
        c.num_experts = g("num_local_experts", 8)
        c.num_experts_per_tok = g("num_experts_per_tok", 2)
        c.moe_intermediate_size = c.intermediate_size
        c.norm_topk_prob = True
    elif mt in ("minimax", "minimax_text_01", "minimax_m1"):
        # MiniMax-Text-01 / M1: lightning (decayed linear) attention layers with a softmax-attention layer every few layers,
        # every layer MoE (softmax scores, renormalised top-k), DeepNorm-style residuals on normalised rows
        # (reference: src/models/minimax.cpp)
        c.num_experts = g("num_local_experts", g("num_experts", 0)) or 0
        c.num_experts_per_tok = g("num_experts_per_tok", 2)
        c.moe_intermediate_size = c.intermediate_size
        c.norm_topk_prob = True
        lt = g("layer_types")
        if lt is None:
            at = g("attn_type_list")                      # original checkpoints: 0 = lightning, 1 = softmax attention
            lt = (["full_attention" if int(t) == 1 else "linear_attention" for t in at] if at
                  else ["full_attention" if (i % 2) else "linear_attention" for i in range(c.num_layers)])
        c.layer_types = list(lt)
        c.lin_kind = "lightning"
        c.lin_block = int(g("block_size", 256) or 256)
        c.lin_num_k_heads = c.lin_num_v_heads = c.num_heads
        c.lin_k_dim = c.lin_v_dim = c.head_dim
        c.lin_conv_kernel = 1
        c.postnorm_residual = True
        c.resid_factors = tuple(float(g(k, g(k2, 1.0)) or 1.0) for k, k2 in (
            ("full_attn_alpha_factor", "layernorm_full_attention_alpha"), ("full_attn_beta_factor", "layernorm_full_attention_beta"),
            ("linear_attn_alpha_factor", "layernorm_linear_attention_alpha"), ("linear_attn_beta_factor", "layernorm_linear_attention_beta"),
            ("mlp_alpha_factor", "layernorm_mlp_alpha"), ("mlp_beta_factor", "layernorm_mlp_beta")))
        if g("rotary_dim") and not prf:
            c.rotary_dim = int(g("rotary_dim"))
    elif mt == "minimax_m2":
        # GQA + full-width QK norm + partial rotary; every layer MoE: sigmoid scores, selection bias, renormalised top-k
        # (reference: src/models/minimax_m2.cpp)
        c.num_experts = g("num_local_experts", g("num_experts", 0)) or 0
        c.num_experts_per_tok = g("num_experts_per_tok", 0)
        c.moe_intermediate_size = c.intermediate_size
        c.norm_topk_prob = True
        c.scoring_func = g("scoring_func", "sigmoid")
        c.router_bias = True
        c.qk_norm = bool(g("use_qk_norm", True))
        c.qk_norm_full = c.qk_norm and g("qk_norm_type", "per_layer") == "per_layer"
        if g("rotary_dim") and not prf:
            c.rotary_dim = int(g("rotary_dim"))
    elif mt in ("deepseek_v2", "deepseek_v3", "kimi_k2", "deepseek_v32", "glm_moe_dsa", "glm4_moe", "ernie4_5_moe"):
        c.num_experts = g("n_routed_experts", g("num_experts", g("moe_num_experts", 0))) or 0
        c.num_experts_per_tok = g("num_experts_per_tok", g("moe_k", 0))
        c.moe_intermediate_size = g("moe_intermediate_size", 0)
        c.norm_topk_prob = bool(g("norm_topk_prob", True))
        c.num_shared_experts = g("n_shared_experts", g("moe_num_shared_experts", 0)) or 0
        c.shared_expert_intermediate_size = c.moe_intermediate_size * c.num_shared_experts
        c.first_k_dense = g("first_k_dense_replace", g("moe_layer_start_index", 0)) or 0
        c.moe_layer_freq = g("moe_layer_freq", 1) or 1
        c.scoring_func = g("scoring_func", "sigmoid" if mt in ("deepseek_v3", "kimi_k2", "deepseek_v32", "glm_moe_dsa", "glm4_moe") else "softmax")
        c.n_group = g("n_group", 1) or 1
        c.topk_group = g("topk_group", 1) or 1
        c.routed_scaling_factor = float(g("routed_scaling_factor", 1.0))
        c.router_bias = g("topk_method", "") == "noaux_tc" or mt in ("deepseek_v3", "kimi_k2", "deepseek_v32", "glm_moe_dsa", "glm4_moe", "ernie4_5_moe")
        if mt in ("deepseek_v2", "deepseek_v3", "kimi_k2", "deepseek_v32", "glm_moe_dsa"):
            c.use_mla = True
            c.q_lora_rank = g("q_lora_rank") or 0
            c.kv_lora_rank = g("kv_lora_rank", 512)
            c.qk_nope_head_dim = g("qk_nope_head_dim", 128)
            c.qk_rope_head_dim = g("qk_rope_head_dim", 64)
            c.v_head_dim = g("v_head_dim", 128)
            c.rope_mode = "neox" if mt == "glm_moe_dsa" else "interleaved"
            if mt in ("glm_moe_dsa", "deepseek_v32"):
                c.index_topk = int(g("index_topk", 2048) or 0)
                c.index_n_heads = int(g("index_n_heads", 64) or 0)
                c.index_head_dim = int(g("index_head_dim", 128) or 0)
            if mt == "glm_moe_dsa":
                c.latent_norm_eps = 1e-6
            c.head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
        if mt == "glm4_moe":
            c.qk_norm = bool(g("use_qk_norm", False))
    elif mt in ("hy_v3", "HYV3ForCausalLM"):
        # Hunyuan v3: per-head QK norm before the rotary embedding, softmax or sigmoid router with a selection bias
        # (``mlp.expert_bias``), renormalised top-k times a scaling factor, shared MLP, leading dense layers; layers stored
        # beyond num_hidden_layers (multi-token-prediction heads) are not part of the decoder
        # (reference: src/models/hy_v3.cpp:2217-2232, 2002-2046)
        c.model_type = "hy_v3"
        c.qk_norm = True
        c.num_experts = g("num_experts", 0) or 0
        c.num_experts_per_tok = g("num_experts_per_tok", g("moe_topk", 0)) or 0
        c.moe_intermediate_size = g("moe_intermediate_size", g("expert_hidden_dim", c.intermediate_size))
        c.norm_topk_prob = bool(g("norm_topk_prob", g("route_norm", True)))
        c.first_k_dense = g("first_k_dense_replace", 0) or 0
        c.num_shared_experts = g("num_shared_experts", g("n_shared_experts", 0)) or 0
        c.shared_expert_intermediate_size = c.moe_intermediate_size * c.num_shared_experts
        c.scoring_func = "sigmoid" if g("moe_router_use_sigmoid", False) else "softmax"
        c.routed_scaling_factor = float(g("routed_scaling_factor", g("router_scaling_factor", 1.0)))
        c.router_bias = True
    elif mt == "PanguProMoE":
        # Pangu Pro MoE (mixture of grouped experts): softmax scores, one expert from each of num_experts_per_tok equal groups,
        # weight = score x a learned per-expert scale, no renormalisation; un-gated shared expert; biases on q / k / v / o
        # (reference: src/models/pangu_moe.cpp:385-432)
        c.num_experts = g("num_experts", 0) or 0
        c.num_experts_per_tok = g("num_experts_per_tok", 0) or 0
        c.moe_intermediate_size = g("moe_intermediate_size", c.intermediate_size)
        c.norm_topk_prob = False
        c.route_group_top1 = True
        c.attention_bias = bool(g("attention_bias", g("qkv_bias", True)))
        sis = g("shared_expert_intermediate_size", 0) or 0
        if sis:
            c.num_shared_experts = 1
            c.shared_expert_intermediate_size = sis
    if mt in ("step3p5", "step3p7", "laguna"):
        _step_family(c, g, mt)
    if mt == "minicpm3":
        # MiniCPM3: multi-head latent attention (rotate-half rotary on the shared rope dims) over dense MLPs, with the MiniCPM
        # embedding / residual / logit multipliers (reference: src/models/minicpm3.cpp:60-90, 147-152)
        c.use_mla = True
        c.q_lora_rank = g("q_lora_rank") or 0
        c.kv_lora_rank = g("kv_lora_rank", 256)
        c.qk_nope_head_dim = g("qk_nope_head_dim", 64)
        c.qk_rope_head_dim = g("qk_rope_head_dim", 32)
        c.v_head_dim = g("v_head_dim", c.hidden_size // c.num_heads)
        c.rope_mode = "neox"
        c.head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
        c.num_kv_heads = c.num_heads
    return c


def _step_family(c: ModelConfig, g, mt: str) -> None:
    """Step-3.5 / 3.7 (text) and Laguna: full-attention and sliding-window layers with their own head counts, rotary base
    and rotary width; per-head QK norm; one learned gate per query head on the attention output; sigmoid router with a
    selection bias, renormalised top-k times a factor, one shared expert; optional clamps inside the SwiGLU.
    Reference: src/models/step3p5.cpp:4322-4446, 6320-6670; src/models/laguna.cpp:670-830, 1123-1160."""
    L = c.num_layers
    c.qk_norm = True
    c.scoring_func = "sigmoid"
    c.router_bias = True
    c.num_shared_experts = 1
    lt = g("layer_types")
    if not isinstance(lt, list) or len(lt) != L:
        lt = ["full_attention" if i % 4 == 0 else "sliding_attention" for i in range(L)]
    win = int(g("sliding_window", 512) or 0)
    c.sliding_window = win or None
    c.layer_windows = [0 if t == "full_attention" else win for t in lt]
    if mt == "laguna":
        c.model_type = "laguna"
        c.head_gate = "softplus"
        kv = int(g("num_key_value_heads", 8))
        hp = g("num_attention_heads_per_layer")
        c.layer_heads = list(hp) if isinstance(hp, list) and len(hp) == L else [c.num_heads] * L
        c.num_experts = g("num_experts", 0) or 0
        c.num_experts_per_tok = g("num_experts_per_tok", 0) or 0
        c.norm_topk_prob = bool(g("norm_topk_prob", True))
        c.routed_scaling_factor = float(g("moe_routed_scaling_factor", 1.0))
        c.shared_expert_intermediate_size = g("shared_expert_intermediate_size", 1024)
        step = max(1, int(g("decoder_sparse_step", 1) or 1))
        dense = set(g("mlp_only_layers", []) or [])
        c.mlp_only_layers = [i for i in range(L) if i in dense or (i + 1) % step != 0]
        rp = g("rope_parameters") or {}
        full, slide = dict(rp.get("full_attention") or {}), dict(rp.get("sliding_attention") or {})
        c.rope_theta = float(full.get("rope_theta", 500000.0))
        c.rope_scaling = None
        c.rope_local_theta = 0.0
        fk = full.get("rope_type", full.get("type", "default"))
        f_rot = max(2, int(c.head_dim * float(full.get("partial_rotary_factor", 0.5))))
        s_rot = max(2, int(c.head_dim * float(slide.get("partial_rotary_factor", 1.0))))
        f_spec = {"theta": c.rope_theta, "rot_dim": f_rot, "scaling": full if fk not in ("default", None) else None}
        s_spec = {"theta": float(slide.get("rope_theta", 10000.0)), "rot_dim": s_rot, "scaling": None}
        c.layer_rope = [f_spec if t == "full_attention" else s_spec for t in lt]
        c.rotary_dim = f_rot
    else:
        c.model_type = "step3p5"
        c.head_gate = "sigmoid"
        c.norm_unit_offset = 1.0               # the checkpoints store norm weights as deltas from one
        kv = int(g("num_attention_groups", g("num_key_value_heads", 8)))
        other = g("attention_other_setting") or {}
        oh = int(other.get("num_attention_heads", c.num_heads))
        if int(other.get("num_attention_groups", kv)) != kv:
            raise NotImplementedError("step3p5: sliding-window layers with their own number of KV heads")
        c.layer_heads = [c.num_heads if t == "full_attention" else oh for t in lt]
        c.num_experts = g("moe_num_experts", 0) or 0
        c.num_experts_per_tok = g("moe_top_k", 0) or 0
        c.norm_topk_prob = bool(g("norm_expert_weight", True))
        c.routed_scaling_factor = float(g("moe_router_scaling_factor", 1.0))
        c.router_bias = bool(g("use_moe_router_bias", True))
        c.shared_expert_intermediate_size = g("share_expert_dim", c.intermediate_size)
        me = g("moe_layers_enum")
        if isinstance(me, str):
            me = [int(v) for v in me.replace(" ", "").split(",") if v]
        moe_layers = set(me) if me else set(range(1, L))
        c.mlp_only_layers = [i for i in range(L) if i not in moe_layers]
        th = g("rope_theta")
        thetas = [float(v) for v in th] if isinstance(th, list) else [float(th or 10000.0)] * L
        thetas += [thetas[-1]] * (L - len(thetas))
        pr = g("partial_rotary_factors")
        prs = [float(v) for v in pr] if isinstance(pr, list) else [1.0] * L
        prs += [1.0] * (L - len(prs))
        sc = g("rope_scaling")
        llama3 = isinstance(sc, dict) and sc.get("rope_type", sc.get("type")) == "llama3"
        c.layer_rope = [{"theta": thetas[i], "rot_dim": max(2, int(c.head_dim * prs[i] + 1e-5)),
                         "scaling": (sc if (llama3 and lt[i] == "full_attention") else None)} for i in range(L)]
        c.rope_theta = thetas[0]
        c.rope_scaling = None
        c.rotary_dim = c.layer_rope[0]["rot_dim"]
        for key, attr in (("swiglu_limits", "swiglu_limits"), ("swiglu_limits_shared", "swiglu_limits_shared")):
            v = g(key)
            if isinstance(v, list) and any(float(x or 0) != 0.0 for x in v):
                setattr(c, attr, [float(x or 0.0) for x in v] + [0.0] * (L - len(v)))
    c.num_kv_heads = kv
    c.moe_intermediate_size = g("moe_intermediate_size", c.intermediate_size)
    c.moe_layer_freq = 1
    c.first_k_dense = 0


def load_config(path: str | Path) -> ModelConfig:
    p = Path(path)
    if p.is_dir():
        p = p / "config.json"
    with open(p, "r", encoding="utf-8") as f:
        return from_hf_dict(json.load(f))


# ---------------------------------------------------------------------------------------------------
# Named architectures used by the benchmarks and tests (random-init, no checkpoint needed)
# ---------------------------------------------------------------------------------------------------
def preset(name: str) -> ModelConfig:
    name = name.lower()
    if name in ("qwen3-0.6b", "qwen3_0.6b"):
        return from_hf_dict(dict(model_type="qwen3", vocab_size=151936, hidden_size=1024, num_hidden_layers=28,
                                 num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
                                 rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True, max_position_embeddings=40960))
    if name in ("llama-3-8b", "llama3-8b"):
        return from_hf_dict(dict(model_type="llama", vocab_size=128256, hidden_size=4096, num_hidden_layers=32,
                                 num_attention_heads=32, num_key_value_heads=8, intermediate_size=14336, rms_norm_eps=1e-5,
                                 rope_theta=5e5, max_position_embeddings=8192))
    if name in ("llama-3-70b", "llama3-70b"):
        return from_hf_dict(dict(model_type="llama", vocab_size=128256, hidden_size=8192, num_hidden_layers=80,
                                 num_attention_heads=64, num_key_value_heads=8, intermediate_size=28672, rms_norm_eps=1e-5,
                                 rope_theta=5e5, max_position_embeddings=8192))
    if name in ("qwen3-30b-a3b",):
        return from_hf_dict(dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, num_hidden_layers=48,
                                 num_attention_heads=32, num_key_value_heads=4, head_dim=128, intermediate_size=6144,
                                 moe_intermediate_size=768, num_experts=128, num_experts_per_tok=8, norm_topk_prob=True,
                                 rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960))
    if name in ("deepseek-v3", "deepseek_v3"):
        return from_hf_dict(dict(model_type="deepseek_v3", vocab_size=129280, hidden_size=7168, num_hidden_layers=61,
                                 num_attention_heads=128, num_key_value_heads=128, intermediate_size=18432,
                                 moe_intermediate_size=2048, n_routed_experts=256, num_experts_per_tok=8, n_shared_experts=1,
                                 first_k_dense_replace=3, n_group=8, topk_group=4, routed_scaling_factor=2.5,
                                 scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True, q_lora_rank=1536,
                                 kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                                 rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=163840))
    if name == "tiny-llama":
        return from_hf_dict(dict(model_type="llama", vocab_size=512, hidden_size=256, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=512,
                                 rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048))
    if name == "tiny-qwen3":
        return from_hf_dict(dict(model_type="qwen3", vocab_size=512, hidden_size=256, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=512,
                                 rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True, max_position_embeddings=2048))
    if name == "tiny-qwen3-moe":
        return from_hf_dict(dict(model_type="qwen3_moe", vocab_size=512, hidden_size=256, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=512,
                                 moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2, norm_topk_prob=True,
                                 rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=2048))
    if name == "tiny-qwen3-next":
        return from_hf_dict(dict(model_type="qwen3_next", vocab_size=512, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=512, num_experts=8, num_experts_per_tok=2,
                                 moe_intermediate_size=128, shared_expert_intermediate_size=128, linear_num_key_heads=2,
                                 linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32, full_attention_interval=2,
                                 max_position_embeddings=2048, rms_norm_eps=1e-6, eos_token_id=511))
    if name == "tiny-minimax-m1":        # lightning-attention / softmax-attention hybrid with DeepNorm-style residual factors
        return from_hf_dict(dict(model_type="minimax", vocab_size=512, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=256, num_local_experts=8, num_experts_per_tok=2,
                                 block_size=32, layer_types=["linear_attention", "full_attention"] * 2,
                                 full_attn_alpha_factor=1.5, full_attn_beta_factor=0.8, linear_attn_alpha_factor=1.25,
                                 linear_attn_beta_factor=0.9, mlp_alpha_factor=1.1, mlp_beta_factor=0.7,
                                 max_position_embeddings=2048, rms_norm_eps=1e-5, eos_token_id=511))
    if name == "tiny-minimax-m2":        # full-width QK norm, partial rotary, sigmoid router with selection bias
        return from_hf_dict(dict(model_type="minimax_m2", vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=256, num_local_experts=8, num_experts_per_tok=2,
                                 rotary_dim=32, max_position_embeddings=2048, rms_norm_eps=1e-6, eos_token_id=511))
    if name == "tiny-minicpm3":          # latent attention over dense MLPs with the MiniCPM multipliers
        return from_hf_dict(dict(model_type="minicpm3", vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                                 intermediate_size=512, q_lora_rank=128, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16,
                                 v_head_dim=32, scale_emb=12.0, scale_depth=1.4, dim_model_base=64, rms_norm_eps=1e-5,
                                 max_position_embeddings=2048, eos_token_id=511))
    if name == "tiny-llama-mtp":         # tiny llama with one multi-token-prediction module (speculative decoding tests)
        return from_hf_dict(dict(model_type="llama", vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=512, rms_norm_eps=1e-5, rope_theta=10000.0,
                                 max_position_embeddings=2048, num_nextn_predict_layers=1))
    if name == "tiny-moss":              # LayerNorm, parallel attention / GELU MLP block, partial pairwise rotary
        return from_hf_dict(dict(model_type="moss", vocab_size=512, n_embd=256, n_layer=2, n_head=4, rotary_dim=32, n_positions=2048,
                                 activation_function="gelu_new", layer_norm_epsilon=1e-5, eos_token_id=511))
    if name == "tiny-step3p5":           # full / sliding layers with 4 / 6 query heads, own rotary base and width, head gates
        return from_hf_dict(dict(model_type="step3p5", vocab_size=512, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                                 num_attention_groups=2, head_dim=64, intermediate_size=512, moe_intermediate_size=128,
                                 moe_num_experts=8, moe_top_k=2, share_expert_dim=128, moe_router_scaling_factor=2.0,
                                 attention_other_setting={"num_attention_heads": 6, "num_attention_groups": 2},
                                 rope_theta=[1e6, 1e4, 1e4, 1e4], partial_rotary_factors=[0.5, 1.0, 1.0, 1.0], sliding_window=16,
                                 swiglu_limits=[0, 0, 0, 7.0], swiglu_limits_shared=[0, 0, 0, 16.0],
                                 max_position_embeddings=2048, rms_norm_eps=1e-5, eos_token_id=511))
    if name == "tiny-laguna":            # Laguna: softplus head gates, yarn rotary on half of each head in the full-attention layers
        return from_hf_dict(dict(model_type="laguna", vocab_size=512, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=512, moe_intermediate_size=128,
                                 num_experts=8, num_experts_per_tok=2, shared_expert_intermediate_size=128,
                                 moe_routed_scaling_factor=2.5, num_attention_heads_per_layer=[4, 6, 6, 6],
                                 layer_types=["full_attention", "sliding_attention", "sliding_attention", "sliding_attention"],
                                 mlp_only_layers=[0], sliding_window=16,
                                 rope_parameters={"full_attention": {"rope_type": "yarn", "rope_theta": 500000.0, "factor": 8.0,
                                                                     "original_max_position_embeddings": 256, "partial_rotary_factor": 0.5},
                                                  "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0}},
                                 max_position_embeddings=2048, rms_norm_eps=1e-6, eos_token_id=511))
    if name == "tiny-hy-v3":             # per-head QK norm, sigmoid router with selection bias, shared MLP, one leading dense layer
        return from_hf_dict(dict(model_type="hy_v3", vocab_size=512, hidden_size=256, num_hidden_layers=3, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=512, moe_intermediate_size=128, num_experts=8,
                                 num_experts_per_tok=2, num_shared_experts=1, first_k_dense_replace=1, moe_router_use_sigmoid=True,
                                 router_scaling_factor=2.0, max_position_embeddings=2048, rms_norm_eps=1e-6, eos_token_id=511))
    if name == "tiny-pangu-moe":         # grouped experts: one expert from each of num_experts_per_tok groups
        return from_hf_dict(dict(model_type="PanguProMoE", vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, intermediate_size=512, moe_intermediate_size=128, num_experts=8,
                                 num_experts_per_tok=4, shared_expert_intermediate_size=256, max_position_embeddings=2048,
                                 rms_norm_eps=1e-5, eos_token_id=511))
    if name == "small-qwen3-next":       # Qwen3-Next layer geometry (128-wide delta-rule heads, 128-wide attention heads) on a small body
        return from_hf_dict(dict(model_type="qwen3_next", vocab_size=1024, hidden_size=512, num_hidden_layers=4, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=128, intermediate_size=1024, num_experts=8, num_experts_per_tok=2,
                                 moe_intermediate_size=256, shared_expert_intermediate_size=256, linear_num_key_heads=2,
                                 linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128, full_attention_interval=2,
                                 max_position_embeddings=2048, rms_norm_eps=1e-6, eos_token_id=1023))
    if name in ("qwen3-next-80b-a3b",):
        return from_hf_dict(dict(model_type="qwen3_next", vocab_size=151936, hidden_size=2048, num_hidden_layers=48, num_attention_heads=16,
                                 num_key_value_heads=2, head_dim=256, intermediate_size=5120, num_experts=512, num_experts_per_tok=10,
                                 moe_intermediate_size=512, shared_expert_intermediate_size=512, linear_num_key_heads=16,
                                 linear_num_value_heads=32, linear_key_head_dim=128, linear_value_head_dim=128, full_attention_interval=4,
                                 max_position_embeddings=262144, rms_norm_eps=1e-6, rope_theta=1e7, eos_token_id=151645))
    if name == "tiny-deepseek-v3":
        return from_hf_dict(dict(model_type="deepseek_v3", vocab_size=512, hidden_size=256, num_hidden_layers=3,
                                 num_attention_heads=4, num_key_value_heads=4, intermediate_size=512,
                                 moe_intermediate_size=128, n_routed_experts=16, num_experts_per_tok=4, n_shared_experts=1,
                                 first_k_dense_replace=1, n_group=4, topk_group=2, routed_scaling_factor=2.5,
                                 scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True, q_lora_rank=128,
                                 kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                                 rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=2048))
    if name == "tiny-deepseek-v32":      # latent attention with the sparse-attention indexer (selection size 32)
        return from_hf_dict(dict(model_type="deepseek_v32", vocab_size=512, hidden_size=256, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=4, intermediate_size=512,
                                 moe_intermediate_size=128, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1,
                                 first_k_dense_replace=1, n_group=1, topk_group=1, routed_scaling_factor=2.5,
                                 scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True, q_lora_rank=128,
                                 kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                                 index_topk=32, index_n_heads=4, index_head_dim=32,
                                 rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=2048, eos_token_id=511))
    if name == "small-deepseek-v3":      # DeepSeek-V3 attention geometry (latent 512 + rope 64) on a small body
        return from_hf_dict(dict(model_type="deepseek_v3", vocab_size=1024, hidden_size=512, num_hidden_layers=2,
                                 num_attention_heads=8, num_key_value_heads=8, intermediate_size=1024,
                                 moe_intermediate_size=256, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1,
                                 first_k_dense_replace=1, n_group=2, topk_group=1, routed_scaling_factor=2.5,
                                 scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True, q_lora_rank=256,
                                 kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                                 rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=4096))
    raise KeyError(f"unknown preset '{name}'")
