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
    "glm4_moe": dict(model_type="glm4_moe", **_C, moe_intermediate_size=128, n_routed_experts=8, num_experts_per_tok=2,
                     n_shared_experts=1, first_k_dense_replace=1, n_group=1, topk_group=1, partial_rotary_factor=0.5, use_qk_norm=True),
    "ernie4_5": dict(model_type="ernie4_5", **_C),
    "hunyuan_v1_dense": dict(model_type="hunyuan_v1_dense", **_C),
    "gpt_oss": dict(model_type="gpt_oss", **_C, num_local_experts=4, num_experts_per_tok=2, sliding_window=16),
    "granite": dict(model_type="granite", **_NH, attention_multiplier=0.2, embedding_multiplier=3.0, residual_multiplier=0.5,
                    logits_scaling=2.0),
}


@pytest.mark.parametrize("name", sorted(FAMILIES))
def test_family_matches_transformers(name, tmp_path):
    torch.manual_seed(0)
    try:
        cfg = transformers.AutoConfig.for_model(**FAMILIES[name])
        ref = transformers.AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.float32)
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
                      logit_rows=torch.tensor([T - 1]), cu_q_host=[0, T])
    got = m.forward(fb, eng.runner.kv.pools)[0].float()[:want.numel()]
    assert torch.nn.functional.cosine_similarity(got, want, dim=0).item() > 0.99999
    assert (got - want).abs().max().item() < 2e-3
    assert int(got.argmax()) == int(want.argmax())
