"""The reference's package names keep working: `ftllm` and `fastllm_pytools` (llm, util, hf_model.create, torch2flm.tofile)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def test_fastllm_pytools_alias(tmp_path):
    import fastllm_pytools
    import ftllm
    from fastllm_b200 import llm
    from fastllm_pytools import hf_model, torch2flm

    assert fastllm_pytools.llm is llm and ftllm.llm is llm
    cfg = transformers.LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=256)
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(cfg).eval().float()
    llm.set_device_map("cpu")
    m = hf_model.create(hf, None, dtype="float32")
    prompt = [5, 9, 17, 33, 2, 8]
    try:
        got = list(m.stream_response_raw(prompt, max_length=6, do_sample=False, stop_token_ids=[]))
    finally:
        m.release_memory()
    with torch.no_grad():
        want = hf.generate(torch.tensor([prompt]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(prompt):].tolist()
    assert got[:len(want)] == want[:len(got)] and len(got) >= 1
    out = tmp_path / "tiny.flm"
    torch2flm.tofile(str(out), hf, None, dtype="float16")
    assert out.stat().st_size > 100_000
    m2 = llm.model(str(out), device="cpu")
    try:
        assert m2.get_type() == "llama"
        assert len(list(m2.stream_response_raw(prompt, max_length=3, do_sample=False, stop_token_ids=[]))) >= 1
    finally:
        m2.release_memory()
