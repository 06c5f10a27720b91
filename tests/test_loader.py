"""Loader: safetensors round trip, HF folder -> model parity with the random-init path, dtype_config rules,
pre-quantised (block FP8) checkpoints, and parity with Hugging Face transformers on tiny random models."""
import json
import os

import pytest
import torch

from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
from fastllm_b200.loader import hf, safetensors as st
from fastllm_b200.models import preset, random_init
from fastllm_b200.ops import quant


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4, 4).bfloat16(), "c": torch.arange(7, dtype=torch.int32),
         "d": torch.randn(8, 8).to(torch.float8_e4m3fn)}
    st.save_file(t, tmp_path / "x.safetensors", metadata={"format": "pt"})
    f = st.SafeTensorFile(tmp_path / "x.safetensors")
    for k, v in t.items():
        got = f.get(k)
        assert got.dtype == v.dtype and torch.equal(got.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else got,
                                                    v.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else v)
    f.close()


def _write_hf(tmp_path, name, transform=None):
    from baseline import synth

    d = synth.write_model(name, str(tmp_path / name), dtype=torch.float32, std=0.05)
    return d


def test_hf_folder_matches_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    d = _write_hf(tmp_path, "tiny-llama")
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=16)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 500, (37,), generator=g).tolist()
    out = eng.generate([prompt], GenerationConfig(max_new_tokens=8, ignore_eos=True))[0]
    ref = transformers.AutoModelForCausalLM.from_pretrained(d, torch_dtype=torch.float32)
    ref.eval()
    with torch.no_grad():
        ids = torch.tensor([prompt])
        gen = ref.generate(ids, max_new_tokens=8, do_sample=False, eos_token_id=None, pad_token_id=0)
    assert gen[0, len(prompt):].tolist() == out


def test_qwen3_matches_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    d = _write_hf(tmp_path, "tiny-qwen3")
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=16)
    prompt = list(range(5, 150, 3))
    out = eng.generate([prompt], GenerationConfig(max_new_tokens=6, ignore_eos=True))[0]
    ref = transformers.AutoModelForCausalLM.from_pretrained(d, torch_dtype=torch.float32)
    ref.eval()
    with torch.no_grad():
        gen = ref.generate(torch.tensor([prompt]), max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)
    assert gen[0, len(prompt):].tolist() == out


def test_dtype_config_rules():
    rules = [{"key": "mlp", "dtype": "int4g128"}, {"key": "down_proj", "dtype": "int8"}]
    assert hf.resolve_wdtype("model.layers.0.mlp.gate_proj.weight", "float16", rules) == "int4g128"
    assert hf.resolve_wdtype("model.layers.0.mlp.down_proj.weight", "float16", rules) == "int8"
    assert hf.resolve_wdtype("model.layers.0.self_attn.q_proj.weight", "float16", rules) == "float16"


def test_fp8_block_checkpoint(tmp_path):
    w = torch.randn(256, 384) * 0.05
    q, s = quant.quantize_fp8_block(w)
    back = hf.dequant_fp8_block(q, s, torch.float32)
    assert (back - w).abs().max() < 0.02
    assert torch.allclose(back, quant.dequantize_fp8_block(q, s, torch.float32))


@pytest.mark.parametrize("kind", ["int8", "int4g128", "fp8"])
def test_quant_roundtrip_error(kind):
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.05
    lw = quant.LinearWeight.from_dense(w, kind, act_dtype=torch.float32)
    err = (lw.dequant(torch.float32) - w).abs().max().item()
    assert err < {"int8": 0.002, "int4g128": 0.03, "fp8": 0.02}[kind]
    x = torch.randn(5, 256)
    y = lw(x)
    assert torch.allclose(y, x @ lw.dequant(torch.float32).t(), atol=1e-4)


def test_int4g_packing_high_nibble_first():
    w = torch.tensor([[0.0, 15.0] * 64])
    packed, scale, mn = quant.quantize_int4g(w, 128)
    assert packed[0, 0].item() == 0x0F      # first value (0) in the high nibble, second (15) in the low nibble


def test_lora_adapter_is_merged_at_load(tmp_path):
    """A PEFT-style adapter folder: the loaded projection equals W + (alpha / r) * B @ A."""
    import json

    from fastllm_b200.loader.safetensors import save_file

    d = _write_hf(tmp_path, "tiny-llama")
    base = hf.load_model(d, device="cpu", dtype=torch.float32)
    torch.manual_seed(0)
    r, alpha = 4, 8
    H = base.cfg.hidden_size
    K = base.cfg.num_heads * base.cfg.head_dim
    a, b = torch.randn(r, K) * 0.1, torch.randn(H, r) * 0.1          # o_proj of layer 1: [H, heads * head_dim]
    ad = tmp_path / "adapter"
    ad.mkdir()
    (ad / "adapter_config.json").write_text(json.dumps({"r": r, "lora_alpha": alpha, "target_modules": ["o_proj"]}))
    save_file({"base_model.model.model.layers.1.self_attn.o_proj.lora_A.weight": a,
               "base_model.model.model.layers.1.self_attn.o_proj.lora_B.weight": b}, ad / "adapter_model.safetensors")
    tuned = hf.load_model(d, device="cpu", dtype=torch.float32, lora=str(ad))
    want = base.layers[1].attn.o.w + (alpha / r) * (b @ a)
    assert torch.allclose(tuned.layers[1].attn.o.w, want, atol=1e-6)
    assert torch.equal(tuned.layers[0].attn.o.w, base.layers[0].attn.o.w)


def test_runtime_adapter_matches_merged_and_switches(tmp_path):
    """Run-time adapters on every projection kind (fused qkv, o, interleaved gate/up, down): same logits as the merged load,
    and the base logits again after ``set_adapter(None)``."""
    import json

    from fastllm_b200 import lora
    from fastllm_b200.engine import EngineConfig, LLMEngine
    from fastllm_b200.loader.safetensors import save_file
    from fastllm_b200.models.decoder import ForwardBatch

    d = _write_hf(tmp_path, "tiny-llama")
    base = hf.load_model(d, device="cpu", dtype=torch.float32)
    c = base.cfg
    torch.manual_seed(1)
    r, alpha = 4, 8
    shapes = {"self_attn.q_proj": (c.num_heads * c.head_dim, c.hidden_size), "self_attn.v_proj": (c.num_kv_heads * c.head_dim, c.hidden_size),
              "self_attn.o_proj": (c.hidden_size, c.num_heads * c.head_dim), "mlp.gate_proj": (c.intermediate_size, c.hidden_size),
              "mlp.up_proj": (c.intermediate_size, c.hidden_size), "mlp.down_proj": (c.hidden_size, c.intermediate_size)}
    t = {}
    for i in range(c.num_layers):
        for nm, (n, k) in shapes.items():
            t[f"base_model.model.model.layers.{i}.{nm}.lora_A.weight"] = torch.randn(r, k) * 0.1
            t[f"base_model.model.model.layers.{i}.{nm}.lora_B.weight"] = torch.randn(n, r) * 0.1
    ad = tmp_path / "adapter"
    ad.mkdir()
    (ad / "adapter_config.json").write_text(json.dumps({"r": r, "lora_alpha": alpha}))
    save_file(t, ad / "adapter_model.safetensors")
    merged = hf.load_model(d, device="cpu", dtype=torch.float32, lora=str(ad))

    def logits(m):
        prompt = list(range(3, 40, 2))
        T = len(prompt)
        eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=256), num_pages=4)
        fb = ForwardBatch(ids=torch.tensor(prompt, dtype=torch.int32), positions=torch.arange(T, dtype=torch.int32),
                          slots=torch.arange(T, dtype=torch.int32), page_table=torch.tensor([[0, 1]], dtype=torch.int32),
                          kv_lens=torch.tensor([T], dtype=torch.int32), cu_q=torch.tensor([0, T], dtype=torch.int32),
                          logit_rows=torch.tensor([T - 1]), cu_q_host=[0, T])
        return m.forward(fb, eng.runner.kv.pools)[0].float()

    want_base, want_tuned = logits(base), logits(merged)
    assert (want_base - want_tuned).abs().max() > 1e-3
    assert lora.load_adapter(base, "a", str(ad)) == 4 * c.num_layers
    try:
        lora.set_adapter("a")
        assert torch.allclose(logits(base), want_tuned, atol=2e-4)
        lora.set_adapter("other")                      # a name no weight carries: base behaviour
        assert torch.allclose(logits(base), want_base, atol=1e-5)
    finally:
        lora.set_adapter(None)
    assert torch.allclose(logits(base), want_base, atol=1e-5)


def test_split_layers_by_device_map():
    from fastllm_b200.loader.shard import split_layers_by_map

    d = split_layers_by_map(10, {"cuda:0": 3, "cuda:1": 2})
    assert [str(x) for x in d] == ["cuda:0"] * 6 + ["cuda:1"] * 4
    assert [str(x) for x in split_layers_by_map(3, {"cuda:0": 1, "cuda:1": 1, "cuda:2": 1})] == ["cuda:0", "cuda:1", "cuda:2"]
    assert len(split_layers_by_map(7, {"cuda:0": 1})) == 7


def test_moe_device_disk_keeps_experts_in_the_file_mapping(tmp_path):
    """``moe_device="disk"``: expert matrices are views of the checkpoint mapping (no copy), results equal the normal load."""
    import mmap

    from fastllm_b200.engine import EngineConfig, LLMEngine
    from fastllm_b200.models.decoder import ForwardBatch

    import json
    import os

    from fastllm_b200.loader.safetensors import save_file

    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    cfg = transformers.AutoConfig.for_model(model_type="qwen3_moe", vocab_size=512, hidden_size=256, num_hidden_layers=2,
                                            num_attention_heads=4, num_key_value_heads=2, intermediate_size=512, head_dim=64,
                                            max_position_embeddings=512, num_experts=4, num_experts_per_tok=2,
                                            moe_intermediate_size=128, decoder_sparse_step=1, norm_topk_prob=True)
    ref = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    sd = {}
    for k, v in ref.state_dict().items():          # classic per-expert names, written in sorted order (gate_proj next to up_proj)
        v = v.detach()
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(v.shape[0]):
                sd[k[:-len("gate_up_proj")] + f"{e}.gate_proj.weight"] = v[e][:v.shape[1] // 2].contiguous()
                sd[k[:-len("gate_up_proj")] + f"{e}.up_proj.weight"] = v[e][v.shape[1] // 2:].contiguous()
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(v.shape[0]):
                sd[k[:-len("down_proj")] + f"{e}.down_proj.weight"] = v[e].contiguous()
        else:
            sd[k] = v.contiguous()
    d = str(tmp_path / "moe")
    os.makedirs(d)
    save_file({k: sd[k] for k in sorted(sd)}, os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    base = hf.load_model(d, device="cpu", dtype=torch.float32)
    disk = hf.load_model(d, device="cpu", dtype=torch.float32, moe_device="disk")
    ex_b, ex_d = base.layers[0].mlp.experts, disk.layers[0].mlp.experts
    assert torch.equal(ex_b.gate_up[1].w, ex_d.gate_up[1].w) and torch.equal(ex_b.down[1].w, ex_d.down[1].w)
    # a view of a file mapping is page-aligned storage + header offset, and two experts are file-distance apart, not malloc-distance
    w0, w1 = ex_d.gate_up[0].w, ex_d.gate_up[1].w
    per_expert = 3 * w0.numel() // 2 * w0.element_size()          # gate + up + down bytes of one expert
    assert abs(w1.data_ptr() - w0.data_ptr()) == per_expert
    assert not w0.requires_grad and w0._base is not None             # a view, not an owning tensor

    def logits(m):
        prompt = list(range(3, 40, 2))
        T = len(prompt)
        eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=256), num_pages=4)
        fb = ForwardBatch(ids=torch.tensor(prompt, dtype=torch.int32), positions=torch.arange(T, dtype=torch.int32),
                          slots=torch.arange(T, dtype=torch.int32), page_table=torch.tensor([[0, 1]], dtype=torch.int32),
                          kv_lens=torch.tensor([T], dtype=torch.int32), cu_q=torch.tensor([0, T], dtype=torch.int32),
                          logit_rows=torch.tensor([T - 1]), cu_q_host=[0, T])
        return m.forward(fb, eng.runner.kv.pools)[0].float()

    assert torch.allclose(logits(base), logits(disk), atol=1e-5)


def test_activation_mode_routing():
    """Which activation form a quantised projection asks its producer for (fused quantiser in the norm / attention combine)."""
    from fastllm_b200.ops import quant_gemm as QG
    from fastllm_b200.ops.quant import LinearWeight

    w = torch.randn(256, 512) * 0.05
    dense, i8, i4, f8 = (LinearWeight.from_dense(w, k) for k in ("dense", "int8", "int4g128", "fp8"))
    assert QG.act_quant_mode(dense, 4) == 0 and QG.act_quant_mode(None, 4) == 0
    assert QG.act_quant_mode(i8, 1) == 1 and QG.act_quant_mode(i8, 128) == 1 and QG.act_quant_mode(i8, 129) == 3
    assert QG.act_quant_mode(i4, 64) == 1 and QG.act_quant_mode(i4, 65) == 3
    assert QG.act_quant_mode(f8, 128) == 2 and QG.act_quant_mode(f8, 4096) == 4
    i8.adapters = {"a": (torch.zeros(4, 512), torch.zeros(256, 4))}
    assert QG.act_quant_mode(i8, 1) == 0          # a run-time adapter needs the 16-bit activations
    odd = LinearWeight.from_dense(torch.randn(64, 192) * 0.05, "int8")
    assert QG.act_quant_mode(odd, 1) == 0         # K not a multiple of the 128-wide quantisation block


def test_fp4_quantiser_roundtrip():
    """NVFP4 (block 16, e4m3-valued scales under a per-tensor factor) and MXFP4 (block 32, power-of-two scales): the packed
    form de-quantises to the nearest e2m1 grid point of every block, and agrees with the checkpoint de-quantisers."""
    import torch

    from fastllm_b200.loader import hf
    from fastllm_b200.ops import quant

    torch.manual_seed(0)
    w = torch.randn(32, 128) * 0.05
    for name, block in (("nvfp4", 16), ("mxfp4", 32)):
        lw = quant.LinearWeight.from_dense(w, name)
        assert lw.kind == "fp4" and lw.group == block and lw.w.shape == (32, 64) and lw.scale.shape == (32, 128 // block)
        dq = lw.dequant(torch.float32)
        rel = (dq - w).norm() / w.norm()
        assert rel < 0.12, (name, float(rel))
        # every de-quantised value is scale x an e2m1 value
        eff = lw.scale.float() * (lw.zero.float() if lw.zero is not None else 1.0)
        ratio = (dq.reshape(32, -1, block) / eff[..., None]).abs()
        grid = torch.tensor(quant._E2M1)
        assert ((ratio[..., None] - grid).abs().amin(-1) < 1e-4).all()
        # the checkpoint-format de-quantiser reads the same bytes the same way
        if block == 16:
            want = hf.dequant_nvfp4(lw.w, lw.scale.float().to(torch.float8_e4m3fn), lw.zero, torch.float32)
        else:
            e8 = (torch.log2(lw.scale.float()) + 127).to(torch.uint8)
            want = hf.dequant_mxfp4(lw.w.reshape(32, 128 // 32, 16), e8, torch.float32)
        assert torch.allclose(dq, want, rtol=1e-6, atol=1e-8)
    # values halfway between two grid points go to the even code
    codes = quant._fp4_codes(torch.tensor([0.25, 0.75, 1.25, 2.5, 5.0, -2.5]))
    assert codes.tolist() == [0, 2, 2, 4, 6, 12]


def test_awq_weights_keep_their_grid():
    """AWQ ``(q - zero) * scale`` weights, de-quantised in fp32, come back from the group-wise 4-bit quantiser on their own
    grid: the run-time weight de-quantises to exactly the checkpoint's values, also for groups that use only a few codes and
    after rows of several matrices are concatenated."""
    import torch

    from fastllm_b200.loader import hf
    from fastllm_b200.ops import quant

    torch.manual_seed(0)
    K, N, g = 256, 64, 128
    q = torch.randint(0, 16, (K, N))
    q[:g, 0] = torch.randint(3, 6, (g,))                     # a group that uses three neighbouring codes
    q[:g, 1] = torch.tensor([2, 9])[torch.randint(0, 2, (g,))]   # ... and one with a gap of seven steps
    z = torch.randint(0, 16, (K // g, N))
    sc = (torch.rand(K // g, N) * 0.02 + 0.001).half()
    order = hf._AWQ_ORDER
    pack = lambda t: sum((t[:, i::8].to(torch.int64) << (4 * order[i])) for i in range(8)).to(torch.int32)
    qweight, qzeros = pack(q), pack(z)
    dense = hf.dequant_awq(qweight, qzeros, sc, torch.float32)
    want = ((q.float() - z.float().repeat_interleave(g, 0)) * sc.float().repeat_interleave(g, 0)).t()
    assert torch.equal(dense, want)
    lw = quant.LinearWeight.from_dense(dense, "int4g128", act_dtype=torch.bfloat16)
    assert lw.kind == "int4g" and torch.allclose(lw.dequant(torch.float32), want, rtol=0, atol=1e-7)
    both = quant.LinearWeight.from_dense(torch.cat([dense, dense.flip(0)], dim=0), "int4g128", act_dtype=torch.bfloat16)
    assert torch.allclose(both.dequant(torch.float32), torch.cat([want, want.flip(0)], dim=0), rtol=0, atol=1e-7)
    # the same values rounded to bf16 first no longer sit on a grid: the min / max quantiser takes over (small error, not exact)
    lossy = quant.LinearWeight.from_dense(dense.bfloat16(), "int4g128")
    assert (lossy.dequant(torch.float32) - want).abs().max() > 0
