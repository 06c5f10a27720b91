"""GGUF loader: block de-quantisation against the ``gguf`` package's own tables, and a tiny llama written as GGUF
(llama.cpp tensor names, permuted Q/K rows) generating the same tokens as the Hugging Face folder it came from."""
import numpy as np
import pytest
import torch

from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
from fastllm_b200.loader import gguf as G
from fastllm_b200.loader import hf

ggufpkg = pytest.importorskip("gguf")


@pytest.mark.parametrize("t", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1"])
def test_simple_blocks_match_package(t):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 256)).astype(np.float32)
    qt = getattr(ggufpkg.GGMLQuantizationType, t)
    q = ggufpkg.quants.quantize(x, qt)
    ref = ggufpkg.quants.dequantize(q, qt).reshape(-1)
    mine = G.dequantize(np.ascontiguousarray(q).view(np.uint8).reshape(-1), t, x.size)
    assert np.array_equal(mine, ref)


@pytest.mark.parametrize("t,scale_offsets", [("Q2_K", (80, 82)), ("Q3_K", (108,)), ("Q4_K", (0, 2)), ("Q5_K", (0, 2)), ("Q6_K", (208,))])
def test_k_blocks_match_package(t, scale_offsets):
    rng = np.random.default_rng(1)
    per, nbytes = next((p, b) for _, (n, p, b) in G.GGML_TYPES.items() if n == t)
    nb = 8
    raw = rng.integers(0, 256, size=(nb, nbytes), dtype=np.uint8)
    for off in scale_offsets:       # finite fp16 super-block scales
        raw[:, off:off + 2] = np.frombuffer(rng.uniform(0.01, 1, size=nb).astype("<f2").tobytes(), dtype=np.uint8).reshape(nb, 2)
    ref = ggufpkg.quants.dequantize(raw, getattr(ggufpkg.GGMLQuantizationType, t)).reshape(-1)
    assert np.array_equal(G.dequantize(raw.reshape(-1), t, nb * per), ref)


def _permute(w, n_head):      # what llama.cpp's converter does to llama Q/K rows
    return w.reshape(n_head, 2, w.shape[0] // n_head // 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)


def test_tiny_llama_gguf_generates_same_tokens(tmp_path):
    from baseline import synth
    from fastllm_b200.loader.safetensors import SafeTensorFile

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    ref = hf.load_model(d, device="cpu", dtype=torch.float32)
    cfg = ref.cfg
    sd = {}
    import glob
    for f in glob.glob(d + "/*.safetensors"):
        st = SafeTensorFile(f)
        sd.update({k: st.get(k).clone() for k in st.keys()})
        st.close()
    out = str(tmp_path / "m.gguf")
    w = ggufpkg.GGUFWriter(out, "llama")
    w.add_block_count(cfg.num_layers)
    w.add_embedding_length(cfg.hidden_size)
    w.add_head_count(cfg.num_heads)
    w.add_head_count_kv(cfg.num_kv_heads)
    w.add_key_length(cfg.head_dim)
    w.add_value_length(cfg.head_dim)
    w.add_feed_forward_length(cfg.intermediate_size)
    w.add_layer_norm_rms_eps(cfg.rms_eps)
    w.add_rope_freq_base(cfg.rope_theta)
    w.add_context_length(cfg.max_position)
    w.add_vocab_size(cfg.vocab_size)
    inv_top = {v: k for k, v in G._TOP.items()}
    inv_blk = {v: k for k, v in G._BLK.items()}
    for name, t in sd.items():
        a = t.float().numpy()
        if name in inv_top:
            w.add_tensor(inv_top[name], a)
            continue
        _, _, idx, rest = name.split(".", 3)
        if rest == "self_attn.q_proj.weight":
            a = _permute(a, cfg.num_heads)
        if rest == "self_attn.k_proj.weight":
            a = _permute(a, cfg.num_kv_heads)
        # projections as Q8_0 blocks, norms as fp32
        if a.ndim == 2:
            q = ggufpkg.quants.quantize(a, ggufpkg.GGMLQuantizationType.Q8_0)
            w.add_tensor(f"blk.{idx}.{inv_blk[rest]}", q, raw_shape=q.shape, raw_dtype=ggufpkg.GGMLQuantizationType.Q8_0)
        else:
            w.add_tensor(f"blk.{idx}.{inv_blk[rest]}", a)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    f = G.GGUFFile(out)
    assert f.meta["general.architecture"] == "llama" and f.meta["llama.block_count"] == cfg.num_layers
    got = G.load_model(out, device="cpu", dtype=torch.float32)
    assert got.cfg.num_kv_heads == cfg.num_kv_heads and got.cfg.hidden_size == cfg.hidden_size
    prompt = list(range(3, 60, 2))
    res = []
    for m in (ref, got):
        eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512), num_pages=8)
        res.append(eng.generate([prompt], GenerationConfig(max_new_tokens=6, ignore_eos=True))[0])
    # Q8_0 perturbs the weights slightly: the first tokens of a greedy run still agree
    assert res[0][:3] == res[1][:3]
