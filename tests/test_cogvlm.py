"""CogVLM (visual-expert decoder behind an EVA-CLIP tower): a checkpoint in the family's own naming, loaded through
``llm.model`` and served by the paged engine, against a plain full-sequence evaluation of the model's definition written here
(token types, expert mask, position ids as in the model's published modelling code)."""
import json
import math

import torch
import torch.nn.functional as F

H, LAYERS, HEADS, INTER, VOCAB = 64, 2, 4, 128, 300
VC = dict(hidden_size=32, num_heads=2, num_hidden_layers=2, patch_size=4, image_size=32, in_channels=3, intermediate_size=64,
          layer_norm_eps=1e-6, num_positions=65)
EPS = 1e-5


def _weights():
    g = torch.Generator().manual_seed(0)
    r = lambda *s, std=0.08: torch.randn(*s, generator=g) * std
    w = {"model.embed_tokens.weight": r(VOCAB, H, std=0.5), "model.norm.weight": 1 + r(H), "lm_head.weight": r(VOCAB, H, std=0.2)}
    for i in range(LAYERS):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = 1 + r(H)
        w[p + "post_attention_layernorm.weight"] = 1 + r(H)
        for e in ("language", "vision"):
            w[p + f"self_attn.{e}_expert_query_key_value.weight"] = r(3 * H, H, std=0.15)
            w[p + f"self_attn.{e}_expert_dense.weight"] = r(H, H, std=0.15)
            m = "language_mlp" if e == "language" else "vision_mlp"
            w[p + f"mlp.{m}.gate_proj.weight"] = r(INTER, H, std=0.15)
            w[p + f"mlp.{m}.up_proj.weight"] = r(INTER, H, std=0.15)
            w[p + f"mlp.{m}.down_proj.weight"] = r(H, INTER, std=0.15)
    v, Hv = "model.vision.", VC["hidden_size"]
    w[v + "patch_embedding.proj.weight"] = r(Hv, 3, 4, 4, std=0.2)
    w[v + "patch_embedding.proj.bias"] = r(Hv)
    w[v + "patch_embedding.cls_embedding"] = r(1, Hv, std=0.3)
    w[v + "patch_embedding.position_embedding.weight"] = r(VC["num_positions"], Hv, std=0.3)
    for i in range(VC["num_hidden_layers"]):
        p = v + f"transformer.layers.{i}."
        for name, shape in (("attention.query_key_value", (3 * Hv, Hv)), ("attention.dense", (Hv, Hv)), ("mlp.fc1", (64, Hv)), ("mlp.fc2", (Hv, 64))):
            w[p + name + ".weight"] = r(*shape, std=0.2)
            w[p + name + ".bias"] = r(shape[0])
        for name in ("input_layernorm", "post_attention_layernorm"):
            w[p + name + ".weight"] = 1 + r(Hv)
            w[p + name + ".bias"] = r(Hv)
    w[v + "conv.weight"] = r(Hv, Hv, 2, 2, std=0.2)
    w[v + "conv.bias"] = r(Hv)
    w[v + "linear_proj.linear_proj.weight"] = r(H, Hv, std=0.3)
    w[v + "linear_proj.norm1.weight"] = 1 + r(H)
    w[v + "linear_proj.norm1.bias"] = r(H)
    w[v + "linear_proj.gate_proj.weight"] = r(INTER, H, std=0.2)
    w[v + "linear_proj.dense_h_to_4h.weight"] = r(INTER, H, std=0.2)
    w[v + "linear_proj.dense_4h_to_h.weight"] = r(H, INTER, std=0.2)
    w[v + "boi"] = r(1, 1, H, std=0.5)
    w[v + "eoi"] = r(1, 1, H, std=0.5)
    return w


def _ref_vision(w, px):
    v, Hv, nh = "model.vision.", VC["hidden_size"], VC["num_heads"]
    x = F.conv2d(px[None], w[v + "patch_embedding.proj.weight"], w[v + "patch_embedding.proj.bias"], stride=4).flatten(2).transpose(1, 2)
    x = torch.cat([w[v + "patch_embedding.cls_embedding"][None], x], 1) + w[v + "patch_embedding.position_embedding.weight"][None]
    L = x.shape[1]
    for i in range(VC["num_hidden_layers"]):
        p = v + f"transformer.layers.{i}."
        qkv = F.linear(x, w[p + "attention.query_key_value.weight"], w[p + "attention.query_key_value.bias"]).reshape(1, L, 3, nh, Hv // nh)
        q, k, vv = qkv.permute(2, 0, 3, 1, 4)
        a = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(Hv // nh), -1) @ vv
        a = F.linear(a.transpose(1, 2).reshape(1, L, Hv), w[p + "attention.dense.weight"], w[p + "attention.dense.bias"])
        x = x + F.layer_norm(a, (Hv,), w[p + "input_layernorm.weight"], w[p + "input_layernorm.bias"], 1e-6)
        m = F.linear(F.gelu(F.linear(x, w[p + "mlp.fc1.weight"], w[p + "mlp.fc1.bias"])), w[p + "mlp.fc2.weight"], w[p + "mlp.fc2.bias"])
        x = x + F.layer_norm(m, (Hv,), w[p + "post_attention_layernorm.weight"], w[p + "post_attention_layernorm.bias"], 1e-6)
    x = x[:, 1:].reshape(1, 8, 8, Hv).permute(0, 3, 1, 2)
    x = F.conv2d(x, w[v + "conv.weight"], w[v + "conv.bias"], stride=2).flatten(2).transpose(1, 2)
    y = F.gelu(F.layer_norm(F.linear(x, w[v + "linear_proj.linear_proj.weight"]), (H,), w[v + "linear_proj.norm1.weight"], w[v + "linear_proj.norm1.bias"], 1e-5))
    y = F.linear(F.silu(F.linear(y, w[v + "linear_proj.gate_proj.weight"])) * F.linear(y, w[v + "linear_proj.dense_h_to_4h.weight"]),
                 w[v + "linear_proj.dense_4h_to_h.weight"])
    return torch.cat([w[v + "boi"], y, w[v + "eoi"]], 1)[0]


def _ref_logits(w, text_ids, image_rows):
    """Logits of every position of ``[bos] image text[1:]`` (model definition: token types -> expert mask and position ids)."""
    V = image_rows.shape[0]
    emb = w["model.embed_tokens.weight"]
    x = torch.cat([emb[text_ids[:1]], image_rows, emb[text_ids[1:]]], 0)
    T = x.shape[0]
    tt = torch.zeros(T, dtype=torch.long)
    tt[1:1 + V] = 1
    vmask = torch.zeros(T, dtype=torch.bool)
    vmask[:-1] = (tt[:-1] == 1) & (tt[1:] == 1)
    tmp = tt.clone()
    edge = torch.zeros(T, dtype=torch.bool)
    edge[1:] |= (tmp[1:] == 1) & (tmp[:-1] == 0)
    edge[0] |= tmp[0] == 1
    edge[:-1] |= (tmp[:-1] == 1) & (tmp[1:] == 0)
    edge[-1] |= tmp[-1] == 1
    tmp[edge] = 0
    y = torch.zeros(T, dtype=torch.long)
    y[1:] = ((tmp[1:] == 0) | ((tmp[1:] == 1) & (tmp[:-1] == 0))).long()
    pos = y.cumsum(0)
    D = H // HEADS
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = pos[:, None].float() * inv[None]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
    rot = lambda t: torch.cat([-t[..., D // 2:], t[..., :D // 2]], -1)
    rms = lambda t, g: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + EPS) * g
    pick = lambda t, lang, vis: torch.where(vmask[:, None], F.linear(t, w[vis]), F.linear(t, w[lang]))
    causal = torch.ones(T, T).tril().bool()
    for i in range(LAYERS):
        p = f"model.layers.{i}."
        h = rms(x, w[p + "input_layernorm.weight"])
        qkv = pick(h, p + "self_attn.language_expert_query_key_value.weight", p + "self_attn.vision_expert_query_key_value.weight")
        q, k, v = [t.reshape(T, HEADS, D) for t in qkv.split(H, -1)]
        q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s.masked_fill(~causal, float("-inf")), -1), v).reshape(T, H)
        x = x + pick(a, p + "self_attn.language_expert_dense.weight", p + "self_attn.vision_expert_dense.weight")
        h = rms(x, w[p + "post_attention_layernorm.weight"])
        mlp = lambda m: F.linear(F.silu(F.linear(h, w[p + f"mlp.{m}.gate_proj.weight"])) * F.linear(h, w[p + f"mlp.{m}.up_proj.weight"]),
                                 w[p + f"mlp.{m}.down_proj.weight"])
        x = x + torch.where(vmask[:, None], mlp("vision_mlp"), mlp("language_mlp"))
    return F.linear(rms(x, w["model.norm.weight"]), w["lm_head.weight"])


def test_cogvlm_checkpoint_matches_model_definition(tmp_path):
    from fastllm_b200 import llm
    from fastllm_b200.models import cogvlm

    w = _weights()
    d = tmp_path / "cogvlm"
    _write_folder(d, w)
    g = torch.Generator().manual_seed(3)
    image = torch.rand(3, 32, 32, generator=g)
    text = [1] + torch.randint(3, VOCAB, (9,), generator=g).tolist()

    rows = _ref_vision(w, cogvlm.preprocess(image, 32))
    assert rows.shape == (18, H)
    seq = list(text)
    want = []
    for _ in range(6):
        nxt = int(_ref_logits(w, torch.tensor(seq), rows)[-1].argmax())
        want.append(nxt)
        seq.append(nxt)

    pos, delta = cogvlm.positions_for(len(text) + 18, 18)
    assert pos.tolist()[:3] == [0, 1, 2] and pos.tolist()[17:20] == [2, 3, 4] and delta == -15

    llm.set_device_map("cpu")
    model = llm.model(str(d), device="cpu", dtype="float32")
    try:
        tm = model.torch_model
        assert type(tm).__name__ == "CogVLMModel" and tm.vision is not None and len(tm.vexp) == LAYERS
        got_rows = tm.vision.forward(cogvlm.preprocess(image, 32)[None])[0]
        assert torch.allclose(got_rows, rows, atol=2e-4, rtol=1e-4)
        h = model.launch_stream_response(text, images=[image], max_length=6, do_sample=False, stop_token_ids=[])
        got = []
        while True:
            t = model.engine.fetch(h)
            if t < 0:
                break
            got.append(t)
        assert got == want
        # a text-only request on the same model takes the ordinary decoder path (language expert everywhere)
        out = list(model.stream_response_raw(text, max_length=3, do_sample=False))
        assert len(out) >= 1
    finally:
        model.release_memory()


def _write_folder(d, w):
    import sys

    sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parent.parent))
    from baseline import synth
    from fastllm_b200.loader.safetensors import save_file

    d.mkdir()
    save_file({k: v.contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps(dict(
        architectures=["CogVLMForCausalLM"], vocab_size=VOCAB, hidden_size=H, num_hidden_layers=LAYERS, num_attention_heads=HEADS,
        intermediate_size=INTER, rms_norm_eps=EPS, max_position_embeddings=512, bos_token_id=1, eos_token_id=2, pad_token_id=0,
        torch_dtype="float32", vision_config=VC)))
    synth.write_tokenizer(d, 256)


@__import__("pytest").mark.gpu
def test_cogvlm_on_gpu(tmp_path, monkeypatch):
    """The mixed-expert prefill on the GPU (bf16 linear kernels, paged pools) against the model definition in fp32, then decode
    steps through the ordinary kernels."""
    import sys

    from fastllm_b200 import llm
    from fastllm_b200.models import cogvlm
    from fastllm_b200.ops import _lib

    me = sys.modules[__name__]
    monkeypatch.setattr(me, "H", 256)
    monkeypatch.setattr(me, "HEADS", 2)
    monkeypatch.setattr(me, "INTER", 256)
    w = _weights()
    w = {k: (v * 0.5 if v.dim() >= 2 and "layernorm" not in k else v) for k, v in w.items()}
    _write_folder(tmp_path / "cogvlm_gpu", w)
    g = torch.Generator().manual_seed(3)
    image = torch.rand(3, 32, 32, generator=g)
    text = [1] + torch.randint(3, VOCAB, (9,), generator=g).tolist()
    rows = _ref_vision(w, cogvlm.preprocess(image, 32))
    want = _ref_logits(w, torch.tensor(text), rows)[-1]

    model = llm.model(str(tmp_path / "cogvlm_gpu"), device="cuda", dtype="bfloat16")
    try:
        tm = model.torch_model
        ids, mm = cogvlm.build_context(tm, text, [image])
        model.engine.start()
        got = model.engine.runner.prefill([(ids, 0, [0], True, 0, mm)])[0].float().cpu()
        _lib.check_device_errors()
        cs = torch.nn.functional.cosine_similarity(got, want, dim=0).item()
        assert cs > 0.99, cs
        out = []
        h = model.launch_stream_response(text, images=[image], max_length=5, do_sample=False, stop_token_ids=[])
        while True:
            t = model.engine.fetch(h)
            if t < 0:
                break
            out.append(t)
        assert len(out) == 5
        _lib.check_device_errors()
    finally:
        model.release_memory()
