"""Vision tower and multimodal position tests (CPU): the tower against transformers' Qwen3.5 vision model, the interleaved
(time, row, column) rotary tables against transformers' text rotary embedding, patch ordering and image loading."""
import base64
import io

import pytest
import torch

from fastllm_b200.models import vision as V

transformers = pytest.importorskip("transformers")

_VC = dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, in_channels=3, patch_size=4, spatial_merge_size=2,
           temporal_patch_size=2, out_hidden_size=96, num_position_embeddings=64)


def _hf_vision():
    try:
        from transformers.models.qwen3_5 import modeling_qwen3_5 as M
        from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5VisionConfig
    except Exception as e:
        pytest.skip(f"transformers has no qwen3_5 vision model: {e}")
    torch.manual_seed(0)
    ref = M.Qwen3_5VisionModel(Qwen3_5VisionConfig(**_VC)).eval().float()
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(torch.randn_like(p) * 0.1)
    return ref


def test_vision_tower_matches_transformers():
    ref = _hf_vision()
    cfg = V.VisionConfig(_VC)
    tower = V.VisionTower(cfg, {k: v.detach() for k, v in ref.state_dict().items()}, "cpu", torch.float32)
    grids = [(1, 4, 6), (1, 8, 4)]
    n = sum(t * h * w for t, h, w in grids)
    patches = torch.randn(n, 3 * 2 * 4 * 4)
    with torch.no_grad():
        want = ref(patches, torch.tensor(grids)).pooler_output
    got = tower.forward(patches, grids)
    assert got.shape == want.shape == (n // 4, 96)
    assert (got - want).abs().max().item() < 2e-4


def test_patch_order_and_image_loading():
    cfg = V.VisionConfig(_VC)
    x = torch.arange(3 * 8 * 16, dtype=torch.float32).view(3, 8, 16)
    patches, grid = V.pixels_to_patches(x, cfg)
    assert grid == (1, 2, 4) and patches.shape == (8, 3 * 2 * 16)
    # patch 1 is the second patch of the first 2 x 2 block: rows 0..3, columns 4..7; both temporal slots hold the image
    p1 = patches[1].view(3, 2, 4, 4)
    assert torch.equal(p1[:, 0], x[:, 0:4, 4:8]) and torch.equal(p1[:, 1], x[:, 0:4, 4:8])
    # patch 2 is the block's lower-left patch, patch 4 starts the next block to the right
    assert torch.equal(patches[2].view(3, 2, 4, 4)[:, 0], x[:, 4:8, 0:4])
    assert torch.equal(patches[4].view(3, 2, 4, 4)[:, 0], x[:, 0:4, 8:12])
    from PIL import Image

    img = Image.new("RGB", (30, 17), (255, 0, 128))
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    pt, g = V.image_to_patches(url, cfg, min_pixels=64, max_pixels=4096)
    assert g[1] % 2 == 0 and g[2] % 2 == 0 and pt.shape == (g[1] * g[2], 96)
    assert abs(float(pt.view(-1, 3, 2, 16)[:, 0].mean()) - 1.0) < 1e-5 and abs(float(pt.view(-1, 3, 2, 16)[:, 1].mean()) + 1.0) < 1e-5
    assert V.smart_resize(17, 30, 8, 64, 4096) == (16, 32)


def test_mrope_positions_and_tables():
    img = 9
    ids = [1, 2, img, img, img, img, img, img, 3, 4]           # one image: grid 1 x 4 x 6 patches -> 2 x 3 tokens
    pos, delta = V.mrope_positions(ids, img, [(1, 4, 6)], 2)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8:].tolist() == [[5, 6]] * 3 and delta == 7 - 10
    try:
        from transformers.models.qwen3_5 import modeling_qwen3_5 as M
        from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    except Exception as e:
        pytest.skip(f"transformers has no qwen3_5: {e}")
    tc = Qwen3_5TextConfig(hidden_size=64, num_attention_heads=2, num_key_value_heads=1, head_dim=32, num_hidden_layers=1,
                           rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 1.0,
                                            "mrope_section": [6, 5, 5], "mrope_interleaved": True})
    rot = M.Qwen3_5TextRotaryEmbedding(tc)
    cos_w, sin_w = rot(torch.zeros(1, 1, 32), pos[:, None, :])
    cos, sin = V.mrope_tables(pos, 32, 10000.0, [6, 5, 5])
    assert torch.allclose(cos, cos_w[0, :, :16], atol=1e-5) and torch.allclose(sin, sin_w[0, :, :16], atol=1e-5)


def test_qwen3_5_image_prompt_matches_transformers(tmp_path):
    """A prompt with an image through the whole path -- checkpoint with ``visual.*`` weights, image -> patches -> tower,
    placeholder expansion, embeddings in place of the image tokens, (time, row, column) rotary positions in the full-attention
    layers, chunked prefill and decode -- against transformers' Qwen3.5 conditional-generation model."""
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.loader import hf

    try:
        from transformers import Qwen3_5Config, Qwen3_5ForConditionalGeneration
    except Exception as e:
        pytest.skip(f"transformers has no qwen3_5: {e}")
    torch.manual_seed(0)
    text = dict(vocab_size=512, hidden_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                intermediate_size=128, max_position_embeddings=512, linear_num_key_heads=2, linear_num_value_heads=4,
                linear_key_head_dim=16, linear_value_head_dim=16, layer_types=["linear_attention", "full_attention"],
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                                 "mrope_section": [3, 3, 2], "mrope_interleaved": True})
    cfg = Qwen3_5Config(text_config=text, vision_config=_VC, image_token_id=500, video_token_id=501, vision_start_token_id=502,
                        vision_end_token_id=503)
    ref = Qwen3_5ForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() >= 2:
                torch.nn.init.normal_(p, std=0.08)
    d = str(tmp_path / "q35vl")
    ref.save_pretrained(d, safe_serialization=True)
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    assert getattr(m, "vision", None) is not None and m.image_token_id == 500
    from PIL import Image

    g = torch.Generator().manual_seed(1)
    img = Image.fromarray((torch.rand(40, 56, 3, generator=g) * 255).to(torch.uint8).numpy())
    ids = [5, 6, 7, 502, 500, 503, 8, 9, 10, 11]
    ids2, mm = V.build_context(m, ids, [img], min_pixels=64, max_pixels=2048)
    n_img = ids2.count(500)
    patches, grid = V.image_to_patches(img, m.vision.cfg, min_pixels=64, max_pixels=2048)
    assert n_img == grid[1] * grid[2] // 4 and n_img > 4 and mm.embeds.shape == (n_img, 96)
    with torch.no_grad():
        out = ref(input_ids=torch.tensor([ids2]), pixel_values=patches, image_grid_thw=torch.tensor([grid]),
                  mm_token_type_ids=torch.tensor([[1 if t == 500 else 0 for t in ids2]]))
    want = out.logits[0, -1].float()
    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512, chunked_prefill_size=16), num_pages=8)
    h = eng.launch(ids2, GenerationConfig(max_new_tokens=3, ignore_eos=True), mm=mm)
    req = eng.requests[h]
    while not req.finished():
        eng.step()
    assert int(req.output_ids[0]) == int(want.argmax())
    # the second token: transformers continues from the 3-D positions (rope delta), one-shot over the longer prompt
    ids3 = ids2 + [int(req.output_ids[0])]
    with torch.no_grad():
        out2 = ref(input_ids=torch.tensor([ids3]), pixel_values=patches, image_grid_thw=torch.tensor([grid]),
                   mm_token_type_ids=torch.tensor([[1 if t == 500 else 0 for t in ids3]]))
    assert int(req.output_ids[1]) == int(out2.logits[0, -1].argmax())
    # logits of the one-shot prefill
    pages = [0, 1]
    lg = eng.runner.prefill([(ids2, 0, pages, True, 0, mm)])[0].float()
    assert torch.nn.functional.cosine_similarity(lg[:want.numel()], want, dim=0).item() > 0.9999


def test_image_parts_of_chat_messages():
    """OpenAI ``image_url`` / Responses ``input_image`` / Qwen ``image`` content parts become the placeholder markup, the
    images are returned in prompt order; the server's prompt builder hands them on with the token ids."""
    from fastllm_b200.serving.completion import Completion, PromptIds

    msgs = [{"role": "system", "content": "s"},
            {"role": "user", "content": [{"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}},
                                         {"type": "text", "text": "what is this?"}, {"type": "image", "image": "/tmp/x.png"}]},
            {"role": "assistant", "content": "a"}, {"role": "user", "content": [{"type": "input_image", "image_url": "file:///y.jpg"}]}]
    out, images = V.extract_images(msgs)
    assert images == ["data:image/png;base64,AAAA", "/tmp/x.png", "file:///y.jpg"]
    assert out[1]["content"] == V.IMAGE_MARKER + "what is this?" + V.IMAGE_MARKER and out[3]["content"] == V.IMAGE_MARKER
    assert out[0]["content"] == "s" and out[2]["content"] == "a"

    class _TM:
        vision = object()

    class _M:
        torch_model = _TM()

        def apply_chat_template(self, messages, add_generation_prompt=True, tools=None, **kw):
            return "|".join(m["content"] for m in messages)

        def encode(self, text):
            return [len(text), 7]

    ids, text = Completion(_M()).build_prompt_ids(messages=msgs)
    assert isinstance(ids, PromptIds) and ids.images == images and V.IMAGE_MARKER in text and list(ids) == [len(text), 7]


def test_llm_model_answers_about_an_image(tmp_path):
    """``llm.model(...).response(messages with an image_url part)``: chat template, special-token ids of the placeholder
    markup, placeholder expansion, tower, engine -- the generated tokens equal transformers' greedy continuation of the same
    expanded prompt with the same patches."""
    import base64
    import io
    import json

    from fastllm_b200 import llm

    try:
        from transformers import Qwen3_5Config, Qwen3_5ForConditionalGeneration
    except Exception as e:
        pytest.skip(f"transformers has no qwen3_5: {e}")
    import sys

    sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parent.parent))
    from baseline import synth

    torch.manual_seed(0)
    text = dict(vocab_size=512, hidden_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                intermediate_size=128, max_position_embeddings=512, linear_num_key_heads=2, linear_num_value_heads=4,
                linear_key_head_dim=16, linear_value_head_dim=16, layer_types=["linear_attention", "full_attention"],
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                                 "mrope_section": [3, 3, 2], "mrope_interleaved": True})
    cfg = Qwen3_5Config(text_config=text, vision_config=_VC, image_token_id=257, video_token_id=260, vision_start_token_id=258,
                        vision_end_token_id=259, eos_token_id=256)
    ref = Qwen3_5ForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() >= 2:
                torch.nn.init.normal_(p, std=0.08)
    d = tmp_path / "q35vl"
    ref.save_pretrained(str(d), safe_serialization=True)
    synth.write_tokenizer(d, 256)
    tk = json.loads((d / "tokenizer.json").read_text())
    for tid, name in ((257, "<|image_pad|>"), (258, "<|vision_start|>"), (259, "<|vision_end|>"), (260, "<|video_pad|>")):
        tk["added_tokens"].append({"id": tid, "content": name, "single_word": False, "lstrip": False, "rstrip": False,
                                   "normalized": False, "special": True})
    (d / "tokenizer.json").write_text(json.dumps(tk))
    (d / "preprocessor_config.json").write_text(json.dumps({"image_mean": [0.5, 0.5, 0.5], "image_std": [0.5, 0.5, 0.5],
                                                           "size": {"shortest_edge": 64, "longest_edge": 2048}}))
    from PIL import Image

    g = torch.Generator().manual_seed(1)
    img = Image.fromarray((torch.rand(40, 56, 3, generator=g) * 255).to(torch.uint8).numpy())
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    model = llm.model(str(d), device="cpu", dtype="float32")
    try:
        assert model.torch_model.vision is not None and model._image_options["max_pixels"] == 2048
        msgs = [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}}, {"type": "text", "text": "hi"}]}]
        h = model.launch_stream_response(msgs, max_length=4, do_sample=False)
        req = model.engine.requests[h]
        toks = []
        while (t := model.engine.fetch(h)) >= 0:
            toks.append(t)
        ids2 = req.prompt_ids
        n_img = ids2.count(257)
        i0 = ids2.index(257)
        assert n_img > 4 and ids2[i0 - 1] == 258 and ids2[i0 + n_img] == 259 and req.mm is not None
        patches, grid = V.image_to_patches(img, model.torch_model.vision.cfg, min_pixels=64, max_pixels=2048)
        assert n_img == grid[1] * grid[2] // 4
        with torch.no_grad():
            out = ref(input_ids=torch.tensor([ids2]), pixel_values=patches, image_grid_thw=torch.tensor([grid]),
                      mm_token_type_ids=torch.tensor([[1 if t == 257 else 0 for t in ids2]]))
        assert toks and toks[0] == int(out.logits[0, -1].argmax())
        # a video part: frames sampled and grouped, one time stamp + placeholder run per group in the rendered prompt
        clip = [Image.fromarray((torch.rand(40, 56, 3, generator=g) * 255).to(torch.uint8).numpy()) for _ in range(4)]
        vmsgs = [{"role": "user", "content": [{"type": "video", "video": {"frames": clip, "fps": 2.0}}, {"type": "text", "text": "hi"}]}]
        h = model.launch_stream_response(vmsgs, max_length=3, do_sample=False)
        req = model.engine.requests[h]
        vt = []
        while (t := model.engine.fetch(h)) >= 0:
            vt.append(t)
        ids3 = req.prompt_ids
        groups = V.frames_to_patches(clip, [0.0, 0.5, 1.0, 1.5], model.torch_model.vision.cfg, min_pixels=64, max_pixels=2048)
        per = groups[0][1][1] * groups[0][1][2] // 4
        assert ids3.count(260) == 2 * per and ids3.count(258) == 2 and req.mm is not None
        with torch.no_grad():
            out = ref(input_ids=torch.tensor([ids3]), pixel_values_videos=torch.cat([p for p, _g, _t in groups]),
                      video_grid_thw=torch.tensor([[2, groups[0][1][1], groups[0][1][2]]]),
                      mm_token_type_ids=torch.tensor([[2 if t == 260 else 0 for t in ids3]]))
        assert vt and vt[0] == int(out.logits[0, -1].argmax())
    finally:
        model.shutdown() if hasattr(model, "shutdown") else None


def test_qwen3_5_video_prompt_matches_transformers(tmp_path):
    """A prompt with a video: frames in temporal groups (two frames per group fill the tower's temporal patch), one placeholder
    run per group with text between the runs, every group laid out on its own (row, column) grid -- against transformers'
    Qwen3.5 model given the same frames as one ``(t, h, w)`` video grid.  Also frame loading / sampling and the markup."""
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.loader import hf

    try:
        from transformers import Qwen3_5Config, Qwen3_5ForConditionalGeneration
    except Exception as e:
        pytest.skip(f"transformers has no qwen3_5: {e}")
    torch.manual_seed(0)
    text = dict(vocab_size=512, hidden_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                intermediate_size=128, max_position_embeddings=512, linear_num_key_heads=2, linear_num_value_heads=4,
                linear_key_head_dim=16, linear_value_head_dim=16, layer_types=["linear_attention", "full_attention"],
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                                 "mrope_section": [3, 3, 2], "mrope_interleaved": True})
    cfg = Qwen3_5Config(text_config=text, vision_config=_VC, image_token_id=500, video_token_id=501, vision_start_token_id=502,
                        vision_end_token_id=503)
    ref = Qwen3_5ForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() >= 2:
                torch.nn.init.normal_(p, std=0.08)
    d = str(tmp_path / "q35vid")
    ref.save_pretrained(d, safe_serialization=True)
    m = hf.load_model(d, device="cpu", dtype=torch.float32)
    assert m.video_token_id == 501
    from PIL import Image

    g = torch.Generator().manual_seed(2)
    clip = [Image.fromarray((torch.rand(24, 32, 3, generator=g) * 255).to(torch.uint8).numpy()) for _ in range(7)]
    frames, times = V.load_video({"frames": clip, "fps": 4.0}, target_fps=2.0, min_frames=2)
    assert len(frames) == 4 and times == [0.0, 0.5, 1.0, 1.5]
    groups = V.frames_to_patches(frames, times, m.vision.cfg, min_pixels=64, max_pixels=2048)
    assert len(groups) == 2 and groups[0][1][0] == 1 and abs(groups[1][2] - 1.25) < 1e-6
    assert V.video_markup(groups) == "<0.2 seconds>" + V.VIDEO_MARKER + "<1.2 seconds>" + V.VIDEO_MARKER
    gh, gw = groups[0][1][1:]
    ids = [5, 6, 7, 20, 21, 502, 501, 503, 22, 23, 502, 501, 503, 8, 9, 10]
    ids2, mm = V.build_context(m, ids, [], videos=[groups])
    n = gh * gw // 4
    assert ids2.count(501) == 2 * n and mm.embeds.shape == (2 * n, 96)
    with torch.no_grad():
        out = ref(input_ids=torch.tensor([ids2]), pixel_values_videos=torch.cat([p for p, _g, _t in groups]),
                  video_grid_thw=torch.tensor([[2, gh, gw]]), mm_token_type_ids=torch.tensor([[2 if t == 501 else 0 for t in ids2]]))
    want = out.logits[0, -1].float()
    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512, chunked_prefill_size=16), num_pages=8)
    h = eng.launch(ids2, GenerationConfig(max_new_tokens=2, ignore_eos=True), mm=mm)
    req = eng.requests[h]
    while not req.finished():
        eng.step()
    assert int(req.output_ids[0]) == int(want.argmax())
    lg = eng.runner.prefill([(ids2, 0, [0, 1], True, 0, mm)])[0].float()
    assert torch.nn.functional.cosine_similarity(lg[:want.numel()], want, dim=0).item() > 0.9999
    # message parts: a video part leaves a slot that the expansion fills with the groups' markup
    vids = []
    msgs, imgs = V.extract_images([{"role": "user", "content": [{"type": "video", "video": {"frames": clip, "fps": 4.0}},
                                                                 {"type": "text", "text": "what happens?"}]}], vids)
    assert not imgs and len(vids) == 1 and msgs[0]["content"] == V.video_slot(0) + "what happens?"
    with pytest.raises(ValueError):
        V.extract_images([{"role": "user", "content": [{"type": "video_url", "video_url": {"url": "x.gif"}}]}])
