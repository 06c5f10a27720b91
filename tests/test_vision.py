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
