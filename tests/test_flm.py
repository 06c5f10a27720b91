""".flm format: golden bytes of the header / tensor records, round trip through every storage dtype, and a model
exported to .flm generating the same tokens as the HF folder it came from."""
import struct

import pytest
import torch

from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
from fastllm_b200.loader import flm, hf


def test_golden_bytes(tmp_path):
    p = tmp_path / "g.flm"
    t = torch.tensor([[1.0, -2.0], [0.5, 4.0]])
    flm.write_flm(p, {"model_type": "llama"}, [(b"ab", 0, 1.0)], [], [("x.bias", t[0])], "float16")
    b = p.read_bytes()
    pos = 0

    def i32():
        nonlocal pos
        v = struct.unpack_from("<i", b, pos)[0]
        pos += 4
        return v

    def s():
        nonlocal pos
        n = i32()
        v = b[pos:pos + n]
        pos += n
        return v

    assert i32() == 2                       # version
    n = i32()
    kv = {s(): s() for _ in range(n)}
    assert kv[b"model_type"] == b"llama" and kv[b"tokenizer_use_score"] == b"1"
    assert i32() == 1                       # vocab length
    assert i32() == 2 and i32() == ord("a") and i32() == ord("b") and i32() == 0
    assert struct.unpack_from("<f", b, pos)[0] == 1.0
    pos += 4
    assert i32() == 1                       # tensors
    assert s() == b"x.bias" and i32() == 1 and i32() == 2 and i32() == flm.FLOAT32
    assert struct.unpack_from("<2f", b, pos) == (1.0, -2.0)


@pytest.mark.parametrize("dtype,tol", [("float32", 0), ("float16", 2e-3), ("bfloat16", 2e-2), ("int8", 0.02), ("int4g128", 0.3), ("int4", 0.45)])
def test_tensor_roundtrip(tmp_path, dtype, tol):
    torch.manual_seed(0)
    w = torch.randn(16, 256)
    p = tmp_path / "t.flm"
    flm.write_flm(p, {}, [], [], [("layer.q_proj.weight", w)], dtype)
    _, _, tensors = flm.read_flm(p)
    assert (tensors["layer.q_proj.weight"].float() - w).abs().max().item() <= tol


def test_int4_high_nibble_first(tmp_path):
    w = torch.tensor([[0.0, 15.0] * 64])
    p = tmp_path / "n.flm"
    flm.write_flm(p, {}, [], [], [("a.q_proj.weight", w)], "int4g128")
    data = p.read_bytes()
    assert data[-64] == 0x0F               # first value (0) high nibble, second (15) low nibble


def test_export_and_reload_generates_same_tokens(tmp_path):
    from baseline import synth

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    out = tmp_path / "m.flm"
    flm.export_hf_to_flm(d, str(out), "float32")
    prompt = list(range(3, 90, 2))
    res = []
    for m in (hf.load_model(d, device="cpu", dtype=torch.float32), flm.load_model(str(out), device="cpu", dtype=torch.float32)):
        eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=512), num_pages=8)
        res.append(eng.generate([prompt], GenerationConfig(max_new_tokens=6, ignore_eos=True))[0])
    assert res[0] == res[1]
