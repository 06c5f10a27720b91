"""Native CPU backend against the plain PyTorch definition of every operator (both ISA builds run where the host has them)."""
import ctypes
import os

import pytest
import torch

from fastllm_b200.ops import attention as A
from fastllm_b200.ops import cpu, quant

pytestmark = pytest.mark.skipif(not cpu.available(), reason="libfb_cpu.so not built")


@pytest.mark.parametrize("M,N,K", [(1, 96, 256), (3, 130, 192), (9, 257, 136), (33, 64, 1024)])
@pytest.mark.parametrize("wd", [torch.float32, torch.bfloat16, torch.float16])
def test_linear_dense(M, N, K, wd):
    torch.manual_seed(0)
    x = torch.randn(M, K)
    w = (torch.randn(N, K) * 0.1).to(wd)
    b = torch.randn(N)
    ref = x @ w.float().t() + b
    got = cpu.linear(x, w, b)
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-4)


@pytest.mark.parametrize("M", [1, 5, 16])
def test_linear_int8_int4g(M):
    torch.manual_seed(1)
    x = torch.randn(M, 512)
    w = torch.randn(200, 512) * 0.05
    q, s, z = quant.quantize_int8(w)
    ref = x @ quant.dequantize_int8(q, s, z, torch.float32).t()
    assert torch.allclose(cpu.linear(x, q, None, "int8", s, z), ref, atol=2e-3, rtol=1e-3)
    q4, s4, m4 = quant.quantize_int4g(w, 128)
    ref4 = x @ quant.dequantize_int4g(q4, s4, m4, torch.float32, 128).t()
    assert torch.allclose(cpu.linear(x, q4, None, "int4g", s4, m4, 128), ref4, atol=2e-3, rtol=1e-3)


def test_norms_and_activations():
    torch.manual_seed(2)
    x = torch.randn(7, 320)
    w, b = torch.randn(320), torch.randn(320)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * (w + 1.0)
    assert torch.allclose(cpu.rmsnorm(x, w, 1e-6, 1.0), ref, atol=1e-5)
    assert torch.allclose(cpu.layernorm(x, w, b, 1e-5), torch.nn.functional.layer_norm(x, (320,), w, b, 1e-5), atol=1e-4)
    gu = torch.randn(5, 256)
    assert torch.allclose(cpu.swiglu(gu), torch.nn.functional.silu(gu[:, :128]) * gu[:, 128:], atol=1e-5)
    assert torch.allclose(cpu.softmax(x), torch.softmax(x, -1), atol=1e-6)
    assert torch.allclose(cpu.activation(x, "gelu"), torch.nn.functional.gelu(x), atol=1e-5)
    assert torch.allclose(cpu.activation(x, "gelu_new"), torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-5)
    assert torch.allclose(cpu.activation(x, "silu"), torch.nn.functional.silu(x), atol=1e-5)


@pytest.mark.parametrize("mode", [A.ROPE_NEOX, A.ROPE_INTERLEAVED])
def test_rope(mode):
    torch.manual_seed(3)
    heads, D, rot = 4, 64, 32
    cos, sin = A.build_rope_tables(rot, 128, 10000.0)
    x = torch.randn(6, heads * D)
    pos = torch.tensor([0, 3, 7, 100, 127, 1])
    ref = A.apply_rope_ref(x.reshape(6, heads, D).clone(), pos, cos, sin, mode, rot).reshape(6, heads * D)
    got = cpu.rope_(x.clone(), pos, cos, sin, heads, D, rot, mode)
    assert torch.allclose(got, ref, atol=1e-5)


@pytest.mark.parametrize("window", [0, 37])
def test_paged_attention(window):
    torch.manual_seed(4)
    Hq, Hkv, D, page = 8, 2, 64, 16
    k_pool = torch.randn(40, page, Hkv, D)
    v_pool = torch.randn(40, page, Hkv, D)
    kv_lens = torch.tensor([50, 1, 97])
    q_lens = [5, 1, 97]
    cu = torch.tensor([0, 5, 6, 103])
    table = torch.randperm(40)[:21].reshape(3, 7).to(torch.int32)
    q = torch.randn(103, Hq * D)
    got = cpu.attention_paged(q, k_pool, v_pool, table, kv_lens, cu, 0.125, Hq, Hkv, D, window=window)
    if window == 0:
        ref = A.paged_attention_ref(q, k_pool, v_pool, table, kv_lens, cu, 0.125, Hq, Hkv, D)
        assert torch.allclose(got, ref, atol=2e-4)
    else:
        # sliding window: compare request 0's last query row against a direct evaluation
        L, ql = 50, q_lens[0]
        pages = table[0, :4].long()
        k = k_pool[pages].reshape(-1, Hkv, D)[:L]
        v = v_pool[pages].reshape(-1, Hkv, D)[:L]
        qpos = L - 1
        lo = max(0, qpos + 1 - window)
        qq = q[ql - 1].reshape(Hkv, Hq // Hkv, D)
        s = torch.einsum("hgd,khd->hgk", qq, k[lo:qpos + 1]) * 0.125
        o = torch.einsum("hgk,khd->hgd", torch.softmax(s, -1), v[lo:qpos + 1]).reshape(-1)
        assert torch.allclose(got[ql - 1], o, atol=2e-4)


def test_select_expert_and_embedding():
    torch.manual_seed(5)
    lg = torch.randn(9, 32)
    bias = torch.randn(32) * 0.1
    idx, w = cpu.select_expert(lg, bias, 4, "sigmoid", True, 2.5)
    sc = torch.sigmoid(lg)
    ref_idx = torch.topk(sc + bias, 4, dim=-1).indices
    ref_w = torch.gather(sc, 1, ref_idx)
    ref_w = ref_w / ref_w.sum(-1, keepdim=True) * 2.5
    assert torch.equal(idx.long(), ref_idx) and torch.allclose(w, ref_w, atol=1e-6)
    table = torch.randn(50, 24)
    ids = torch.tensor([3, 49, 0])
    assert torch.equal(cpu.embedding(table, ids), table[ids])


def test_thread_count_roundtrip():
    n = cpu.get_threads()
    cpu.set_threads(2)
    assert cpu.get_threads() == 2
    x, w = torch.randn(4, 128), torch.randn(300, 128)
    assert torch.allclose(cpu.linear(x, w), x @ w.t(), atol=1e-4)
    cpu.set_threads(n)


@pytest.mark.parametrize("wd", ["auto", "int8", "int4g128"])
def test_native_model_runner_matches_operator_path(wd):
    """Whole-model native forward vs the per-operator path (plain PyTorch definitions) on a tiny Qwen3."""
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.models import cpu_native
    from fastllm_b200.models.config import preset
    from fastllm_b200.models.decoder import random_init

    cfg = preset("tiny-qwen3")
    m = random_init(cfg, "cpu", torch.float32, std=0.05, wdtype=wd)
    assert cpu_native.eligible(m)
    prompt = list(range(5, 45))
    eng = LLMEngine(m, EngineConfig(max_batch=2, max_context=256), num_pages=8)
    got = eng.generate([prompt, prompt[:7]], GenerationConfig(max_new_tokens=8, ignore_eos=True))
    m2 = random_init(cfg, "cpu", torch.float32, std=0.05, wdtype=wd)
    m2._cpu_runner = False          # operator path only
    import os
    os.environ["FB_CPU_NATIVE"] = "0"
    try:
        eng2 = LLMEngine(m2, EngineConfig(max_batch=2, max_context=256), num_pages=8)
        ref = eng2.generate([prompt, prompt[:7]], GenerationConfig(max_new_tokens=8, ignore_eos=True))
    finally:
        os.environ.pop("FB_CPU_NATIVE")
    assert got == ref


@pytest.mark.parametrize("wd", ["auto", "int4g128"])
def test_host_expert_ffn_matches_operator_path(wd):
    """Native routed-expert FFN (the hybrid-placement path) vs the per-expert operator loop."""
    from fastllm_b200.models.config import preset
    from fastllm_b200.models.decoder import random_init
    from fastllm_b200.ops import moe as MOE

    m = random_init(preset("tiny-qwen3-moe"), "cpu", torch.float32, std=0.05, moe_wdtype=wd)
    ex = m.layers[0].mlp.experts
    torch.manual_seed(7)
    x = torch.randn(11, m.cfg.hidden_size)
    logits = torch.randn(11, m.cfg.num_experts)
    idx, wts = MOE.route_topk(logits, None, 2, 0, True)
    ref = MOE.moe_forward(x, idx, wts, ex)
    ex.host = True
    got = MOE.moe_forward(x, idx, wts, ex)
    ex.host = False
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3)


@pytest.mark.parametrize("wd", ["auto", "int8", "int4g128"])
def test_numa_expert_placement_matches_single_node(wd, monkeypatch):
    """Experts cut across two (emulated) memory nodes with pinned thread teams: same result as the single-node host path,
    bit for bit (the row kernels and the summation order per token are the same)."""
    from fastllm_b200.models.config import preset
    from fastllm_b200.models.decoder import random_init
    from fastllm_b200.ops import cpu
    from fastllm_b200.ops import moe as MOE

    ncpu = len(os.sched_getaffinity(0))
    cpus = sorted(os.sched_getaffinity(0))
    half = max(1, ncpu // 2)
    groups = [cpus[:half], cpus[half:] or cpus[:half]]
    monkeypatch.setenv("FB_NUMA_NODES", ";".join(",".join(map(str, g)) for g in groups))
    assert cpu.lib().fbnuma_node_count() == 2
    m = random_init(preset("tiny-qwen3-moe"), "cpu", torch.float32, std=0.05, moe_wdtype=wd)
    ex = m.layers[0].mlp.experts
    torch.manual_seed(9)
    for T in (1, 13, 70):
        x = torch.randn(T, m.cfg.hidden_size)
        logits = torch.randn(T, m.cfg.num_experts)
        idx, wts = MOE.route_topk(logits, None, 2, 0, True)
        ex.host, ex.numa = True, False
        ex._host_arrays = None
        ref = MOE.moe_forward(x, idx, wts, ex)
        ex.numa = True
        ex._host_arrays = None
        got = MOE.moe_forward(x, idx, wts, ex)
        assert getattr(ex, "_numa_handle", None)
        assert torch.equal(got, ref), (wd, T, (got - ref).abs().max())
        cpu.lib().fbnuma_destroy(ctypes.c_void_p(ex._numa_handle))
        ex._numa_handle = None
    ex.host = ex.numa = False


def _blocks_s8(x):
    """Activations rounded to int8 per (row, 128-wide block), as the VNNI / AMX kernels see them."""
    M, K = x.shape
    xb = x.reshape(M, K // 128, 128)
    sc = xb.abs().amax(-1, keepdim=True).clamp(min=1e-20) / 127.0
    return (torch.round(xb / sc).clamp(-127, 127) * sc).reshape(M, K)


@pytest.mark.parametrize("M", [1, 5, 16, 37])
def test_accelerated_cpu_kernels(M):
    """VNNI / AVX-512 BF16 / AMX kernels (where the CPU has them) against the same arithmetic in PyTorch: activations rounded
    to int8 blocks or bf16, exact integer / fp32 accumulation."""
    caps = cpu.accel_caps()
    if caps == 0:
        pytest.skip("no VNNI / AVX-512 BF16 / AMX on this CPU")
    torch.manual_seed(5)
    K, N = 512, 200
    x = torch.randn(M, K)
    w = torch.randn(N, K) * 0.05
    b = torch.randn(N)
    try:
        for flags in sorted({caps & 3, caps}):          # without and with AMX
            if flags == 0:
                continue
            assert cpu.set_accel(flags) == flags
            if flags & (cpu.ACCEL_BF16 | cpu.ACCEL_AMX):
                wb = w.to(torch.bfloat16)
                ref = x.to(torch.bfloat16).float() @ wb.float().t() + b
                got = cpu.linear(x, wb, b)
                assert torch.allclose(got, ref, atol=2e-4, rtol=1e-4), (flags, (got - ref).abs().max())
            if flags & cpu.ACCEL_VNNI:
                q, s, z = quant.quantize_int8(w)
                ref8 = _blocks_s8(x) @ quant.dequantize_int8(q, s, z, torch.float32).t() + b
                got8 = cpu.linear(x, q, b, "int8", s, z)
                assert torch.allclose(got8, ref8, atol=3e-4, rtol=1e-4), (flags, (got8 - ref8).abs().max())
                q4, s4, m4 = quant.quantize_int4g(w, 128)
                ref4 = _blocks_s8(x) @ quant.dequantize_int4g(q4, s4, m4, torch.float32, 128).t()
                got4 = cpu.linear(x, q4, None, "int4g", s4, m4, 128)
                assert torch.allclose(got4, ref4, atol=3e-4, rtol=1e-4), (flags, (got4 - ref4).abs().max())
    finally:
        cpu.set_accel(0)
    assert cpu.get_accel() == 0
