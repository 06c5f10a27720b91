"""Small single-kernel workloads for profiling (`python -m fastllm_b200.utils.profile_cases <case>`).

Each case allocates a few hundred MB (inputs larger than the 126 MB L2 so DRAM counters mean something), runs
the kernel a handful of times and exits; meant to be wrapped as
`ncu --set full --clock-control none -k regex:<kernel> -s 2 -c 2 -o <out> python -m fastllm_b200.utils.profile_cases <case>`.
"""
from __future__ import annotations

import math
import sys

import torch

from ..ops import _lib
from ..ops import attention as A
from ..ops import basic as B


def gemm_decode(n=28672, k=4096, m=64, swiglu=True, iters=4):
    dev = "cuda"
    ws = [(torch.randn(n, k, device=dev) * 0.02).bfloat16() for _ in range(2)]
    x = torch.randn(m, k, device=dev).bfloat16()
    for i in range(iters):
        B.linear(x, ws[i % 2], swiglu=swiglu)
    torch.cuda.synchronize()


def attn_decode(batch=64, length=1100, hq=32, hkv=8, iters=4):
    dev, D = "cuda", 128
    npg = (length + 127) // 128
    pages = batch * npg
    k_pool = (torch.randn(pages, 128, hkv, D, device=dev) * 0.5).bfloat16()
    v_pool = torch.randn(pages, 128, hkv, D, device=dev).bfloat16()
    pt = torch.randperm(pages, device=dev).int().view(batch, npg)
    seq = torch.full((batch,), length, dtype=torch.int32, device=dev)
    q = torch.randn(batch, hq * D, device=dev).bfloat16()
    ws = A.DecodeWorkspace(batch, hkv, hq // hkv, npg, dev)
    torch.cuda.synchronize()
    for _ in range(iters):
        A.attn_decode(q, k_pool, v_pool, pt, seq, 1 / math.sqrt(D), hq, hkv, D, ws=ws)
    torch.cuda.synchronize()


def gemm_prefill(m=4096, n=6144, k=4096, iters=4):
    dev = "cuda"
    w = (torch.randn(n, k, device=dev) * 0.02).bfloat16()
    x = torch.randn(m, k, device=dev).bfloat16()
    for _ in range(iters):
        B.linear(x, w)
    torch.cuda.synchronize()


def gemm_quant(kind="fp8", n=28672, k=4096, m=64, iters=4):
    from ..ops.quant import LinearWeight

    dev = "cuda"
    ws = [LinearWeight.from_dense((torch.randn(n, k, device=dev) * 0.02).bfloat16(), kind, interleaved=True) for _ in range(2)]
    x = torch.randn(m, k, device=dev).bfloat16()
    for i in range(iters):
        ws[i % 2](x, swiglu=True)
    torch.cuda.synchronize()


def mla_decode(batch=32, length=2300, heads=16, iters=4):
    dev = "cuda"
    npg = (length + 127) // 128
    pages = batch * npg
    lat = (torch.randn(pages + 1, 128, 1, 576, device=dev) * 0.5).bfloat16()
    pt = torch.randperm(pages, device=dev).int().view(batch, npg)
    seq = torch.full((batch,), length, dtype=torch.int32, device=dev)
    q = (torch.randn(batch, heads, 576, device=dev) * 0.5).bfloat16()
    for _ in range(iters):
        A.mla_decode(q, lat, pt, seq, 0.07)
    torch.cuda.synchronize()


def attn_prefill(batch=4, length=2048, hq=32, hkv=8, iters=3):
    dev, D = "cuda", 128
    npg = (length + 127) // 128
    pages = batch * npg
    k_pool = (torch.randn(pages, 128, hkv, D, device=dev) * 0.5).bfloat16()
    v_pool = torch.randn(pages, 128, hkv, D, device=dev).bfloat16()
    pt = torch.randperm(pages, device=dev).int().view(batch, npg)
    kv = torch.full((batch,), length, dtype=torch.int32, device=dev)
    cu = (torch.arange(batch + 1, device=dev) * length).int()
    q = torch.randn(batch * length, hq * D, device=dev).bfloat16()
    for _ in range(iters):
        A.attn_prefill(q, k_pool, v_pool, pt, kv, cu, 1 / math.sqrt(D), hq, hkv, D)
    torch.cuda.synchronize()


def moe_grouped(tokens=128, experts=128, topk=8, hidden=2048, inter=768, kind="fp8", iters=4):
    from ..models.config import preset
    from ..models.decoder import random_init
    from ..ops import moe as MOE

    cfg = preset("qwen3-30b-a3b")
    cfg.num_layers = 1
    m = random_init(cfg, "cuda", torch.bfloat16, moe_wdtype=kind)
    ex = m.layers[0].mlp.experts
    x = torch.randn(tokens, hidden, device="cuda").bfloat16()
    idx, w = MOE.route_topk(torch.randn(tokens, experts, device="cuda"), None, topk, 0, True)
    for _ in range(iters):
        MOE.moe_forward(x, idx, w, ex)
    torch.cuda.synchronize()


def moe_ep_rank(model="deepseek-v3", tokens=32, ranks=8, kind="int4g128", iters=6, timed=True):
    """One expert-parallel rank's share of a routed-expert layer at decode size (e.g. DeepSeek-V3: 32 of 256 experts, top-8,
    hidden 7168, intermediate 2048): routing of all tokens, only the local experts' rows computed.  Prints the device time per
    layer call (CUDA events around a CUDA graph of ``iters`` calls over rotating weight copies)."""
    import dataclasses

    from ..models import TPInfo
    from ..models.config import preset
    from ..models.decoder import random_init
    from ..ops import moe as MOE
    from ..parallel.ep import EPInfo

    cfg = preset(model)
    first = cfg.first_k_dense
    copies = 3
    cfg = dataclasses.replace(cfg, num_layers=first + copies)
    tp = TPInfo(0, ranks, None)
    m = random_init(cfg, "cuda", torch.bfloat16, tp=tp, ep=EPInfo.from_tp(tp), wdtype="dense", moe_wdtype=kind, expert_pool=4)
    exs = [m.layers[first + i].mlp.experts for i in range(copies)]
    x = torch.randn(tokens, cfg.hidden_size, device="cuda").bfloat16()
    idx, w = MOE.route_topk(torch.randn(tokens, cfg.num_experts, device="cuda"), None, cfg.num_experts_per_tok, 0, True)
    for i in range(3):
        MOE.moe_forward(x, idx, w, exs[i % copies])
    torch.cuda.synchronize()
    if not timed:
        return
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        MOE.moe_forward(x, idx, w, exs[0])
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        for i in range(iters):
            MOE.moe_forward(x, idx, w, exs[i % copies])
    g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    g.replay()
    e.record()
    torch.cuda.synchronize()
    local = ((idx >= exs[0].first) & (idx < exs[0].first + exs[0].count))
    hit = int(torch.unique(idx[local]).numel())
    per = sum(l.nbytes() for l in exs[0].gate_up[:1] + exs[0].down[:1])
    print(f"moe_ep_rank {model} {kind} tokens={tokens}: {s.elapsed_time(e) / iters * 1e3:.1f} us per layer call; "
          f"{int(local.sum())} local rows on {hit} of {exs[0].count} local experts; {hit * per / 1e6:.0f} MB of expert weights touched")


def attn_decode_kv8(batch=64, length=1100, hq=32, hkv=8, iters=10, only_e4m3=False):
    """Decode attention over bf16 and over e4m3 page pools, device time per call (CUDA events around a CUDA graph)."""
    from ..ops import attention as A

    D = 128
    npg = (length + 127) // 128
    pages = batch * npg
    pt = torch.randperm(pages, device="cuda").int().view(batch, npg)
    seq = torch.full((batch,), length, dtype=torch.int32, device="cuda")
    q = torch.randn(batch, hq * D, device="cuda").bfloat16()
    k16 = (torch.randn(pages, 128, hkv, D, device="cuda") * 0.5).bfloat16()
    v16 = torch.randn(pages, 128, hkv, D, device="cuda").bfloat16()
    for name, (kp, vp) in (("bf16 pages", (k16, v16)), ("e4m3 pages", (k16.to(torch.float8_e4m3fn), v16.to(torch.float8_e4m3fn)))):
        if only_e4m3 and name.startswith("bf16"):
            continue
        ws = A.DecodeWorkspace(batch, hkv, hq // hkv, npg, "cuda")
        for _ in range(3):
            A.attn_decode(q, kp, vp, pt, seq, D ** -0.5, hq, hkv, D, ws=ws)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                A.attn_decode(q, kp, vp, pt, seq, D ** -0.5, hq, hkv, D, ws=ws)
        g.replay()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); g.replay(); e.record()
        torch.cuda.synchronize()
        print(f"attn_decode {name}: {s.elapsed_time(e) / iters * 1e3:.1f} us per call ({batch} x {length} tokens, {hq}/{hkv} heads)")


def gemm_qkv_post(tokens=64, hq=32, hkv=8, k=4096, iters=4):
    from ..ops.quant import LinearWeight

    dev, D = "cuda", 128
    n = (hq + 2 * hkv) * D
    ws = [LinearWeight.from_dense((torch.randn(n, k, device=dev) * 0.02).bfloat16()) for _ in range(3)]       # 3 x 50 MB > L2
    x = torch.randn(tokens, k, device=dev).bfloat16()
    cos, sin = A.build_rope_tables(D, 4096, 5e5, None, dev)
    pos = torch.arange(tokens, device=dev).int()
    slots = torch.arange(tokens, device=dev).int()
    kp = torch.zeros(4, 128, hkv, D, device=dev, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    for i in range(iters):
        A.qkv_proj_post(x, ws[i % 3], pos, slots, kp, vp, hq, hkv, D, cos, sin)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(12):
            A.qkv_proj_post(x, ws[i % 3], pos, slots, kp, vp, hq, hkv, D, cos, sin)
    g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(); g.replay(); e.record()
    torch.cuda.synchronize()
    print(f"gemm_qkv_post: {s.elapsed_time(e) / 12 * 1e3:.1f} us per call ({tokens} tokens, N = {n}, K = {k}, weights rotated)")


def gdn_decode(batch=64, hk=16, hv=32, iters=4):
    from ..ops import linear_attn as L

    dev, D, dt = "cuda", 128, torch.bfloat16
    C = 2 * hk * D + hv * D
    conv = torch.zeros(batch + 1, C, 3, device=dev, dtype=dt)
    rec = torch.randn(batch + 1, hv, D, D, device=dev) * 0.05            # 64 x 32 x 64 KB = 134 MB of state
    w = (torch.randn(C, 4, device=dev) * 0.3).to(dt)
    slots = torch.arange(batch, device=dev).int()
    A_log, dtb = torch.zeros(hv, device=dev), torch.ones(hv, device=dev)
    nw = torch.ones(D, device=dev, dtype=dt)
    for _ in range(iters):
        x = torch.randn(batch, C, device=dev).to(dt)
        a, b = torch.randn(batch, hv, device=dev).to(dt), torch.randn(batch, hv, device=dev).to(dt)
        z = torch.randn(batch, hv * D, device=dev).to(dt)
        y = L.causal_conv1d_decode(x, w, conv, slots)
        L.gated_delta_decode(y, a, b, z, A_log, dtb, nw, 1e-6, rec, slots, hk, hv, D, D)
    torch.cuda.synchronize()


def model_kernel_table(model="qwen3-30b-a3b", wdtype="fp8", batch=128, prompt=512, steps=4):
    """Per-launcher device-time table of whole decode steps (eager, CUDA events around every launch): where a model's step goes."""
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.models import preset, random_init

    cfg = preset(model)
    m = random_init(cfg, "cuda", torch.bfloat16, std=0.02, wdtype=wdtype, moe_wdtype=wdtype, expert_pool=8)
    eng = LLMEngine(m, EngineConfig(max_batch=batch, max_context=prompt + 512, use_cuda_graph=False, prefix_cache=False,
                                    chunked_prefill_size=8192, max_tokens=int(batch * (prompt + 300) / 0.75)))
    g = torch.Generator().manual_seed(1)
    for _ in range(batch):
        eng.launch(torch.randint(0, cfg.vocab_size, (prompt,), generator=g).tolist(), GenerationConfig(max_new_tokens=64, ignore_eos=True))
    while any(r.state.name in ("WAITING", "PREFILL") for r in eng.requests.values()):
        eng.step()
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    _lib.start_profile()
    torch.cuda.profiler.start()          # `ncu --profile-from-start off` then sees the decode steps only
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(_lib.stop_profile().format())


CASES = {
    "model_kernel_table_qwen3_moe_fp8": model_kernel_table,
    "gemm_qkv_post": gemm_qkv_post,
    "attn_decode_kv8": attn_decode_kv8,
    "attn_decode_kv8_only": lambda: attn_decode_kv8(iters=2, only_e4m3=True),
    "moe_ep_rank_dsv3_int4g": lambda: moe_ep_rank("deepseek-v3", 32, 8, "int4g128"),
    "moe_ep_rank_dsv3_int4g_untimed": lambda: moe_ep_rank("deepseek-v3", 32, 8, "int4g128", timed=False),
    "moe_ep_rank_dsv3_fp8": lambda: moe_ep_rank("deepseek-v3", 32, 8, "fp8"),
    "moe_ep_rank_qwen3_fp8": lambda: moe_ep_rank("qwen3-30b-a3b", 128, 8, "fp8"),
    "gdn_decode": gdn_decode,
    "gemm_prefill_gate_up": lambda: gemm_prefill(4096, 28672, 4096),
    "gemm_quant_fp8": lambda: gemm_quant("fp8"),
    "gemm_quant_int4g": lambda: gemm_quant("int4g128"),
    "gemm_quant_fp8_m16": lambda: gemm_quant("fp8", m=16),
    "gemm_quant_int8": lambda: gemm_quant("int8"),
    "gemm_quant_int8_m16": lambda: gemm_quant("int8", m=16),
    "gemm_quant_int4g_m16": lambda: gemm_quant("int4g128", m=16),
    "mla_decode": mla_decode,
    "attn_prefill": attn_prefill,
    "moe_grouped_fp8": moe_grouped,
    "gemm_decode_gate_up": lambda: gemm_decode(28672, 4096, 64, True),
    "gemm_decode_down": lambda: gemm_decode(4096, 14336, 64, False),
    "attn_decode": attn_decode,
    "gemm_prefill": gemm_prefill,
}

if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else "gemm_decode_gate_up"
    CASES[name]()
    _lib.check_device_errors()
    print("ok", name)
