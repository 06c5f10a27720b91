"""Numerics of every CUDA kernel against the plain PyTorch fp32 definition of the same op."""
import math

import pytest
import torch

from fastllm_b200.ops import _lib, attention as A, basic as B

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol, what="", fro=None):
    """Element-wise tolerance; with ``fro`` also a bound on the relative Frobenius error, which a dropped k-block or a stale
    tile cannot hide behind the absolute tolerance of small outputs."""
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{what}: {bad}/{a.numel()} mismatches, max err {err.max().item():.4g}, ref max {b.abs().max().item():.4g}"
    if fro is not None:
        rel = (a - b).norm().item() / max(b.norm().item(), 1e-20)
        assert rel < fro, f"{what}: relative Frobenius error {rel:.4g} >= {fro}"


@pytest.fixture(autouse=True)
def _device_errors():
    yield
    torch.cuda.synchronize()
    _lib.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,nsplit", [(1, 256, 256, 1), (7, 384, 512, 2), (16, 4096, 4096, 0), (33, 1024, 2048, 4),
                                          (64, 6144, 4096, 0), (64, 4096, 14336, 8), (100, 512, 1024, 0), (200, 1024, 512, 2),
                                          (256, 256, 4096, 0)])
def test_gemm_small_m(dtype, M, N, K, nsplit):
    torch.manual_seed(0)
    x = (torch.randn(M, K, device=DEV) * 0.5).to(dtype)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(dtype)
    y = B.linear(x, w, nsplit=nsplit)
    ref = B.linear_ref(x, w)
    _close(y, ref, 2e-2, 2e-2, f"gemm {M}x{N}x{K}", fro=1e-2)


def test_gemm_epilogues():
    torch.manual_seed(1)
    M, N, K = 48, 1024, 1024
    dt = torch.bfloat16
    x = (torch.randn(M, K, device=DEV) * 0.5).to(dt)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(dt)
    bias = torch.randn(N, device=DEV).to(dt)
    res = torch.randn(M, N, device=DEV).to(dt)
    _close(B.linear(x, w, bias=bias), B.linear_ref(x, w, bias=bias), 3e-2, 2e-2, "bias", fro=1e-2)
    _close(B.linear(x, w, residual=res), B.linear_ref(x, w, residual=res), 3e-2, 2e-2, "residual", fro=1e-2)
    _close(B.linear(x, w, bias=bias, residual=res, out_f32=True), B.linear_ref(x, w, bias, res, out_dtype=torch.float32), 2e-2,
           2e-2, "f32 out")
    for ns in (1, 2, 4, 8):
        y = B.linear(x, w, swiglu=True, nsplit=ns)
        _close(y, B.linear_ref(x, w, swiglu=True), 3e-2, 3e-2, f"swiglu split {ns}")
    res2 = torch.randn(M, N // 2, device=DEV).to(dt)
    _close(B.linear(x, w, bias=bias, swiglu=True, residual=res2), B.linear_ref(x, w, bias, res2, swiglu=True), 3e-2, 3e-2,
           "swiglu+bias+res")


@pytest.mark.parametrize("M,N,K", [(257, 256, 256), (1024, 4096, 4096), (300, 384, 1024), (2048, 1024, 512)])
def test_gemm_large_m(M, N, K):
    torch.manual_seed(2)
    dt = torch.bfloat16
    x = (torch.randn(M, K, device=DEV) * 0.5).to(dt)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(dt)
    bias = torch.randn(N, device=DEV).to(dt)
    res = torch.randn(M, N, device=DEV).to(dt)
    _close(B.linear(x, w), B.linear_ref(x, w), 3e-2, 2e-2, "plain", fro=1e-2)
    _close(B.linear(x, w, bias=bias, residual=res), B.linear_ref(x, w, bias, res), 3e-2, 2e-2, "bias+res", fro=1e-2)
    if N % 128 == 0:
        _close(B.linear(x, w, swiglu=True), B.linear_ref(x, w, swiglu=True), 3e-2, 3e-2, "swiglu")


@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (70, 1024, 512), (600, 256, 2048)])
def test_linear_fp32_on_split_bf16_operands(M, N, K):
    """fp32 activations x fp32 weights as three bf16 tensor-core GEMMs over (head, remainder) splits: the error against an fp64
    evaluation stays at fp32-matmul level, two orders of magnitude below a single bf16 GEMM."""
    torch.manual_seed(30)
    x = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV) * 0.05
    bias = torch.randn(N, device=DEV)
    res = torch.randn(M, N, device=DEV)
    ref = (x.double() @ w.double().t() + bias.double() + res.double())
    y = B.linear(x, w, bias, res)
    assert y.dtype == torch.float32
    rel = ((y.double() - ref).norm() / ref.norm()).item()
    one = B.linear(x.bfloat16(), w.bfloat16(), out_f32=True).double() + bias.double() + res.double()
    rel_bf16 = ((one - ref).norm() / ref.norm()).item()
    assert rel < 2e-5 and rel < rel_bf16 / 50, (rel, rel_bf16)


def test_interleave_roundtrip():
    g, u = torch.randn(256, 8), torch.randn(256, 8)
    w = B.interleave_gate_up(g, u)
    g2, u2 = B.deinterleave_gate_up(w)
    assert torch.equal(g, g2) and torch.equal(u, u2)


@pytest.mark.parametrize("H", [1024, 4096, 7168])
def test_rmsnorm(H):
    torch.manual_seed(3)
    dt = torch.bfloat16
    x = torch.randn(37, H, device=DEV).to(dt)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(dt)
    _close(B.rmsnorm(x, w, 1e-6), B.rmsnorm_ref(x, w, 1e-6)[0], 2e-2, 2e-2, "rmsnorm")
    res = torch.randn(37, H, device=DEV).to(dt)
    res_k = res.clone()
    y = B.rmsnorm(x, w, 1e-5, residual=res_k)
    yr, rr = B.rmsnorm_ref(x, w, 1e-5, residual=res)
    _close(res_k, rr, 1e-2, 1e-2, "residual out")
    _close(y, yr, 3e-2, 2e-2, "rmsnorm+res")


@pytest.mark.parametrize("act", ["gelu_pytorch_tanh", "gelu", "relu", "silu"])
@pytest.mark.parametrize("interleaved", [False, True])
def test_glu_act(act, interleaved):
    """GeGLU / ReGLU kernel (both gate/up layouts) against the fp32 PyTorch statement."""
    torch.manual_seed(14)
    for dt in (torch.bfloat16, torch.float16):
        x = (torch.randn(37, 2 * 704, device=DEV) * 1.5).to(dt)
        got = B.glu_act(x, act, interleaved)
        ref = B.glu_act_ref(x.float(), act, interleaved)
        assert got.shape == (37, 704) and got.dtype == dt
        _close(got, ref, 2e-2, 2e-2, f"glu_act {act} {interleaved}", fro=6e-3)


def test_silu_embedding_argmax():
    torch.manual_seed(4)
    dt = torch.bfloat16
    x = torch.randn(19, 2 * 768, device=DEV).to(dt)
    _close(B.silu_mul(x), B.silu_mul(x.cpu()).to(DEV), 2e-2, 2e-2, "silu_mul")
    table = torch.randn(1000, 256, device=DEV).to(dt)
    ids = torch.randint(0, 1000, (33,), device=DEV)
    assert torch.equal(B.embedding(ids, table), table[ids])
    logits = torch.randn(9, 50000, device=DEV)
    assert torch.equal(B.argmax(logits).long(), logits.argmax(-1))
    big = torch.randn(64, 128256, device=DEV)
    big[3, 70000] = big[3, 1000] = 50.0                      # a tie: the lowest index wins
    big[5] = float("-inf")
    got = B.argmax(big).long()
    assert torch.equal(got[:5], big[:5].argmax(-1)) and int(got[3]) == 1000 and int(got[5]) == 0
    assert torch.equal(got[6:], big[6:].argmax(-1))
    odd = torch.randn(7, 1003, device=DEV)                  # row length that is no multiple of four: scalar path
    assert torch.equal(B.argmax(odd).long(), odd.argmax(-1))
    assert torch.equal(B.argmax(logits.to(dt)).long().cpu(), B.argmax(logits.to(dt).cpu()).long())


def _make_cache(B_, lens, Hkv, D, dt, extra_pages=3):
    n_pages = sum((l + 127) // 128 for l in lens) + extra_pages
    perm = torch.randperm(n_pages)
    max_pages = max((l + 127) // 128 for l in lens)
    pt = torch.zeros(B_, max_pages, dtype=torch.int32)
    c = 0
    for b, l in enumerate(lens):
        n = (l + 127) // 128
        pt[b, :n] = perm[c:c + n].int()
        c += n
    k_pool = torch.zeros(n_pages, 128, Hkv, D, dtype=dt)
    v_pool = torch.zeros(n_pages, 128, Hkv, D, dtype=dt)
    for b, l in enumerate(lens):
        for i in range((l + 127) // 128):
            n = min(128, l - i * 128)
            k_pool[pt[b, i], :n] = (torch.randn(n, Hkv, D) * 0.7).to(dt)
            v_pool[pt[b, i], :n] = torch.randn(n, Hkv, D).to(dt)
            # recycled pages hold stale (finite) data behind the last token: it must not leak into the result
            k_pool[pt[b, i], n:] = 50.0
            v_pool[pt[b, i], n:] = -80.0
    return k_pool, v_pool, pt


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (16, 8), (8, 1), (16, 16)])
def test_attn_decode(Hq, Hkv):
    torch.manual_seed(5)
    D, dt = 128, torch.bfloat16
    lens = [1, 127, 128, 129, 300, 1025, 77]
    Bn = len(lens)
    k_pool, v_pool, pt = _make_cache(Bn, lens, Hkv, D, dt)
    q = torch.randn(Bn, Hq * D).to(dt)
    seq = torch.tensor(lens, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    ref = A.attn_decode(q, k_pool, v_pool, pt, seq, scale, Hq, Hkv, D)
    out = A.attn_decode(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), pt.to(DEV), seq.to(DEV), scale, Hq, Hkv, D)
    _close(out.cpu(), ref, 2e-2, 2e-2, "attn_decode")
    # one workspace reused by consecutive launches (the fused combine's arrival counters must be back at zero)
    ws = A.DecodeWorkspace(Bn, Hkv, Hq // Hkv, pt.shape[1], DEV)
    args = (q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), pt.to(DEV), seq.to(DEV), scale, Hq, Hkv, D)
    for _ in range(3):
        out = A.attn_decode(*args, ws=ws)
    _close(out.cpu(), ref, 2e-2, 2e-2, "attn_decode (reused workspace)")
    assert int(ws.counters.abs().sum()) == 0
    # the in-kernel merge of the partials (off by default) gives the same result
    A._FUSED_COMBINE = True
    try:
        for _ in range(2):
            out = A.attn_decode(*args, ws=ws)
    finally:
        A._FUSED_COMBINE = False
    _close(out.cpu(), ref, 2e-2, 2e-2, "attn_decode (fused combine)")
    assert int(ws.counters.abs().sum()) == 0
    _lib.check_device_errors()


@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4)])
def test_attn_prefill(Hq, Hkv):
    torch.manual_seed(6)
    D, dt = 128, torch.bfloat16
    kv_lens = [5, 128, 200, 513, 300]
    q_lens = [5, 128, 200, 513, 45]          # last request: chunk continuing a 255-token history
    Bn = len(kv_lens)
    k_pool, v_pool, pt = _make_cache(Bn, kv_lens, Hkv, D, dt)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    q = (torch.randn(int(cu[-1]), Hq * D) * 0.7).to(dt)
    kvl = torch.tensor(kv_lens, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    ref = A.paged_attention_ref(q, k_pool, v_pool, pt, kvl, cu, scale, Hq, Hkv, D)
    out = A.attn_prefill(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), pt.to(DEV), kvl.to(DEV), cu.to(DEV), scale, Hq, Hkv, D)
    _close(out.cpu(), ref, 2e-2, 2e-2, "attn_prefill")


@pytest.mark.parametrize("mode,rot,qknorm", [(A.ROPE_NEOX, 128, True), (A.ROPE_NEOX, 128, False), (A.ROPE_INTERLEAVED, 64, False),
                                             (A.ROPE_NEOX, 64, True), (A.ROPE_NONE, 128, False)])
def test_qkv_post(mode, rot, qknorm):
    torch.manual_seed(7)
    Hq, Hkv, D, dt, T = 16, 8, 128, torch.bfloat16, 21
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D).to(dt)
    pos = torch.randint(0, 500, (T,), dtype=torch.int32)
    slots = torch.randperm(4 * 128)[:T].int()
    slots[3] = -1
    cos, sin = A.build_rope_tables(rot, 512, 10000.0)
    qn = (1 + 0.1 * torch.randn(D)).to(dt) if qknorm else None
    kn = (1 + 0.1 * torch.randn(D)).to(dt) if qknorm else None
    kp, vp = torch.zeros(4, 128, Hkv, D, dtype=dt), torch.zeros(4, 128, Hkv, D, dtype=dt)
    q_ref = A.qkv_post(qkv, pos, slots, kp, vp, Hq, Hkv, D, cos, sin, mode, rot, qn, kn, 1e-6)
    kp2, vp2 = torch.zeros_like(kp).to(DEV), torch.zeros_like(vp).to(DEV)
    q_out = A.qkv_post(qkv.to(DEV), pos.to(DEV), slots.to(DEV), kp2, vp2, Hq, Hkv, D, cos.to(DEV), sin.to(DEV), mode, rot,
                       qn.to(DEV) if qknorm else None, kn.to(DEV) if qknorm else None, 1e-6)
    _close(q_out.cpu(), q_ref, 3e-2, 2e-2, "q")
    _close(kp2.cpu(), kp, 3e-2, 2e-2, "k pool")
    _close(vp2.cpu(), vp, 0, 0, "v pool")


@pytest.mark.parametrize("kind", ["int8", "int4g128", "fp8", "nvfp4", "mxfp4"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (13, 384, 1024), (64, 4096, 4096), (200, 1024, 2048), (300, 512, 512)])
def test_gemm_quant(kind, dtype, M, N, K, fp8_w8a16):
    from fastllm_b200.ops import quant

    torch.manual_seed(8)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(dtype)
    lw = quant.LinearWeight.from_dense(w, kind, act_dtype=dtype)
    assert lw.kind != "dense"
    x = (torch.randn(M, K, device=DEV) * 0.5).to(dtype)
    ref = B.linear_ref(x, lw.dequant(torch.float32))
    y = lw(x)
    _close(y, ref, 4e-2, 3e-2, f"quant gemm {kind} {M}x{N}x{K}")


@pytest.mark.parametrize("kind", ["nvfp4", "mxfp4"])
def test_gemm_fp4_operand_forms(kind, monkeypatch):
    """fp4 weights with fp16 activations: the half2 de-quantiser and the fp32 one give the same result as the fp32 evaluation
    of the de-quantised weights."""
    from fastllm_b200.ops import quant, quant_gemm as QG

    torch.manual_seed(18)
    M, N, K, dt = 40, 512, 1024, torch.float16
    w = (torch.randn(N, K, device=DEV) * 0.05).to(dt)
    x = (torch.randn(M, K, device=DEV) * 0.5).to(dt)
    outs = []
    for fast in (True, False):
        monkeypatch.setattr(QG, "FP4_F16W", fast)
        lw = quant.LinearWeight.from_dense(w, kind, act_dtype=dt)
        ref = B.linear_ref(x, lw.dequant(torch.float32))
        y = lw(x)
        assert QG._kernel_tensors(lw)[2] == fast
        _close(y, ref, 3e-2, 2e-2, f"fp4 {kind} fast={fast}", fro=6e-3)
        outs.append(y.float())
    assert (outs[0] - outs[1]).norm() / outs[1].norm() < 5e-3


@pytest.mark.parametrize("kind", ["int8", "int4g128", "int4g64", "fp8", "nvfp4", "mxfp4"])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_dequant_weight_kernel(kind, dt, monkeypatch):
    """Whole-matrix de-quantisation kernel (the form prefill-sized batches multiply with) vs the PyTorch statement of each
    format; int8 also in its q - 128 operand form."""
    from fastllm_b200.ops import quant

    torch.manual_seed(31)
    w = (torch.randn(384, 512, device=DEV) * 0.05).to(dt)
    lw = quant.LinearWeight.from_dense(w, kind, act_dtype=dt)
    assert lw.kind != "dense"
    got = lw.dequant(dt)
    monkeypatch.setattr(quant, "DEQUANT_KERNEL", False)
    want = lw.dequant(torch.float32)
    assert got.dtype == dt and got.shape == want.shape
    _close(got, want, 1e-3, 1e-2, f"dequant {kind}", fro=4e-3)
    x = (torch.randn(1500, 512, device=DEV) * 0.5).to(dt)           # above the chunked small-batch route: dense GEMM on the result
    monkeypatch.setattr(quant, "DEQUANT_KERNEL", True)
    y = lw(x)
    ref = B.linear_ref(x, want)
    # (formats with 8-bit-activation decode kernels round the activations of large batches the same way: compare in norm)
    rel = ((y.float() - ref.float()).norm() / ref.float().norm()).item()
    assert rel < 3e-2, (kind, rel)


def test_gemm_quant_epilogues(fp8_w8a16):
    from fastllm_b200.ops import quant

    torch.manual_seed(9)
    M, N, K, dt = 48, 1024, 1024, torch.bfloat16
    w = (torch.randn(N, K, device=DEV) * 0.05).to(dt)
    x = (torch.randn(M, K, device=DEV) * 0.5).to(dt)
    bias = torch.randn(N, device=DEV).to(dt)
    res = torch.randn(M, N // 2, device=DEV).to(dt)
    for kind in ("int8", "int4g128", "fp8", "nvfp4", "mxfp4"):
        lw = quant.LinearWeight.from_dense(w, kind, bias=bias, interleaved=True, act_dtype=dt)
        y = lw(x, residual=res, swiglu=True)
        ref = B.linear_ref(x, lw.dequant(torch.float32), bias, res, swiglu=True)
        _close(y, ref, 5e-2, 4e-2, f"quant epilogue {kind}")


@pytest.mark.parametrize("T,E,first,n_local,topk", [(7, 8, 0, 8, 2), (64, 16, 4, 8, 4), (130, 32, 0, 32, 8), (300, 8, 2, 4, 2)])
def test_moe_grouped(T, E, first, n_local, topk):
    """Grouped expert path vs the per-expert PyTorch definition, including experts owned by other ranks."""
    from fastllm_b200.ops import moe as MOE, moe_grouped, quant

    torch.manual_seed(10)
    H, I, dt = 256, 128, torch.bfloat16
    gu, dn = [], []
    for e in range(n_local):
        g = (torch.randn(I, H, device=DEV) * 0.05).to(dt)
        u = (torch.randn(I, H, device=DEV) * 0.05).to(dt)
        gu.append(quant.LinearWeight.from_dense(B.interleave_gate_up(g, u), interleaved=True))
        dn.append(quant.LinearWeight.from_dense((torch.randn(H, I, device=DEV) * 0.05).to(dt)))
    ex = MOE.ExpertWeights(E, first, gu, dn)
    x = torch.randn(T, H, device=DEV).to(dt)
    logits = torch.randn(T, E, device=DEV)
    idx, w = MOE.route_topk(logits, None, topk, 0, True)
    ref = MOE.moe_forward(x, idx, w, ex)                 # stacked is None -> per-expert loop
    ex.stacked = moe_grouped.stack_experts(ex)
    assert ex.stacked is not None
    out = moe_grouped.forward(x, idx, w, ex)
    _close(out, ref, 3e-2, 3e-2, "moe grouped")
    idx_ref, w_ref = MOE.route_topk_ref(logits, None, topk, 0, True)
    assert torch.equal(idx.sort(1)[0], idx_ref.sort(1)[0])


@pytest.mark.parametrize("kind", ["int8", "int4g128", "fp8", "nvfp4", "mxfp4"])
def test_moe_grouped_quant(kind, fp8_w8a16):
    from fastllm_b200.ops import moe as MOE, moe_grouped, quant

    torch.manual_seed(11)
    T, E, topk, H, I, dt = 40, 8, 2, 256, 128, torch.bfloat16
    gu, dn = [], []
    for e in range(E):
        g = (torch.randn(I, H, device=DEV) * 0.05).to(dt)
        u = (torch.randn(I, H, device=DEV) * 0.05).to(dt)
        gu.append(quant.LinearWeight.from_dense(B.interleave_gate_up(g, u), kind, interleaved=True, act_dtype=dt))
        dn.append(quant.LinearWeight.from_dense((torch.randn(H, I, device=DEV) * 0.05).to(dt), kind, act_dtype=dt))
    ex = MOE.ExpertWeights(E, 0, gu, dn)
    x = torch.randn(T, H, device=DEV).to(dt)
    idx, w = MOE.route_topk(torch.randn(T, E, device=DEV), None, topk, 0, True)
    ref = MOE.moe_forward(x, idx, w, ex)
    ex.stacked = moe_grouped.stack_experts(ex)
    assert ex.stacked is not None and ex.stacked.kind != "dense"
    out = moe_grouped.forward(x, idx, w, ex)
    _close(out, ref, 4e-2, 4e-2, f"moe grouped {kind}")


def _sample_ref_support(logits, temperature, top_k, top_p):
    """Per-row probabilities of the truncated distribution (plain PyTorch definition)."""
    lg = logits.float() / temperature
    V = lg.numel()
    k = top_k if 0 < top_k <= 1024 else 1024
    vals, idx = lg.topk(min(k, V))
    pr = torch.softmax(vals, -1)
    cum = pr.cumsum(-1)
    keep = (cum - pr) < top_p
    keep[0] = True
    pr = pr * keep
    pr = pr / pr.sum()
    out = torch.zeros(V, device=logits.device)
    out[idx] = pr
    return out


def test_fused_sampling_greedy_penalty_and_support():
    from fastllm_b200.engine import sampling

    torch.manual_seed(0)
    R, V = 6, 151936
    logits = torch.randn(R, V, device=DEV) * 3
    # greedy rows = arg-max, with and without a penalty that dethrones the best token
    best = logits.argmax(-1).tolist()
    lg = logits.clone()
    out = sampling.sample_fused(lg, [[] for _ in range(R)], [1.0] * R, [1] * R, [1.0] * R, [1.0] * R, uniforms=[0.3] * R)
    assert out.tolist() == best
    lg = logits.clone()
    out = sampling.sample_fused(lg, [[b] for b in best], [100.0] * R, [1] * R, [1.0] * R, [1.0] * R, uniforms=[0.3] * R)
    ref = logits.clone()
    for r, b in enumerate(best):
        ref[r, b] = ref[r, b] / 100.0 if ref[r, b] > 0 else ref[r, b] * 100.0
    assert out.tolist() == ref.argmax(-1).tolist()
    # every draw lies in the top-k / top-p support and reports that token's probability
    for (t, k, p_) in [(0.7, 40, 0.9), (1.3, 5, 1.0), (1.0, 0, 0.5), (0.5, 1000, 0.95)]:
        us = torch.rand(R).tolist()
        lg = logits.clone()
        ids, prob = sampling.sample_fused(lg, [[] for _ in range(R)], [1.0] * R, [k] * R, [p_] * R, [t] * R, uniforms=us, want_prob=True)
        for r in range(R):
            sup = _sample_ref_support(logits[r], t, k, p_)
            tok = int(ids[r])
            assert sup[tok] > 0, (t, k, p_, r)
            assert abs(float(prob[r]) - float(sup[tok])) < 1e-4 + 1e-3 * float(sup[tok])
            # inverse CDF: the draw is the first token (in descending probability order) whose cumulative mass exceeds u
            order = torch.argsort(sup, descending=True, stable=True)
            cum = sup[order].cumsum(0)
            want = int(order[int((cum <= us[r] * float(cum[-1])).sum().clamp(max=V - 1))])
            assert tok == want or abs(float(sup[tok]) - float(sup[want])) < 1e-6
    _lib.check_device_errors()


def test_fused_sampling_distribution():
    from fastllm_b200.engine import sampling

    torch.manual_seed(1)
    V = 4096
    base = torch.randn(V, device=DEV) * 2
    R = 512
    logits = base[None, :].repeat(R, 1).contiguous()
    ids = sampling.sample_fused(logits, [[] for _ in range(R)], [1.0] * R, [8] * R, [1.0] * R, [1.0] * R)
    sup = _sample_ref_support(base, 1.0, 8, 1.0)
    counts = torch.bincount(ids.long(), minlength=V).float() / R
    assert (counts[sup == 0] == 0).all()
    top = sup.topk(8)
    assert (counts[top.indices] - top.values).abs().max().item() < 0.08


def test_kernel_profile_table():
    """Per-kernel device-time table (the --profile flag): counts and non-zero times for the kernels that ran."""
    prof = _lib.start_profile()
    try:
        x = torch.randn(8, 1024, device=DEV, dtype=torch.bfloat16)
        w = torch.randn(1024, device=DEV, dtype=torch.bfloat16)
        for _ in range(3):
            B.rmsnorm(x, w, 1e-6)
        rep = prof.report()
    finally:
        _lib.stop_profile()
    assert rep["fb_rmsnorm"]["calls"] == 3 and rep["fb_rmsnorm"]["ms"] > 0


@pytest.mark.parametrize("H", [16, 4, 40, 128])
def test_mla_decode(H):
    """Absorbed MLA decode kernel vs the PyTorch evaluation over the same paged latent cache."""
    from types import SimpleNamespace

    from fastllm_b200.ops import moe as MOE

    torch.manual_seed(11)
    dt = torch.bfloat16
    lens = [1, 127, 128, 129, 700, 2049, 77, 300]
    Bn = len(lens)
    n_pages = sum((l + 127) // 128 for l in lens) + 2
    max_p = max((l + 127) // 128 for l in lens)
    pt = torch.zeros(Bn, max_p, dtype=torch.int32)
    perm = torch.randperm(n_pages)
    c = 0
    lat = torch.full((n_pages, 128, 1, 576), 3.0, dtype=dt)            # stale finite data behind the last token
    for b, l in enumerate(lens):
        n = (l + 127) // 128
        pt[b, :n] = perm[c:c + n].int()
        c += n
        for i in range(n):
            k = min(128, l - i * 128)
            lat[pt[b, i], :k, 0] = (torch.randn(k, 576) * 0.5).to(dt)
    q = (torch.randn(Bn, H, 576) * 0.5).to(dt)
    seq = torch.tensor(lens, dtype=torch.int32)
    scale = 0.07
    fb_cpu = SimpleNamespace(is_decode=False, cu_q_host=list(range(Bn + 1)), cu_q=torch.arange(Bn + 1), kv_lens=seq, page_table=pt)
    ref = MOE.mla_paged_attention(q.float(), lat.float(), fb_cpu, scale, 512)
    out = A.mla_decode(q.to(DEV), lat.to(DEV), pt.to(DEV), seq.to(DEV), scale)
    _lib.check_device_errors()
    _close(out.float().cpu(), ref, 3e-2, 3e-2, f"mla_decode H={H}")
    out2 = A.mla_decode(q.to(DEV), lat.to(DEV), pt.to(DEV), seq.to(DEV), scale)      # workspace reuse
    assert torch.equal(out, out2)


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (8, 8), (16, 1)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mma8", [True, False])
def test_attn_decode_fp8_kv(Hq, Hkv, dt, mma8, monkeypatch):
    """Decode attention over e4m3 page pools vs the PyTorch evaluation on the same e4m3 values.  ``mma8``: pages straight into
    the fp8 tensor core with two-term e4m3 queries / probabilities; else raw pages converted to fp16 operand tiles in shared
    memory."""
    monkeypatch.setattr(A, "KV8_MMA", mma8)
    torch.manual_seed(21)
    D = 128
    lens = [1, 127, 128, 129, 700, 1500, 77, 300]
    Bn = len(lens)
    n_pages = sum((l + 127) // 128 for l in lens) + 3
    max_p = max((l + 127) // 128 for l in lens)
    pt = torch.zeros(Bn, max_p, dtype=torch.int32)
    perm = torch.randperm(n_pages)
    c = 0
    k8 = torch.zeros(n_pages, 128, Hkv, D, dtype=torch.float8_e4m3fn)
    v8 = torch.zeros(n_pages, 128, Hkv, D, dtype=torch.float8_e4m3fn)
    for b, l in enumerate(lens):
        n = (l + 127) // 128
        pt[b, :n] = perm[c:c + n].int()
        c += n
        for i in range(n):
            k = min(128, l - i * 128)
            k8[pt[b, i], :k] = (torch.randn(k, Hkv, D) * 0.7).to(torch.float8_e4m3fn)
            v8[pt[b, i], :k] = torch.randn(k, Hkv, D).to(torch.float8_e4m3fn)
    q = (torch.randn(Bn, Hq * D) * 0.7).to(dt)
    seq = torch.tensor(lens, dtype=torch.int32)
    cu = torch.arange(Bn + 1, dtype=torch.int32)
    ref = A.paged_attention_general(q.float(), k8.float(), v8.float(), pt, seq, cu, D ** -0.5, Hq, Hkv, D)
    out = A.attn_decode(q.to(DEV), k8.to(DEV), v8.to(DEV), pt.to(DEV), seq.to(DEV), D ** -0.5, Hq, Hkv, D)
    _lib.check_device_errors()
    assert out.dtype == dt
    _close(out.float().cpu(), ref.float(), 2e-2, 2e-2, f"attn_decode kv8 {Hq}/{Hkv}", fro=8e-3)
    out2 = A.attn_decode(q.to(DEV), k8.to(DEV), v8.to(DEV), pt.to(DEV), seq.to(DEV), D ** -0.5, Hq, Hkv, D, window=256)
    ref2 = A.paged_attention_general(q.float(), k8.float(), v8.float(), pt, seq, cu, D ** -0.5, Hq, Hkv, D, window=256)
    _lib.check_device_errors()
    _close(out2.float().cpu(), ref2.float(), 2e-2, 2e-2, "attn_decode kv8 window", fro=8e-3)


def test_attn_prefill_fp8_kv():
    """Chunked prefill over e4m3 page pools (the pages a batch reads are de-quantised into a scratch pool for the tensor-core
    prefill kernel) vs the PyTorch evaluation on the same e4m3 values."""
    torch.manual_seed(22)
    Hq, Hkv, D, dt = 8, 2, 128, torch.bfloat16
    new = [5, 130, 64, 300]
    ctx = [5, 130, 200, 700]
    Bn = len(new)
    n_pages = sum((l + 127) // 128 for l in ctx) + 2
    max_p = max((l + 127) // 128 for l in ctx)
    pt = torch.zeros(Bn, max_p, dtype=torch.int32)
    perm = torch.randperm(n_pages)
    c = 0
    k8 = torch.zeros(n_pages, 128, Hkv, D, dtype=torch.float8_e4m3fn)
    v8 = torch.zeros(n_pages, 128, Hkv, D, dtype=torch.float8_e4m3fn)
    for b, l in enumerate(ctx):
        n = (l + 127) // 128
        pt[b, :n] = perm[c:c + n].int()
        c += n
        for i in range(n):
            k = min(128, l - i * 128)
            k8[pt[b, i], :k] = (torch.randn(k, Hkv, D) * 0.7).to(torch.float8_e4m3fn)
            v8[pt[b, i], :k] = torch.randn(k, Hkv, D).to(torch.float8_e4m3fn)
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32)
    q = (torch.randn(sum(new), Hq * D) * 0.7).to(dt)
    seq = torch.tensor(ctx, dtype=torch.int32)
    ref = A.paged_attention_general(q.float(), k8.float(), v8.float(), pt, seq, cu, D ** -0.5, Hq, Hkv, D)
    out = A.attn_prefill(q.to(DEV), k8.to(DEV), v8.to(DEV), pt.to(DEV), seq.to(DEV), cu.to(DEV), D ** -0.5, Hq, Hkv, D,
                         cu_q_host=cu.tolist())
    _close(out.float().cpu(), ref.float(), 2e-2, 2e-2, "attn_prefill kv8", fro=8e-3)


def test_mla_prefill_on_gemm_kernels():
    """Absorbed MLA prefill (heads folded into GEMM rows, both contractions on the tensor-core GEMM kernels, chunked prefill
    with earlier context) vs the fp32 evaluation."""
    from types import SimpleNamespace

    from fastllm_b200.ops import moe as MOE

    torch.manual_seed(12)
    dt = torch.bfloat16
    H = 16
    new = [5, 130, 64, 300]                  # new tokens per request
    ctx = [5, 130, 200, 1000]                # total length after this chunk (>= new: the third and fourth continue a context)
    Bn = len(new)
    n_pages = sum((l + 127) // 128 for l in ctx) + 1
    max_p = max((l + 127) // 128 for l in ctx)
    pt = torch.zeros(Bn, max_p, dtype=torch.int32)
    perm = torch.randperm(n_pages)
    c = 0
    lat = torch.full((n_pages, 128, 1, 576), 2.0, dtype=dt)
    for b, l in enumerate(ctx):
        n = (l + 127) // 128
        pt[b, :n] = perm[c:c + n].int()
        c += n
        for i in range(n):
            k = min(128, l - i * 128)
            lat[pt[b, i], :k, 0] = (torch.randn(k, 576) * 0.5).to(dt)
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    q = (torch.randn(cu[-1], H, 576) * 0.5).to(dt)
    seq = torch.tensor(ctx, dtype=torch.int32)
    mk = lambda dev: SimpleNamespace(is_decode=False, cu_q_host=cu, cu_q=torch.tensor(cu), kv_lens=seq.to(dev), page_table=pt.to(dev))
    ref = MOE.mla_paged_attention(q.float(), lat.float(), mk("cpu"), 0.07, 512)
    out = MOE.mla_paged_attention(q.to(DEV), lat.to(DEV), mk(DEV), 0.07, 512)
    _lib.check_device_errors()
    _close(out.float().cpu(), ref, 3e-2, 3e-2, "mla prefill on GEMM kernels", fro=1e-2)


def _fp8_ref(x, lw):
    """What the W8A8 kernel computes: activations rounded to e4m3 per (token, 128-wide k block), weights as stored."""
    from fastllm_b200.ops import quant as Q

    M, K = x.shape
    xb = x.float().reshape(M, K // 128, 128)
    sc = (xb.abs().amax(-1, keepdim=True).clamp(min=1e-12) / 448.0)
    xq = (xb / sc).to(torch.float8_e4m3fn).float() * sc
    w = Q.dequantize_fp8_block(lw.w, lw.scale, torch.float32, 128)
    return xq.reshape(M, K) @ w.t()


@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (16, 384, 1024), (64, 4096, 4096), (100, 1024, 14336), (128, 512, 2048)])
def test_gemm_fp8_native(M, N, K):
    from fastllm_b200.ops import quant as Q
    from fastllm_b200.ops import quant_gemm as QG

    torch.manual_seed(M + N)
    dt = torch.bfloat16
    w = (torch.randn(N, K, device=DEV) * 0.03).to(dt)
    lw = Q.LinearWeight.from_dense(w, "fp8")
    x = torch.randn(M, K, device=DEV).to(dt)
    assert QG.FP8_NATIVE
    out = lw(x)
    ref = _fp8_ref(x, lw)
    _lib.check_device_errors()
    _close(out.float().cpu(), ref.cpu(), 2e-2, 1e-2, f"gemm_fp8 {M}x{N}x{K}")
    # and it stays close to the un-quantised product
    exact = x.float() @ w.float().t()
    rel = (out.float() - exact).norm() / exact.norm()
    assert rel < 0.06, rel


def test_gemm_fp8_native_epilogues():
    from fastllm_b200.ops import quant as Q

    torch.manual_seed(9)
    dt = torch.bfloat16
    M, K, I = 48, 1024, 512
    g, u = (torch.randn(I, K, device=DEV) * 0.03).to(dt), (torch.randn(I, K, device=DEV) * 0.03).to(dt)
    lw = Q.LinearWeight.from_dense(B.interleave_gate_up(g, u), "fp8", interleaved=True)
    x = torch.randn(M, K, device=DEV).to(dt)
    out = lw(x, swiglu=True)
    full = _fp8_ref(x, lw)                                  # interleaved columns
    t = full.reshape(M, (2 * I) // 128, 2, 64)
    ref = (torch.nn.functional.silu(t[:, :, 0]) * t[:, :, 1]).reshape(M, I)
    _close(out.float().cpu(), ref.cpu(), 3e-2, 2e-2, "gemm_fp8 swiglu")
    wd = (torch.randn(K, I, device=DEV) * 0.03).to(dt)
    ld = Q.LinearWeight.from_dense(wd, "fp8", bias=torch.randn(K, device=DEV).to(dt))
    res = torch.randn(M, K, device=DEV).to(dt)
    a = torch.randn(M, I, device=DEV).to(dt)
    out2 = ld(a, residual=res)
    ref2 = _fp8_ref(a, ld) + ld.bias.float() + res.float()
    _close(out2.float().cpu(), ref2.cpu(), 3e-2, 2e-2, "gemm_fp8 bias+residual")
    _lib.check_device_errors()


def test_moe_grouped_fp8_native_matches_w8a16():
    """Grouped expert GEMMs with FP8 activations vs the 16-bit-activation path on the same FP8 expert weights."""
    from fastllm_b200.models.config import preset
    from fastllm_b200.models.decoder import random_init
    from fastllm_b200.ops import moe as MOE
    from fastllm_b200.ops import quant_gemm as QG

    cfg = preset("tiny-qwen3-moe")
    m = random_init(cfg, "cuda", torch.bfloat16, std=0.05, moe_wdtype="fp8")
    ex = m.layers[0].mlp.experts
    assert ex.stacked is not None and ex.stacked.kind == "fp8"
    torch.manual_seed(3)
    x = torch.randn(37, cfg.hidden_size, device=DEV).bfloat16()
    idx, w = MOE.route_topk(torch.randn(37, cfg.num_experts, device=DEV), None, 2, 0, True)
    y8 = MOE.moe_forward(x, idx, w, ex)
    QG.FP8_NATIVE = False
    try:
        y16 = MOE.moe_forward(x, idx, w, ex)
    finally:
        QG.FP8_NATIVE = True
    _lib.check_device_errors()
    rel = (y8.float() - y16.float()).norm() / y16.float().norm()
    assert rel < 0.08, rel


@pytest.mark.parametrize("M,E,K,topk,mode,renorm,bias", [(128, 128, 2048, 8, 0, True, False), (37, 64, 512, 6, 1, True, True),
                                                         (1, 128, 4096, 8, 0, False, False), (16, 8, 256, 2, 0, True, False),
                                                         (100, 96, 1024, 4, 1, False, True)])
def test_router_gemm_with_selection_epilogue(M, E, K, topk, mode, renorm, bias):
    """Router projection + expert selection in one launch against the two-launch path (tensor-core GEMM to fp32 logits, then the
    selection kernel) and against the PyTorch definition on the same logits."""
    from fastllm_b200.ops import moe as MOE

    torch.manual_seed(M + E)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(E, K, device=DEV) * 0.05).bfloat16()
    b = torch.randn(E, device=DEV) * 0.1 if bias else None
    idx, wt = MOE.route_fused(x, w, b, topk, mode, renorm, 2.5)
    torch.cuda.synchronize()
    _lib.check_device_errors()
    logits = B.linear(x, w, out_f32=True)
    idx2, wt2 = MOE.route_topk(logits, b, topk, mode, renorm, 1, 1, 2.5)
    idx3, wt3 = MOE.route_topk_ref(x.float() @ w.float().t(), b, topk, mode, renorm, 1, 1, 2.5)
    # the k-split partial sums are added in another order than the unfused GEMM's: near-ties may swap, so compare as sets
    # with a small allowance and the weights of the common experts
    same = sum(len(set(a.tolist()) & set(c.tolist())) for a, c in zip(idx.cpu(), idx2.cpu()))
    assert same >= 0.98 * M * topk, same
    same3 = sum(len(set(a.tolist()) & set(c.tolist())) for a, c in zip(idx.cpu(), idx3.cpu()))
    assert same3 >= 0.97 * M * topk, same3
    d1 = torch.zeros(M, E, device=DEV).scatter_(1, idx.long(), wt)
    d2 = torch.zeros(M, E, device=DEV).scatter_(1, idx2.long(), wt2)
    rows = ((d1 != 0) == (d2 != 0)).all(dim=1)              # tokens whose selection is the same in both paths
    assert rows.float().mean() > 0.9
    assert torch.allclose(d1[rows], d2[rows], rtol=2e-3, atol=1e-5)


@pytest.mark.parametrize("T,topk,E,first,n_local,pad", [(128, 8, 128, 0, 128, 4), (37, 2, 8, 0, 8, 4), (100, 8, 256, 64, 32, 16),
                                                        (512, 8, 64, 0, 64, 4), (1, 6, 160, 0, 160, 1), (700, 8, 16, 8, 8, 4), (400, 8, 128, 0, 128, 4)])
def test_moe_plan_matches_definition(T, topk, E, first, n_local, pad):
    """Routing plan: per local expert the row count, the padded segment start, and for every (token, k) pair its row = segment
    start + number of earlier pairs of the same expert (-1 for experts of other ranks).  Covers the warp-vote kernel, the
    shared-memory kernel (pairs * experts beyond its table) and the one-thread-per-expert kernel (> 4096 pairs)."""
    from fastllm_b200.ops import moe_grouped  # noqa: F401  (registers the launcher signatures)

    lib = _lib.kernels()
    g = torch.Generator().manual_seed(T + E)
    idx = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]).int().to(DEV)
    counts = torch.zeros(n_local, dtype=torch.int32, device=DEV)
    offsets = torch.zeros(n_local, dtype=torch.int32, device=DEV)
    pos = torch.full((T * topk,), -7, dtype=torch.int32, device=DEV)
    total = torch.zeros(1, dtype=torch.int32, device=DEV)
    _lib.check(lib.fb_moe_plan(idx.data_ptr(), T, topk, first, n_local, counts.data_ptr(), offsets.data_ptr(), pos.data_ptr(),
                               total.data_ptr(), pad, torch.cuda.current_stream().cuda_stream), "fb_moe_plan")
    torch.cuda.synchronize()
    flat = idx.flatten().cpu().tolist()
    want_cnt = [0] * n_local
    want_rank = []
    for e in flat:
        l = e - first
        if 0 <= l < n_local:
            want_rank.append((l, want_cnt[l]))
            want_cnt[l] += 1
        else:
            want_rank.append(None)
    off, acc = [], 0
    for c in want_cnt:
        off.append(acc)
        acc += (c + pad - 1) // pad * pad
    assert counts.cpu().tolist() == want_cnt and offsets.cpu().tolist() == off and int(total) == acc
    assert pos.cpu().tolist() == [-1 if r is None else off[r[0]] + r[1] for r in want_rank]


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("tiles", [0, 3, 4, 8])
def test_moe_grouped_fp8_tiles_per_cta(tiles, swiglu):
    """The grouped FP8 projections (plain: an expert's down projection; SwiGLU: its gate / up projection) with several output
    tiles per CTA give the bits of the one-tile-per-CTA launch (same accumulation order), and both match an fp32 reference of
    the de-quantised operands."""
    from fastllm_b200.ops import quant_gemm as QG

    torch.manual_seed(5)
    E, N, K = 8, 1024, 256
    lib = _lib.kernels()
    w = torch.randn(E * N, K, device=DEV) * 0.05
    wb = w.reshape(E * N // 128, 128, K // 128, 128)
    ws = (wb.abs().amax((1, 3)) / 448.0).clamp(min=1e-12).contiguous()          # (row blocks, k blocks)
    wq = (wb / ws[:, None, :, None]).reshape(E * N, K).to(torch.float8_e4m3fn).contiguous()
    counts = torch.tensor([0, 30, 1, 17, 74, 3, 0, 25], device=DEV, dtype=torch.int32)
    padded = (counts + 3) // 4 * 4          # the routing plan starts every expert's segment on a multiple of four rows (16-byte scale rows)
    offsets = (torch.cumsum(padded, 0) - padded).int()
    rows = int(padded.sum())
    x = torch.randn(rows, K, device=DEV).bfloat16()
    xq, sa, ld_a = QG.quant_act_fp8(x)
    xd = (xq.view(torch.float8_e4m3fn).float().reshape(rows, K // 128, 128) * sa[:, :rows].t()[:, :, None]).reshape(rows, K)
    wd = (wq.float().reshape(E * N // 128, 128, K // 128, 128) * ws[:, None, :, None]).reshape(E, N, K)
    ref = torch.zeros(rows, N, device=DEV)
    for e in range(E):
        o, c = int(offsets[e]), int(counts[e])
        ref[o:o + c] = xd[o:o + c] @ wd[e].t()
    if swiglu:                                  # a 128-row tile holds 64 gate rows, then the 64 up rows of the same output columns
        r4 = ref.reshape(rows, N // 128, 2, 64)
        ref = (torch.nn.functional.silu(r4[:, :, 0]) * r4[:, :, 1]).reshape(rows, N // 2)
    n_out = ref.shape[1]

    def run(t):
        old = lib.fb_moe_grouped_fp8_set_tiles(t)
        out = torch.zeros(rows, n_out, device=DEV, dtype=torch.bfloat16)
        try:
            _lib.check(lib.fb_moe_grouped_gemm_fp8(xq.data_ptr(), K, sa.data_ptr(), ld_a, wq.data_ptr(), ws.data_ptr(), out.data_ptr(),
                                                   counts.data_ptr(), offsets.data_ptr(), E, N, K, rows, n_out, 1, 4 if swiglu else 0, 74, rows,
                                                   torch.cuda.current_stream().cuda_stream), "grouped fp8")
        finally:
            lib.fb_moe_grouped_fp8_set_tiles(old)
        torch.cuda.synchronize()
        _lib.check_device_errors()
        return out

    base = run(1)
    _close(base.float().cpu(), ref.cpu(), 2e-2, 2e-2, "grouped fp8 one tile")
    assert torch.equal(run(tiles), base)


def _i8_act(x):
    M, K = x.shape
    xb = x.float().reshape(M, K // 128, 128)
    sc = xb.abs().amax(-1, keepdim=True).clamp(min=1e-12) / 127.0
    return (torch.round(xb / sc).clamp(-127, 127) * sc).reshape(M, K)


@pytest.mark.parametrize("kind", ["int8", "int4g128"])
@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (16, 384, 1024), (64, 4096, 4096), (100, 1024, 14336), (128, 520, 2048), (300, 1024, 2048)])
def test_gemm_int_a8(kind, M, N, K):
    """Integer tensor-core path: int8 activations x int8 / int4-group weights vs the same quantised operands in fp32."""
    from fastllm_b200.ops import quant as Q
    from fastllm_b200.ops import quant_gemm as QG

    torch.manual_seed(M + N)
    dt = torch.bfloat16
    w = (torch.randn(N, K, device=DEV) * 0.03).to(dt)
    lw = Q.LinearWeight.from_dense(w, kind)
    wdq = lw.dequant(torch.float32)
    x = torch.randn(M, K, device=DEV).to(dt)
    assert QG.uses_int_a8(lw)
    old, QG.INT_A8_MAX_M = QG.INT_A8_MAX_M, {"int8": 512, "int4g": 512}          # also the 128-row chunk loop
    try:
        out = lw(x)
    finally:
        QG.INT_A8_MAX_M = old
    _lib.check_device_errors()
    ref = _i8_act(x) @ wdq.t()
    _close(out.float().cpu(), ref.cpu(), 2e-2, 1e-2, f"gemm_i8 {kind} {M}x{N}x{K}")
    assert torch.allclose(lw.dequant(torch.float32), wdq)          # int8 storage switched to q - 128 without changing the values
    exact = x.float() @ w.float().t()
    rel = (out.float() - exact).norm() / exact.norm()
    assert rel < (0.03 if kind == "int8" else 0.15), rel


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(256, 512), (4096, 7168), (7168, 2048), (384, 1536)])
def test_gemv_int4_dp4a(M, N, K):
    """int4-group weights at one to four rows (CUDA-core dp4a kernel) vs fp32 on the same quantised operands, and vs the
    tensor-core route; plain and SwiGLU (interleaved gate / up) outputs."""
    from fastllm_b200.ops import quant as Q
    from fastllm_b200.ops import quant_gemm as QG

    torch.manual_seed(M * 7 + N)
    dt = torch.bfloat16
    x = torch.randn(M, K, device=DEV).to(dt)
    w = (torch.randn(N, K, device=DEV) * 0.03).to(dt)
    lw = Q.LinearWeight.from_dense(w, "int4g128")
    assert QG.I4_GEMV and QG.uses_int_a8(lw)
    out = lw(x)
    ref = _i8_act(x) @ lw.dequant(torch.float32).t()
    _close(out.float(), ref, 2e-2, 1e-2, f"gemv_i4 {M}x{N}x{K}", fro=5e-3)
    QG.I4_GEMV = False
    try:
        tc = lw(x)
    finally:
        QG.I4_GEMV = True
    _close(out.float(), tc.float(), 2e-2, 1e-2, "gemv_i4 vs tensor-core route", fro=5e-3)
    if N % 256 == 0:
        I = N // 2
        g, u = w[:I], w[I:]
        lg = Q.LinearWeight.from_dense(B.interleave_gate_up(g, u), "int4g128", interleaved=True)
        o2 = lg(x, swiglu=True)
        full = _i8_act(x) @ lg.dequant(torch.float32).t()
        t = full.reshape(M, N // 128, 2, 64)
        r2 = (torch.nn.functional.silu(t[:, :, 0]) * t[:, :, 1]).reshape(M, I)
        _close(o2.float(), r2, 3e-2, 2e-2, "gemv_i4 swiglu", fro=8e-3)
    _lib.check_device_errors()


def test_gemm_int_a8_epilogues():
    from fastllm_b200.ops import quant as Q

    torch.manual_seed(9)
    dt = torch.bfloat16
    M, K, I = 48, 1024, 512
    g, u = (torch.randn(I, K, device=DEV) * 0.03).to(dt), (torch.randn(I, K, device=DEV) * 0.03).to(dt)
    x = torch.randn(M, K, device=DEV).to(dt)
    for kind in ("int8", "int4g128"):
        lw = Q.LinearWeight.from_dense(B.interleave_gate_up(g, u), kind, interleaved=True)
        out = lw(x, swiglu=True)
        full = _i8_act(x) @ lw.dequant(torch.float32).t()
        t = full.reshape(M, (2 * I) // 128, 2, 64)
        ref = (torch.nn.functional.silu(t[:, :, 0]) * t[:, :, 1]).reshape(M, I)
        _close(out.float().cpu(), ref.cpu(), 3e-2, 2e-2, f"gemm_i8 swiglu {kind}")
        wd = (torch.randn(K, I, device=DEV) * 0.03).to(dt)
        ld = Q.LinearWeight.from_dense(wd, kind, bias=torch.randn(K, device=DEV).to(dt))
        res = torch.randn(M, K, device=DEV).to(dt)
        a = torch.randn(M, I, device=DEV).to(dt)
        out2 = ld(a, residual=res)
        ref2 = _i8_act(a) @ ld.dequant(torch.float32).t() + ld.bias.float() + res.float()
        _close(out2.float().cpu(), ref2.cpu(), 3e-2, 2e-2, f"gemm_i8 bias+residual {kind}")
    _lib.check_device_errors()


@pytest.mark.parametrize("kind", ["int8", "int4g128"])
def test_moe_grouped_int_a8(kind):
    """Grouped expert GEMMs on the integer tensor-core path vs the per-expert 16-bit evaluation of the same quantised weights."""
    from fastllm_b200.models.config import preset
    from fastllm_b200.models.decoder import random_init
    from fastllm_b200.ops import moe as MOE
    from fastllm_b200.ops import quant_gemm as QG

    cfg = preset("tiny-qwen3-moe")
    m = random_init(cfg, "cuda", torch.bfloat16, std=0.05, moe_wdtype=kind)
    ex = m.layers[0].mlp.experts
    assert ex.stacked is not None
    torch.manual_seed(4)
    for T in (1, 5, 150):          # few rows per expert: int4 experts run the dp4a kernel, int8 and large batches the tensor core
        x = torch.randn(T, cfg.hidden_size, device=DEV).bfloat16()
        idx, w = MOE.route_topk(torch.randn(T, cfg.num_experts, device=DEV), None, 2, 0, True)
        if T == 5:
            idx[:, 0] = 3          # one expert with five rows: a second pass of four over its weight tiles
        y8 = MOE.moe_forward(x, idx, w, ex)
        assert ex.stacked.a8 is not None and (kind != "int8" or ex.stacked.signed)
        QG.INT_A8 = False              # the 16-bit-activation kernels on the same (now q - 128) bytes
        try:
            y16 = MOE.moe_forward(x, idx, w, ex)
        finally:
            QG.INT_A8 = True
        _lib.check_device_errors()
        rel = (y8.float() - y16.float()).norm() / y16.float().norm()
        assert rel < 0.03, (T, rel)


@pytest.mark.parametrize("mode", [0, 1])
def test_round_act(mode):
    """Activation rounding kernel (int8 / e4m3 grid per token and 128-wide block) vs the PyTorch definition."""
    from fastllm_b200.ops import quant_gemm as QG

    torch.manual_seed(mode)
    x = (torch.randn(37, 1024, device=DEV) * 3).bfloat16()
    got = QG.round_act(x, mode).float()
    xb = x.float().reshape(37, 8, 128)
    if mode == 0:
        sc = xb.abs().amax(-1, keepdim=True).clamp(min=1e-12) / 127.0
        ref = torch.round(xb / sc) * sc
    else:
        sc = xb.abs().amax(-1, keepdim=True).clamp(min=1e-12) / 448.0
        ref = (xb / sc).to(torch.float8_e4m3fn).float() * sc
    ref = ref.reshape(37, 1024).bfloat16().float()
    # x * (1 / s) vs x / s can land on the other side of a rounding boundary for a few elements: one grid step there at most
    step = (sc * (1.0 if mode == 0 else 32.0)).expand(37, 8, 128).reshape(37, 1024)
    assert ((got - ref).abs() <= step * 1.01 + ref.abs() / 64 + 1e-6).all()          # + bf16 rounding of both sides
    assert ((got - ref).abs() > 1e-6).float().mean() < 0.01
    _lib.check_device_errors()


@pytest.mark.parametrize("mode", [1, 2])
def test_rmsnorm_fused_quant(mode):
    """RMSNorm with the activation quantiser fused in: same 16-bit output as the plain norm, same bytes / scales / block sums as
    the stand-alone quantiser applied to that output."""
    from fastllm_b200.ops import quant_gemm as QG

    torch.manual_seed(mode)
    for M, H in ((1, 1024), (37, 4096), (64, 2048)):
        x = torch.randn(M, H, device=DEV).bfloat16()
        w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
        y0 = B.rmsnorm(x, w, 1e-5)
        y = B.rmsnorm(x, w, 1e-5, quant_mode=mode)
        assert torch.equal(y, y0)
        m, xq, sa, xs, ld_a = y.fb_quant
        assert m == mode
        if mode == 1:
            rq, rsa, rxs, _ = QG.quant_act_i8(y0)
            assert torch.equal(xq, rq) and torch.equal(sa[:, :M], rsa[:, :M]) and torch.equal(xs[:, :M], rxs[:, :M])
        else:
            rq, rsa, _ = QG.quant_act_fp8(y0)
            assert torch.equal(xq, rq) and torch.equal(sa[:, :M], rsa[:, :M])
    _lib.check_device_errors()


@pytest.mark.parametrize("mode", [3, 4])
def test_rmsnorm_fused_rounding(mode):
    """RMSNorm whose output is rounded to the int8 / e4m3 grid in the same launch == plain norm followed by the rounding kernel."""
    from fastllm_b200.ops import quant_gemm as QG

    torch.manual_seed(mode)
    for M, H in ((3, 1024), (300, 4096)):
        x = torch.randn(M, H, device=DEV).bfloat16()
        w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
        want = QG.round_act(B.rmsnorm(x, w, 1e-5), mode - 3)
        got = B.rmsnorm(x, w, 1e-5, quant_mode=mode)
        assert got.fb_quant[0] == mode
        assert torch.equal(got, want)
    _lib.check_device_errors()


@pytest.mark.parametrize("mode", [1, 2])
def test_attn_decode_fused_quant(mode):
    """Decode attention whose combine also quantises the output for the output projection: same 16-bit output, same bytes /
    scales / block sums as the stand-alone quantiser applied to it."""
    from fastllm_b200.ops import quant_gemm as QG

    torch.manual_seed(6)
    Hq, Hkv, D, dt = 8, 2, 128, torch.bfloat16
    lens = [1, 127, 129, 300, 1025]
    Bn = len(lens)
    k_pool, v_pool, pt = _make_cache(Bn, lens, Hkv, D, dt)
    q = torch.randn(Bn, Hq * D).to(dt)
    seq = torch.tensor(lens, dtype=torch.int32)
    args = (q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), pt.to(DEV), seq.to(DEV), 1 / math.sqrt(D), Hq, Hkv, D)
    plain = A.attn_decode(*args)
    out = A.attn_decode(*args, quant_mode=mode)
    assert torch.equal(out, plain)
    m, xq, sa, xs, ld_a = out.fb_quant
    assert m == mode
    if mode == 1:
        rq, rsa, rxs, _ = QG.quant_act_i8(plain)
        assert torch.equal(xq, rq) and torch.equal(sa[:, :Bn], rsa[:, :Bn]) and torch.equal(xs[:, :Bn], rxs[:, :Bn])
    else:
        rq, rsa, _ = QG.quant_act_fp8(plain)
        assert torch.equal(xq, rq) and torch.equal(sa[:, :Bn], rsa[:, :Bn])
    _lib.check_device_errors()


def test_peer_wait_runs_out_and_is_reported():
    """A fused collective whose peer never arrives: the bounded wait gives up, the kernel returns, the error word says
    "peer timeout", and after the header is cleared a correct launch works.  The missing rank is a second arena on the same
    GPU that nothing ever launches on -- every address the kernel touches is valid local memory, nothing faults."""
    import ctypes

    from fastllm_b200.parallel import symm  # noqa: F401  (registers the signatures of the collective kernels)

    lib = _lib.kernels()
    M, N = 4, 1024
    dt = torch.bfloat16
    off_part, off_h, off_x = 4096, 4096 + 2 * M * N * 4, 4096 + 2 * M * N * 4 + M * N * 2
    nbytes = off_x + M * N * 2 + 4096
    arena = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    ghost = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)         # the rank that never launches
    part = torch.randn(M, N, device=DEV)
    h0 = torch.randn(M, N, device=DEV).to(dt)
    ln = (1 + 0.1 * torch.randn(N, device=DEV)).to(dt)
    hv = arena[off_h:off_h + M * N * 2].view(dt).view(M, N)
    xv = arena[off_x:off_x + M * N * 2].view(dt).view(M, N)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def peers(*ts):
        return (ctypes.c_void_p * 8)(*([ctypes.c_void_p(t.data_ptr()) for t in ts] + [ctypes.c_void_p(0)] * (8 - len(ts))))

    def launch(tp, pp):
        return lib.fb_ar_norm(part.data_ptr(), 1, M, N, ctypes.c_void_p(arena.data_ptr()), ctypes.c_void_p(0), pp, 0, tp,
                              off_part, off_h, off_x, ln.data_ptr(), 1, 1e-5, 0.0, 1, stream)

    _lib.set_wait_limit_ns(20_000_000)                 # 20 ms instead of 2 s
    try:
        hv.copy_(h0)
        assert launch(2, peers(arena, ghost)) == 0
        torch.cuda.synchronize()                        # the kernel ended by itself
        with pytest.raises(_lib.DeviceKernelError, match="code=2"):
            _lib.check_device_errors()
        # recovery: clear the arena header (what FusedComm.reset does on every rank), then a complete group of one rank
        arena[:1024].zero_()
        hv.copy_(h0)
        assert launch(1, peers(arena)) == 0
        torch.cuda.synchronize()
        _lib.check_device_errors()
        ref_h = (part + h0.float()).to(dt)
        _close(hv, ref_h, 2e-2, 2e-2, "h after recovery")
        _close(xv, B.rmsnorm_ref(ref_h, ln, 1e-5)[0], 3e-2, 3e-2, "x after recovery")
    finally:
        _lib.set_wait_limit_ns(2_000_000_000)


@pytest.mark.parametrize("mode,rot,qknorm,bias", [(A.ROPE_NEOX, 128, True, False), (A.ROPE_NEOX, 64, False, True),
                                                  (A.ROPE_INTERLEAVED, 128, False, False), (A.ROPE_NONE, 128, True, True)])
@pytest.mark.parametrize("T,K", [(1, 256), (21, 1024), (64, 4096), (200, 512)])
def test_qkv_projection_with_fused_post(mode, rot, qknorm, bias, T, K):
    """QKV GEMM whose epilogue does split + per-head norm + RoPE + cache append, against the PyTorch fp32 definition of the
    projection followed by the PyTorch definition of the post-processing."""
    from fastllm_b200.ops.quant import LinearWeight

    torch.manual_seed(17)
    Hq, Hkv, D, dt = 8, 2, 128, torch.bfloat16
    N = (Hq + 2 * Hkv) * D
    x = (torch.randn(T, K) * 0.5).to(dt)
    w = (torch.randn(N, K) * 0.05).to(dt)
    b = torch.randn(N).to(dt) if bias else None
    pos = torch.randint(0, 500, (T,), dtype=torch.int32)
    slots = torch.randperm(4 * 128)[:T].int()
    if T > 3:
        slots[3] = -1
    cos, sin = A.build_rope_tables(rot, 512, 10000.0)
    qn = (1 + 0.1 * torch.randn(D)).to(dt) if qknorm else None
    kn = (1 + 0.1 * torch.randn(D)).to(dt) if qknorm else None
    kp, vp = torch.zeros(4, 128, Hkv, D, dtype=dt), torch.zeros(4, 128, Hkv, D, dtype=dt)
    qkv_ref = B.linear_ref(x, w, bias=b)
    q_ref = A.qkv_post(qkv_ref, pos, slots, kp, vp, Hq, Hkv, D, cos, sin, mode, rot, qn, kn, 1e-6)
    kp2, vp2 = torch.zeros_like(kp).to(DEV), torch.zeros_like(vp).to(DEV)
    lw = LinearWeight.from_dense(w.to(DEV), bias=b.to(DEV) if bias else None)
    d = lambda t: t.to(DEV) if t is not None else None
    q_out = A.qkv_proj_post(x.to(DEV), lw, pos.to(DEV), slots.to(DEV), kp2, vp2, Hq, Hkv, D, cos.to(DEV), sin.to(DEV), mode, rot,
                            d(qn), d(kn), 1e-6)
    assert q_out is not None, "fused QKV kernel refused a supported shape"
    _close(q_out.cpu(), q_ref, 4e-2, 3e-2, "q", fro=2e-2)
    _close(kp2.cpu(), kp, 4e-2, 3e-2, "k pool", fro=2e-2)
    _close(vp2.cpu(), vp, 3e-2, 2e-2, "v pool", fro=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gdn_conv_update_and_recurrent_step(dtype):
    """Gated-DeltaNet decode kernels (convolution window step; delta-rule step + gated norm) against the PyTorch fp32
    definition, over three consecutive steps so the carried state is checked too."""
    from fastllm_b200.ops import linear_attn as L

    torch.manual_seed(23)
    Bn, Hk, Hv, Dk, Dv, K = 5, 2, 4, 128, 128, 4
    C = 2 * Hk * Dk + Hv * Dv
    n_slots = 9
    slots = torch.tensor([7, 2, 8, 0, 3], dtype=torch.int32)
    w = (torch.randn(C, K) * 0.4).to(dtype)
    conv_ref = (torch.randn(n_slots, C, K - 1) * 0.5).to(dtype)
    rec_ref = torch.randn(n_slots, Hv, Dk, Dv) * 0.1
    A_log, dt_bias = torch.log(torch.rand(Hv) * 4 + 0.5), torch.rand(Hv)
    norm_w = (1 + 0.1 * torch.randn(Dv)).to(dtype)
    conv_g, rec_g = conv_ref.clone().to(DEV), rec_ref.clone().to(DEV)
    d = lambda t: t.to(DEV)
    for step in range(3):
        x = (torch.randn(Bn, C) * 0.7).to(dtype)
        a, b = torch.randn(Bn, Hv).to(dtype), torch.randn(Bn, Hv).to(dtype)
        z = torch.randn(Bn, Hv * Dv).to(dtype)
        y_ref = L.causal_conv1d_decode(x, w, conv_ref, slots)                       # CPU tensors: the PyTorch definition
        o_ref = L.gated_delta_decode(y_ref, a, b, z, A_log, dt_bias, norm_w, 1e-6, rec_ref, slots, Hk, Hv, Dk, Dv)
        y = L.causal_conv1d_decode(d(x), d(w), conv_g, d(slots))
        _close(y.cpu(), y_ref, 2e-2, 2e-2, f"conv step {step}")
        o = L.gated_delta_decode(d(y_ref), d(a), d(b), d(z), d(A_log), d(dt_bias), d(norm_w), 1e-6, rec_g, d(slots), Hk, Hv, Dk, Dv)
        _close(o.cpu(), o_ref, 3e-2, 3e-2, f"delta step {step}", fro=2e-2)
        _close(conv_g.cpu(), conv_ref, 0, 0, f"conv state {step}")
        _close(rec_g.cpu(), rec_ref, 1e-3, 1e-3, f"rule state {step}", fro=1e-3)
    untouched = [s for s in range(n_slots) if s not in slots.tolist()]
    assert torch.equal(rec_g.cpu()[untouched], rec_ref[untouched])


@pytest.mark.parametrize("M,batch,N,K,x_cols,out_cols", [(1, 4, 512, 128, 192, 576), (37, 16, 512, 128, 192, 576), (64, 8, 128, 512, 512, 128),
                                                        (200, 3, 72, 64, 64, 80), (300, 2, 128, 128, 128, 128)])
def test_gemm_batched_per_head(M, batch, N, K, x_cols, out_cols):
    """One launch, one small GEMM per head: strided activation slices in, strided output slices out (MLA absorb shapes)."""
    torch.manual_seed(19)
    dt = torch.bfloat16
    x = (torch.randn(M, batch * x_cols, device=DEV) * 0.5).to(dt)
    w = (torch.randn(batch, N, K, device=DEV) * 0.08).to(dt)
    out = torch.full((M, batch * out_cols), 7.0, device=DEV, dtype=dt)
    B.linear_batched(x, w, batch, x_cols, out, out_cols)
    ref = torch.einsum("mzk,znk->mzn", x.view(M, batch, x_cols)[..., :K].float(), w.float())
    got = out.view(M, batch, out_cols)
    _close(got[..., :N], ref, 3e-2, 2e-2, "batched gemm", fro=1e-2)
    if out_cols > N:
        assert bool((got[..., N:] == 7.0).all()), "columns outside a head's N outputs were written"


@pytest.mark.parametrize("mode", [A.ROPE_INTERLEAVED, A.ROPE_NEOX])
def test_mla_post_kernel(mode):
    """Latent RMSNorm + shared-key RoPE into the cache entry and per-head query RoPE, against the PyTorch definition."""
    torch.manual_seed(21)
    T, H, nope, rope, lora, dt = 19, 6, 128, 64, 512, torch.bfloat16
    ckv = torch.randn(T, lora + rope).to(dt)
    q = torch.randn(T, H * (nope + rope)).to(dt)
    pos = torch.randint(0, 400, (T,), dtype=torch.int32)
    slots = torch.randperm(3 * 128)[:T].int()
    slots[5] = -1
    nw = (1 + 0.1 * torch.randn(lora)).to(dt)
    cos, sin = A.build_rope_tables(rope, 512, 10000.0)
    pool_c = torch.zeros(3 + 1, 128, 1, lora + rope, dtype=dt)
    qf_c = torch.zeros(T, H, lora + rope, dtype=dt)
    A.mla_post(ckv, q, qf_c, pool_c, pos, slots, nw, cos, sin, H, nope, rope, lora, mode, 1e-6)       # CPU tensors: PyTorch path
    pool_g = torch.zeros_like(pool_c).to(DEV)
    qf_g = torch.zeros_like(qf_c).to(DEV)
    d = lambda t: t.to(DEV)
    A.mla_post(d(ckv), d(q), qf_g, pool_g, d(pos), d(slots), d(nw), d(cos), d(sin), H, nope, rope, lora, mode, 1e-6)
    _close(qf_g.cpu()[..., lora:], qf_c[..., lora:], 3e-2, 2e-2, "q rope")
    flat_g, flat_c = pool_g.cpu().view(-1, lora + rope), pool_c.view(-1, lora + rope)
    keep = slots[slots >= 0].long()
    _close(flat_g[keep], flat_c[keep], 3e-2, 2e-2, "cache entries")
    assert float(flat_g[:-1].abs().sum()) > 0 and float(flat_g[-1].abs().sum()) > 0          # the skipped row went to the spare slot


@pytest.mark.parametrize("window,softcap,use_sinks", [(200, 0.0, False), (0, 30.0, False), (0, 0.0, True), (128, 50.0, True)])
def test_attn_decode_variants(window, softcap, use_sinks):
    """Sliding window, logit soft-capping and sink logits inside the decode attention kernels against the PyTorch evaluation."""
    torch.manual_seed(31)
    Hq, Hkv, D, dt = 16, 4, 128, torch.bfloat16
    lens = [1, 127, 129, 300, 1025, 77, 640]
    Bn = len(lens)
    k_pool, v_pool, pt = _make_cache(Bn, lens, Hkv, D, dt)
    q = torch.randn(Bn, Hq * D).to(dt)
    seq = torch.tensor(lens, dtype=torch.int32)
    sinks = torch.randn(Hq) if use_sinks else None
    scale = 1 / math.sqrt(D)
    cu = torch.arange(Bn + 1, dtype=torch.int32)
    ref = A.paged_attention_general(q, k_pool, v_pool, pt, seq, cu, scale, Hq, Hkv, D, window=window, sinks=sinks, softcap=softcap)
    d = lambda t: t.to(DEV) if t is not None else None
    out = A.attn_decode(d(q), d(k_pool), d(v_pool), d(pt), d(seq), scale, Hq, Hkv, D, window=window, softcap=softcap, sinks=d(sinks))
    _close(out.cpu(), ref, 2e-2, 2e-2, "attn_decode variant", fro=2e-2)
    # with a reused workspace that carries both work lists (what the engine does)
    ws = A.DecodeWorkspace(Bn, Hkv, Hq // Hkv, pt.shape[1], DEV, window=window)
    for _ in range(2):
        out = A.attn_decode(d(q), d(k_pool), d(v_pool), d(pt), d(seq), scale, Hq, Hkv, D, ws=ws, window=window, softcap=softcap, sinks=d(sinks))
    _close(out.cpu(), ref, 2e-2, 2e-2, "attn_decode variant (workspace)", fro=2e-2)
