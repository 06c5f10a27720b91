"""Operator API (reference operator names): every operator against its plain PyTorch definition on the CPU, and, with a
GPU, the CUDA result against the CPU result (the reference's optest scheme: CPU run = baseline, other devices compared)."""
import math

import pytest
import torch

from fastllm_b200.ops import api as O
from fastllm_b200.ops import api
from fastllm_b200.ops import attention as A


def test_elementwise_and_layout_ops_cpu():
    torch.manual_seed(0)
    x = torch.randn(5, 64)
    assert torch.allclose(O.Silu(x), torch.nn.functional.silu(x), atol=1e-5)
    assert torch.allclose(O.GeluNew(x), torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-5)
    assert torch.allclose(O.Swiglu(x), torch.nn.functional.silu(x[:, :32]) * x[:, 32:], atol=1e-5)
    assert torch.allclose(O.SoftMax(x), torch.softmax(x, -1), atol=1e-6)
    assert torch.allclose(O.LayerNorm(x, torch.ones(64), torch.zeros(64)), torch.nn.functional.layer_norm(x, (64,)), atol=1e-4)
    y = x.clone()
    O.AddTo(y, x, 0.5)
    assert torch.allclose(y, 1.5 * x)
    assert O.Cat(x, x, 1).shape == (5, 128) and O.Split(x, 1, 8, 24).shape == (5, 16) and O.Repeat(x, 0, 3).shape == (15, 64)
    assert torch.equal(O.Permute(x.reshape(5, 8, 8), (1, 0, 2)), x.reshape(5, 8, 8).permute(1, 0, 2))
    tk = O.TopK(x, 3)
    assert tk.shape == (5, 3, 2) and torch.equal(tk[..., 0].long(), x.topk(3).indices)


def test_linear_matmul_attention_cpu():
    torch.manual_seed(1)
    x, w, b = torch.randn(6, 96), torch.randn(40, 96) * 0.1, torch.randn(40)
    assert torch.allclose(O.Linear(x, w, b), x @ w.t() + b, atol=1e-4)
    out = torch.ones(6, 40)
    O.LinearAdd(x, w, None, out)
    assert torch.allclose(out, 1 + x @ w.t(), atol=1e-4)
    wg = torch.randn(128, 96) * 0.1
    gu = x @ wg.t()
    assert torch.allclose(O.LinearSwiglu(x, wg), torch.nn.functional.silu(gu[:, :64]) * gu[:, 64:], atol=1e-4)
    assert torch.allclose(O.MatMulTransB(x, w, 0.5), 0.5 * x @ w.t(), atol=1e-5)
    q, k, v = torch.randn(4, 3, 16), torch.randn(2, 7, 16), torch.randn(2, 7, 16)
    got = O.Attention(q, k, v, group=2, causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q[None], k.repeat_interleave(2, 0)[None], v.repeat_interleave(2, 0)[None],
                                                           attn_mask=torch.ones(3, 7, dtype=torch.bool).tril(diagonal=4))[0]
    assert torch.allclose(got, ref, atol=1e-5)
    sc = torch.zeros(2, 3, 5)
    al = O.AlibiMask(sc, torch.tensor([0.5, 0.25]))
    assert al[0, 0, 2] == 0 and al[0, 0, 0] == -1.0 and al[1, 2, 0] == -1.0 and al[0, 0, 3] == -1e4


def test_rope_and_select_expert_cpu():
    torch.manual_seed(2)
    x = torch.randn(4, 2, 32)
    pos = torch.tensor([0, 5, 9, 2])
    cos, sin = A.build_rope_tables(32, 16, 10000.0)
    a = O.LlamaRotatePosition2D(x, pos, sin, cos, 16)
    b = O.RopeEncoding(x, pos, 32, 10000.0)
    assert torch.allclose(a, b, atol=1e-5)
    inter = O.NearlyRotatePosition2D(x, pos, sin, cos, 16)
    assert not torch.allclose(a, inter) and torch.allclose(inter[0], x[0], atol=1e-6)     # position 0 is the identity
    lg = torch.randn(7, 16)
    idx, w = O.FusedSoftmaxSelectExpert(lg, 2, True)
    p = torch.softmax(lg, -1)
    ti = p.topk(2).indices
    assert torch.equal(idx.long(), ti) and torch.allclose(w, p.gather(1, ti) / p.gather(1, ti).sum(-1, keepdim=True), atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["Linear", "LinearSwiglu", "RMSNorm", "Swiglu", "Embedding", "SelectExpert"])
def test_cuda_matches_cpu(name):
    """CPU run = baseline, CUDA compared with atol / rtol (reference: RunSingleCase, test/ops/cppOps.cpp:3395-3470)."""
    from fastllm_b200.ops import basic as B

    torch.manual_seed(3)
    dt = torch.bfloat16
    x = torch.randn(33, 512)
    if name == "Linear":
        w, b = torch.randn(256, 512) * 0.05, torch.randn(256)
        cpu, gpu = O.Linear(x, w, b), O.Linear(x.cuda().to(dt), w.cuda().to(dt), b.cuda().to(dt))
    elif name == "LinearSwiglu":
        g, u = torch.randn(256, 512) * 0.05, torch.randn(256, 512) * 0.05
        cpu = O.LinearSwiglu(x, torch.cat([g, u]))
        gpu = O.LinearSwiglu(x.cuda().to(dt), B.interleave_gate_up(g.cuda().to(dt), u.cuda().to(dt)), interleaved=True)
    elif name == "RMSNorm":
        w = torch.randn(512)
        cpu, gpu = O.RMSNorm(x, w, 1e-6), O.RMSNorm(x.cuda().to(dt), w.cuda().to(dt), 1e-6)
    elif name == "Swiglu":
        cpu, gpu = O.Swiglu(x), O.Swiglu(x.cuda().to(dt))
    elif name == "Embedding":
        tab, ids = torch.randn(100, 512), torch.randint(0, 100, (33,))
        cpu, gpu = O.Embedding(ids, tab), O.Embedding(ids.cuda().int(), tab.cuda().to(dt))
    else:
        lg, bias = torch.randn(33, 64), torch.randn(64) * 0.1
        (ci, cw), (gi, gw) = O.SelectExpert(lg, bias, 4, True, 2.0, "sigmoid"), O.SelectExpert(lg.cuda(), bias.cuda(), 4, True, 2.0, "sigmoid")
        assert torch.equal(ci.long(), gi.cpu().long())
        cpu, gpu = cw, gw
    assert torch.allclose(gpu.float().cpu(), cpu.float(), atol=6e-2, rtol=3e-2)


def test_linear_attention_and_misc_operators_cpu():
    """The operators behind the Gated-DeltaNet layers and the smaller ones of the reference's list, against direct formulas."""
    torch.manual_seed(3)
    x = torch.randn(2, 4, 10)
    w = torch.randn(4, 3)
    y = O.Conv1DPerChannel(x, w)
    ref = torch.stack([sum(w[c, j] * torch.nn.functional.pad(x[:, c], (2, 0))[:, j:j + 10] for j in range(3)) for c in range(4)], dim=1)
    assert torch.allclose(y, ref, atol=1e-5)
    A_ = torch.tril(torch.randn(6, 6), -1) * 0.3
    assert torch.allclose(O.TransferAttn(A_), torch.linalg.inv(torch.eye(6) - A_), atol=1e-5)
    g = -torch.rand(2, 6).cumsum(-1)
    dm = O.MakeDecayMask(g)
    assert torch.allclose(dm[0, 4, 1], (g[0, 4] - g[0, 1]).exp()) and float(dm[0, 1, 4]) == 0.0
    assert torch.allclose(O.CumSumLastDim(torch.ones(3, 5)), torch.arange(1.0, 6.0).expand(3, 5))
    n, H, Dk, Dv = 70, 2, 16, 8
    q, k, v = torch.randn(n, H, Dk), torch.randn(n, H, Dk), torch.randn(n, H, Dv)
    gg, beta = -torch.rand(n, H) * 0.3, torch.rand(n, H)
    s1, s2 = torch.zeros(H, Dk, Dv), torch.zeros(H, Dk, Dv)
    o1 = O.RecurrentGatedDeltaRule(q, k, v, gg, beta, s1)
    o2 = O.ChunkGatedDeltaRulePrefill(q, k, v, gg, beta, s2, chunk=16)
    assert torch.allclose(o1, o2, atol=1e-4) and torch.allclose(s1, s2, atol=1e-4)
    t = torch.randn(3, 8)
    assert torch.allclose(O.CrossSwiglu(t), torch.nn.functional.silu(t[:, 0::2]) * t[:, 1::2], atol=1e-6)
    assert O.Pad(t, 1, 1, 2).shape == (3, 11) and float(O.Pad(t, 1, 1, 2, value=7.0)[0, 0]) == 7.0
    assert torch.allclose(O.Normalize(t).norm(dim=-1), torch.ones(3), atol=1e-5)
    part = O.RMSNormPart(t, torch.ones(4), 1e-6, 2, 6)
    assert torch.equal(part[:, :2], t[:, :2]) and torch.allclose(part[:, 2:6].pow(2).mean(-1), torch.ones(3), atol=1e-3)
    pt, kv, last = O.GeneratePagedBatchParams([[3, 1], [2]], [130, 5])
    assert pt.tolist() == [[3, 1], [2, 0]] and kv.tolist() == [130, 5] and last.tolist() == [2, 5]
    assert O.GenerateAppendPagedCacheBatchParams([[3, 1], [2]], [127, 0], [2, 1]).tolist() == [3 * 128 + 127, 1 * 128, 2 * 128]
    assert [u.shape for u in O.SplitBatch(torch.zeros(4, 6), 0, 2)] == [(2, 6), (2, 6)]
    beta2, g2 = O.SigmoidMambaSoftplus(torch.zeros(2), torch.zeros(2), torch.zeros(2), torch.zeros(2))
    assert torch.allclose(beta2, torch.full((2,), 0.5)) and torch.allclose(g2, torch.full((2,), -math.log(2.0)))


def test_kimi_k3_operators_match_their_definitions():
    """Kimi-K3 operator names: the recurrent KDA against an explicit per-token loop, state replay, gates and activations."""
    torch.manual_seed(3)
    Bn, S, H, D = 2, 5, 3, 8
    q, k, v, g = (torch.randn(Bn, S, H, D) for _ in range(4))
    rb = torch.randn(Bn, S, H)
    a_log, dt = torch.randn(H) * 0.3, torch.randn(H, D) * 0.1
    out, state, decay, beta = api.KimiK3RecurrentKDA(q, k, v, g, rb, a_log, dt, -5.0)
    ref_state = torch.zeros(Bn, H, D, D)
    for b in range(Bn):
        for h in range(H):
            for t in range(S):
                gate = -5.0 * torch.sigmoid(torch.exp(a_log[h]) * (g[b, t, h] + dt[h]))
                ref_state[b, h] *= torch.exp(gate)[:, None]
                pred = k[b, t, h] @ ref_state[b, h]
                delta = (v[b, t, h] - pred) * torch.sigmoid(rb[b, t, h])
                ref_state[b, h] += k[b, t, h][:, None] * delta[None, :]
                assert torch.allclose(out[b, t, h], (q[b, t, h] @ ref_state[b, h]) * D ** -0.5, atol=1e-5)
    assert torch.allclose(state, ref_state, atol=1e-5) and decay.shape == g.shape and beta.shape == rb.shape
    st2 = api.KimiK3RecurrentKDAUpdateState(k, v, g, rb, a_log, dt, -5.0, 3, None if False else torch.zeros(Bn, H, D, D))
    o3, st3 = api.KimiK3RecurrentKDAOutputOnly(q[:, :3], k[:, :3], v[:, :3], g[:, :3], rb[:, :3], a_log, dt, -5.0)
    assert torch.allclose(st2, st3, atol=1e-6)
    x = torch.randn(4, 16)
    assert torch.allclose(api.KimiK3L2Norm(x).norm(dim=-1), torch.ones(4), atol=1e-3)
    gt = torch.randn(4, 16)
    assert torch.allclose(api.KimiK3RMSNormSigmoidGate(x, gt, torch.ones(16), 1e-6), api.KimiK3RMSNorm(x, torch.ones(16), 1e-6) * torch.sigmoid(gt), atol=1e-6)
    assert torch.allclose(api.KimiK3SiTUAndMul(gt, x, 1e6, 0.0), gt * torch.sigmoid(gt) * x, atol=1e-4)      # large beta: SiLU(g) * up
    # convolution with a cache continues the sequence exactly
    xs, w = torch.randn(1, 7, 6), torch.randn(6, 4)
    whole = api.KimiK3CausalConv1D(xs, w, 4)
    cache = torch.zeros(1, 3, 6)
    parts = torch.cat([api.KimiK3CausalConv1D(xs[:, :3], w, 4, cache), api.KimiK3CausalConv1D(xs[:, 3:], w, 4, cache)], dim=1)
    assert torch.allclose(whole, parts, atol=1e-6)
    # residual attention with one block reduces to a two-way softmax mix
    ps, br = torch.randn(3, 16), torch.randn(3, 1, 16)
    mix = api.KimiK3AttnRes(ps, br, torch.randn(16), torch.ones(16))
    assert mix.shape == ps.shape and torch.all((mix - ps).abs() <= (br[:, 0] - ps).abs() + 1e-5)


def test_adapter_softmax_and_settings_names():
    torch.manual_seed(4)
    x, w = torch.randn(3, 8), torch.randn(6, 8)
    a, b = torch.randn(2, 8), torch.randn(6, 2)
    y = api.LoraLayer(x, w, a, b, None, {"lora_alpha": 4, "r": 2})
    assert torch.allclose(y, x @ w.t() + 2.0 * (x @ a.t()) @ b.t(), atol=1e-5)
    l = torch.rand(6)
    assert torch.allclose(api.IA3Layer(x, w, l), (x @ w.t()) * l, atol=1e-5)
    assert torch.allclose(api.Softmax(x, -1).sum(-1), torch.ones(3), atol=1e-6)
    assert torch.allclose(api.LinearEx(x, w, None, api.ExSilu), torch.nn.functional.silu(x @ w.t()), atol=1e-5)
    assert api.NVFP4E8M0ScaleToFloat(127) == 1.0 and api.NVFP4E8M0ScaleToFloat(130) == 8.0
    assert api.GetDataTypeName(9) == "int4_group" and api.HasDeviceType("cpu")
    api.SetThreads(2)
    assert api.GetThreads() == 2
    assert api.SelectDeviceFromMap({"cpu": 1}, 0, 4) == "cpu"
    qn, qp = torch.randn(2, 3, 5), torch.randn(2, 3, 2)
    kv, pe = torch.randn(2, 4, 5), torch.randn(2, 4, 2)
    o = api.MergeMLA(qn, qp, kv, pe, None, 0.3)
    s = torch.softmax((torch.einsum("bhd,bld->bhl", qn, kv) + torch.einsum("bhd,bld->bhl", qp, pe)) * 0.3, -1)
    assert torch.allclose(o, torch.einsum("bhl,bld->bhd", s, kv), atol=1e-5)


def test_executor_device_order_and_migration():
    from fastllm_b200.ops import executor as E

    ex = E.Executor([E.Device("cpu", ops={"Linear", "Softmax"}), E.Device("cpu")])
    x, w = torch.randn(3, 8), torch.randn(5, 8)
    y = ex.Run("Linear", x, w)
    assert torch.allclose(y, x @ w.t(), atol=1e-5)
    assert ex.Run("Silu", x).shape == x.shape                 # not in the first device's set: falls through to the second
    assert ex.profiler["Linear"][0] == 1 and "Silu" in ex.profiler
    ex.SetFirstDevice("cpu")
    assert ex.GetFirstDeviceType() == "cpu" and ex.HasDevice("cpu") and not ex.HasDevice("cuda") and ex.GetDeviceIds("cpu") == [0, 0]
    assert ex.CanRunOnFirstDevice("Linear", x, w)
    with pytest.raises(RuntimeError):
        ex.RunOnDevice("cuda", "Linear", x, w)
    with pytest.raises(RuntimeError):
        ex.Run("NoSuchOperator", x)
    moved = E.ToDevice({"a": [x, 3], "b": (w,)}, "cpu")
    assert moved["a"][0] is x and moved["a"][1] == 3
    assert "Linear" in ex.PrintProfiler()
    ex.ClearProfiler()
    assert not ex.profiler
