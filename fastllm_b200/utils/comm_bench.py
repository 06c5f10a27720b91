"""Collective latency micro-benchmark at decode sizes: NCCL all-reduce vs the fused NVLink kernels.

Counterpart of the reference's ``tools/nccl_latency_bench/nccl_latency.cu`` (one process per GPU here, device-timed inside a
CUDA graph so launch overhead is excluded, max over ranks).  Run with::

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m fastllm_b200.utils.comm_bench [--hidden 4096]
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist


def _timeit(fn, dev, iters=20):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn(0)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    g.replay()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters * 1e3], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    from ..ops import _lib
    from ..ops import basic as B
    from ..ops.quant import LinearWeight
    from ..parallel import symm
    from ..parallel.tp import TPComm, init_distributed

    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--tokens", type=int, nargs="+", default=[1, 16, 64])
    ap.add_argument("--no-multicast", action="store_true")
    ap.add_argument("--big-p2p", action="store_true", help="prefill-sized kernels on plain peer loads / stores")
    ap.add_argument("--prefill-tokens", type=int, nargs="*", default=[],
                    help="also time the prefill-sized (bandwidth-regime) kernels at these token counts")
    args = ap.parse_args()
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    comm = TPComm(rank, world, dev)
    H = args.hidden
    fused = symm.FusedComm(comm, H, max(args.tokens), H, torch.bfloat16, use_multicast=not args.no_multicast,
                           max_big_m=max(args.prefill_tokens, default=0))
    ln = torch.ones(H, device=dev).bfloat16()
    rows = []
    for M in args.tokens:
        part = torch.randn(M, H, device=dev).bfloat16()
        t_nccl = _timeit(lambda i: dist.all_reduce(part), dev)
        t_fused = _timeit(lambda i: fused.ar_norm(part, ln, 1e-5), dev)
        K = args.inter // world
        ws = [LinearWeight.from_dense((torch.randn(H, K, device=dev) * 0.02).bfloat16()) for _ in range(6)]
        x = torch.randn(M, K, device=dev).bfloat16()
        h0 = torch.randn(M, H, device=dev).bfloat16()
        fused.load_h(h0)
        t_gemm_fused = _timeit(lambda i: fused.gemm_ar_norm(ws[i % 6], x, ln, 1e-5), dev)

        def nccl_path(i):
            p = ws[i % 6](x, residual=h0 if rank == 0 else None)
            dist.all_reduce(p)
            return B.rmsnorm(p, ln, 1e-5)

        t_gemm_nccl = _timeit(nccl_path, dev)
        # the pair a decoder layer runs: fused row-parallel GEMM, then the column-parallel GEMM that reads its output --
        # with the all-gather wait inside the first kernel, and with the wait deferred into the consumer GEMM
        wc = [LinearWeight.from_dense((torch.randn(2 * args.inter // world, H, device=dev) * 0.02).bfloat16()) for _ in range(3)]

        def pair(i, defer):
            _h, xn = fused.gemm_ar_norm(ws[i % 6], x, ln, 1e-5, defer=defer)
            return wc[i % 3](xn, swiglu=False)

        t_pair = _timeit(lambda i: pair(i, False), dev)
        t_pair_deferred = _timeit(lambda i: pair(i, True), dev)
        # phase stamps of one traced launch (CTA 0 of this rank; device global timer, ns)
        fused.trace = True
        fused.gemm_ar_norm(ws[0], x, ln, 1e-5)
        tr = fused.read_trace()
        fused.trace = False
        ph = {"gemm_and_push_us": (tr[1] - tr[0]) / 1e3, "sync1_arrive_us": (tr[2] - tr[1]) / 1e3, "sync1_wait_us": (tr[3] - tr[2]) / 1e3,
              "reduce_norm_broadcast_us": (tr[4] - tr[3]) / 1e3, "sync2_arrive_us": (tr[5] - tr[4]) / 1e3, "sync2_wait_us": (tr[6] - tr[5]) / 1e3}
        w_bytes = H * K * 2
        nv_bytes = M * H * 4 * (world - 1) / world + M * H * 2 * (world - 1) / world      # partial rows pushed out + x rows received
        roof_us = max(w_bytes / 6.54e12, nv_bytes / 770e9) * 1e6
        rows.append({"tokens": M, "bytes": M * H * 2, "nccl_allreduce_us": t_nccl, "fused_allreduce_residual_norm_us": t_fused,
                     "gemm_nccl_norm_us": t_gemm_nccl, "fused_gemm_allreduce_norm_us": t_gemm_fused,
                     "pair_us": t_pair, "pair_deferred_wait_us": t_pair_deferred, "phases": ph,
                     "roofline_us": roof_us, "fused_fraction_of_roofline": roof_us / t_gemm_fused})
    big_rows = []
    if args.big_p2p:
        fused.big_mc = 0
    for M in args.prefill_tokens:
        K = args.inter // world
        ws = [LinearWeight.from_dense((torch.randn(H, K, device=dev) * 0.02).bfloat16()) for _ in range(3)]
        x = torch.randn(M, K, device=dev).bfloat16()
        h0 = torch.randn(M, H, device=dev).bfloat16()
        fused.load_h(h0)

        def nccl_big(i):
            p = ws[i % 3](x, residual=h0 if rank == 0 else None)
            dist.all_reduce(p)
            return B.rmsnorm(p, ln, 1e-5)

        t_gemm = _timeit(lambda i: ws[i % 3](x), dev, iters=6)
        t_nccl = _timeit(nccl_big, dev, iters=6)
        t_two = _timeit(lambda i: fused.ar_norm(ws[i % 3](x), ln, 1e-5), dev, iters=6)
        t_one = _timeit(lambda i: fused.gemm_ar_norm(ws[i % 3], x, ln, 1e-5), dev, iters=6)
        part = ws[0](x)
        fused.trace = True
        fused.ar_norm(part, ln, 1e-5)
        tr = fused.read_trace()
        ph2 = {"copy_us": (tr[1] - tr[0]) / 1e3, "sync1_us": (tr[2] - tr[1]) / 1e3, "reduce_norm_broadcast_us": (tr[3] - tr[2]) / 1e3,
               "sync2_us": (tr[4] - tr[3]) / 1e3}
        fused.gemm_ar_norm(ws[0], x, ln, 1e-5)
        tr = fused.read_trace()
        ph1 = {"cta0_last_tile_stored_us": (tr[1] - tr[0]) / 1e3, "cta0_reducer_done_us": (tr[2] - tr[0]) / 1e3,
               "cta0_all_done_us": (tr[3] - tr[0]) / 1e3, "end_us": (tr[4] - tr[0]) / 1e3}
        fused.trace = False
        flops = 2.0 * M * H * K
        nv_bytes = 2 * M * H * 2 * (world - 1) / world          # reduced rows pulled in + normalised rows received, per direction the same
        roof_us = max(flops / 1.4e15, nv_bytes / 770e9) * 1e6
        big_rows.append({"tokens": M, "gemm_only_us": t_gemm, "gemm_nccl_norm_us": t_nccl, "gemm_then_reduce_kernel_us": t_two,
                         "fused_gemm_reduce_norm_us": t_one, "reduce_kernel_phases": ph2, "fused_phases": ph1, "roofline_us": roof_us, "fused_fraction_of_roofline": roof_us / t_one,
                         "gemm_tflops_in_fused": flops / t_one / 1e6})
    torch.cuda.synchronize()
    _lib.check_device_errors()
    dist.barrier()
    if rank == 0:
        print(json.dumps({"ranks": world, "hidden": H, "multicast": not args.no_multicast, "big_multicast": bool(fused.big_mc), "rows": rows, "prefill_rows": big_rows}), flush=True)
    comm.fused = None
    del fused
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
