#!/usr/bin/env python
"""Headline benchmark: decode output tokens/s of Llama-3-8B (bf16, random-init) at 64 concurrent requests,
1024-token prompts, paged KV (page 128), tensor parallel over N GPUs of one node.

A *step* is one decode step of the whole batch (64 new tokens).  The prompts are prefilled first
(untimed), then W warm-up decode steps and K timed decode steps run through the public engine API.

Two numbers come out of the same K steps:
  * ``value``  -- device time: CUDA events around each step's GPU work on the launching stream, summed
                  over the K steps, max over ranks.
  * ``e2e``    -- wall time of the K ``engine.step()`` calls, which every step copy that step's inputs
                  from pinned host memory to the device and read the sampled tokens back.

``--impl reference`` runs the unmodified reference (installed under baseline/_ref) on the same
architecture / batch / lengths through its own Python API and prints the same JSON shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--dtype", default="auto", help="weight dtype: auto(bf16) | int8 | int4g128 | fp8 | nvfp4 | mxfp4")
    ap.add_argument("--comm", default="auto", choices=["auto", "fused", "nccl"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: the CPU configuration (fp32, C++ backend); use with --model qwen3-0.6b --batch 1 --prompt-len 128 --output-len 128")
    ap.add_argument("--moe-dtype", default="")
    ap.add_argument("--kv-cache-dtype", default="", help="page pool dtype: empty (the activation dtype) | fp8_e4m3")
    ap.add_argument("--moe-tp", action="store_true", help="shard every expert over the ranks instead of expert parallelism")
    ap.add_argument("--draw-lengths", action="store_true",
                    help="prompt lengths uniform in [128, --prompt-len] and output lengths uniform in [64, --output-len], drawn from the seed "
                         "(dynamic batching: requests finish at different steps)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _worker_hook(loop, eng):
    """Worker ranks time their own decode steps between the two marks rank 0 publishes, then join the max-over-ranks reduce."""
    import torch
    import torch.distributed as dist

    def begin():
        loop.timing = []

    def end():
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in (loop.timing or []))
        loop.timing = None
        t = torch.tensor([ms, 0.0], device=eng.model.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()

    loop.handlers.update(timing_begin=begin, timing_end=end, barrier=barrier)


def run_ours(args):
    import torch
    import torch.distributed as dist

    from fastllm_b200.engine import GenerationConfig
    from fastllm_b200.models import preset
    from fastllm_b200.ops import _lib
    from fastllm_b200.parallel.launcher import TPGroup

    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    if world_env != args.gpus and args.gpus > 1 and world_env == 1:
        raise SystemExit("launch multi-GPU runs with torchrun (python -m torch.distributed.run --nproc-per-node N ...)")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    cfg = preset(args.model)
    B, P, O = args.batch, args.prompt_len, args.output_len
    need_tokens = int(B * (P + O + 256) / 0.75)   # leaves the 80 % admission limit room for all B prompts
    spec = {"kind": "preset", "model": args.model, "dtype": "bfloat16", "seed": 0, "wdtype": args.dtype,
            "moe_wdtype": args.moe_dtype or None, "moe_tp": bool(args.moe_tp), "comm": args.comm, "max_m": B,
            "kv_cache_dtype": args.kv_cache_dtype or None,
            "engine": dict(max_batch=max(B, 1), max_context=((P + O + 127) // 128 + 1) * 128, max_tokens=need_tokens,
                           use_cuda_graph=not args.no_graph, prefix_cache=False, chunked_prefill_size=8192),
            "_worker_hook": _worker_hook}
    # Every rank builds its shard; ranks > 0 then serve rank 0's step plans inside attach() and return when it is done.
    group, eng, _ = TPGroup.attach(spec, device=f"cuda:{local}")
    if group is None:
        return              # a worker rank: it served inside attach() and has already released its GPU state
    world = group.world
    ctl = eng.control
    tp = eng.model.tp
    dev = eng.model.device
    gen = torch.Generator().manual_seed(1234)
    if args.draw_lengths:
        plens = torch.randint(128, P + 1, (B,), generator=gen).tolist()
        olens = torch.randint(64, O + 1, (B,), generator=gen).tolist()
    else:
        plens, olens = [P] * B, [O] * B
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in plens]
    for p, o in zip(prompts, olens):
        eng.launch(p, GenerationConfig(max_new_tokens=o, ignore_eos=True))
    # ---- prefill (untimed) ----
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while any(r.state.name in ("WAITING", "PREFILL") for r in list(eng.requests.values())):
        eng.step()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    assert args.draw_lengths or sum(r.state.name == "DECODE" for r in eng.requests.values()) == B, "not every request reached decode"
    K, W = args.steps, args.warmup
    if W + K > min(olens) - 1 and not args.draw_lengths:
        K = max(1, O - 1 - W)
    for _ in range(W):
        eng.step()
    _lib.check_device_errors()
    if ctl is not None:
        ctl.call("barrier")
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    if ctl is not None:
        ctl.call("timing_begin")
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    runner = eng.runner
    t_start = time.perf_counter()
    step_wall = []
    produced = 0
    for i in range(K):
        ts = time.perf_counter()
        ev[i][0].record()
        n = eng.step()
        ev[i][1].record()
        step_wall.append(time.perf_counter() - ts)
        produced += n
        assert n == B or args.draw_lengths, f"step produced {n} tokens, expected {B}"
        if not eng.has_work():
            K = i + 1
            ev = ev[:K]
            break
    torch.cuda.synchronize()
    wall = time.perf_counter() - t_start
    clocks = sampler.stop()
    _lib.check_device_errors()
    dev_ms = sum(a.elapsed_time(b) for a, b in ev)
    t = torch.tensor([dev_ms, wall * 1000.0], device=dev, dtype=torch.float64)
    if ctl is not None:
        ctl.call("timing_end")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = t.tolist()
    slot = runner.slots.get(runner._bucket(B))
    per_step_launches = getattr(runner, "launches_per_decode_step", 0)
    value = produced / (dev_ms / 1000.0)
    e2e = produced / (wall_ms / 1000.0)
    meta_bytes = int(slot.meta_host.numel() * 4) if slot is not None else 0
    ep = eng.model.ep
    out = {
        "metric": "decode output tok/s (device-timed, max over ranks)", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": dev_ms / K, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": _vs_baseline(args, world, value), "dtype": "bf16" if args.dtype == "auto" else args.dtype,
        "data": "synthetic (uniform random token ids, random-init weights N(0,0.02))",
        "config": {"model": args.model, "global_batch": B, "seq_len": P, "output_len": O,
                   "lengths": "prompt uniform 128..seq_len, output uniform 64..output_len, drawn from the seed" if args.draw_lengths else "fixed",
                   "parallelism": f"tp{world}" + (f"+ep{world}" if ep is not None else ""),
                   "kv_cache": "paged, page 128, " + (args.kv_cache_dtype or "bf16"), "l2": "inputs larger than L2 (weights + KV >> 126 MB per step)",
                   "cuda_graph": not args.no_graph, "comm": (tp.comm.fused.name if (tp.comm and tp.comm.fused) else ("nccl" if world > 1 else "none")),
                   "control_plane": "rank 0 schedules; ranks 1..N-1 replay its step plans from a shared-memory ring" if world > 1 else "single rank"},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": meta_bytes, "d2h_bytes_per_step": B * 4,
                "p50_tpot_ms": statistics.median(step_wall) * 1000.0},
        "gpu_launches": per_step_launches * K,
        "clocks": clocks,
        "prefill_s": prefill_s,
        "impl": "ours",
    }
    print(json.dumps(out), flush=True)
    _teardown(eng, group)


def _vs_baseline(args, world, value):
    """value / the reference's measured number for the same configuration and GPU count (baseline/measured_reference.json);
    None when that configuration has no reference measurement."""
    try:
        table = json.load(open(os.path.join(ROOT, "baseline", "measured_reference.json")))
    except OSError:
        return None
    key = f"{args.model}|{args.dtype}|b{args.batch}|p{args.prompt_len}"
    ref = table.get(key, {}).get(str(world))
    return (value / ref) if ref else None


def _teardown(eng, group):
    """Orderly exit (release the worker ranks, captured graphs, symmetric arena, process group -- in that order) so that the
    interpreter finishes normally and its exit hooks run."""
    if group is not None:
        eng.shutdown()
        group.shutdown()
    sys.stdout.flush()
    sys.stderr.flush()


def run_cpu(args):
    """CPU configuration: fp32 weights and activations on the native C++ backend, wall-clock timed."""
    import torch

    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.models import preset, random_init
    from fastllm_b200.ops import cpu

    cfg = preset(args.model)
    wd = args.dtype
    model = random_init(cfg, "cpu", torch.float32, seed=0, wdtype=wd)
    B, P, O = args.batch, args.prompt_len, args.output_len
    eng = LLMEngine(model, EngineConfig(max_batch=B, max_context=((P + O + 127) // 128 + 1) * 128, use_cuda_graph=False,
                                        prefix_cache=False), num_pages=B * ((P + O + 127) // 128 + 1) + 2)
    gen = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab_size, (P,), generator=gen).tolist() for _ in range(B)]
    for p in prompts:
        eng.launch(p, GenerationConfig(max_new_tokens=O, ignore_eos=True))
    t0 = time.perf_counter()
    while any(r.state.name in ("WAITING", "PREFILL") for r in list(eng.requests.values())):
        eng.step()
    prefill_s = time.perf_counter() - t0
    K, W = args.steps, args.warmup
    if W + K > O - 1:
        K = max(1, O - 1 - W)
    for _ in range(W):
        eng.step()
    steps = []
    for _ in range(K):
        ts = time.perf_counter()
        n = eng.step()
        steps.append(time.perf_counter() - ts)
        assert n == B
    secs = sum(steps)
    out = {"metric": "decode output tok/s (CPU, wall clock)", "value": B * K / secs, "unit": "tokens/s", "n_gpus": 0, "steps": K,
           "warmup": W, "ms_per_step": secs / K * 1000.0, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "fp32" if wd == "auto" else f"fp32 activations, {wd} weights",
           "data": "synthetic (uniform random token ids, random-init weights N(0,0.02))",
           "config": {"model": args.model, "global_batch": B, "seq_len": P, "output_len": O, "device": "cpu",
                      "threads": cpu.get_threads() if cpu.available() else None, "isa": cpu.lib().fbcpu_isa() if cpu.available() else None,
                      "native_model_runner": bool(model._native_cpu() is not None)},
           "e2e": {"value": B * K / secs, "unit": "tokens/s", "p50_tpot_ms": statistics.median(steps) * 1000.0, "ttft_s": prefill_s},
           "gpu_launches": 0, "impl": "ours"}
    print(json.dumps(out), flush=True)


def main():
    args = parse_args()
    if args.device == "cpu" and args.impl == "ours":
        run_cpu(args)
        return
    if args.impl == "reference":
        from baseline import reference_arm

        reference_arm.run(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
