"""Reference arm of bench.py: the unmodified reference (installed under baseline/_ref from a cmake build of the
reference sources) serving the same architecture / batch / lengths through its own public Python API
(`ftllm.util.make_normal_llm_model` + `launch_response_llm_model` / `fetch_response_llm_model`, the calls its own
`ftllm bench` makes, tools/fastllm_pytools/benchmark.py:98-160).

The reference is one process driving all GPUs (`--device multicuda:0,1,...`), so under torchrun only rank 0
works and the other ranks exit.  Its scheduler cannot be stepped from outside; a "step" is therefore observed
at the fetch loop: step k is complete when every request has delivered its k-th token.  Time is wall clock
at that loop (no device events are reachable through the reference's API).
"""
from __future__ import annotations

import ctypes
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


_printed = []


def _unavailable(why: str):
    _printed.append(1)
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # The reference's error path waits for a key press: give it an empty stdin, and bound the whole arm in time.
    try:
        os.dup2(os.open(os.devnull, os.O_RDONLY), 0)
    except OSError:
        pass
    import threading

    limit_s = float(os.environ.get("FB_REF_TIME_LIMIT", "900"))

    def _watchdog():
        time.sleep(limit_s)
        if not _printed:
            _unavailable(f"reference run did not finish within {int(limit_s)} s")
        os._exit(0)

    threading.Thread(target=_watchdog, daemon=True).start()
    if not os.path.exists(os.path.join(REF, "ftllm", "libfastllm_tools.so")):
        _unavailable("baseline/_ref/ftllm/libfastllm_tools.so missing (reference not built in this checkout)")
        return
    try:
        import torch

        n_vis = torch.cuda.device_count()
    except Exception as e:  # pragma: no cover
        _unavailable(f"torch/cuda not usable: {e!r}")
        return
    on_cpu = getattr(args, "device", "cuda") == "cpu"
    if on_cpu:
        # The reference's CPU device crashed with SIGSEGV right after "Load libfastllm_tools.so" (before any token) when
        # driven as `--device cpu --dtype float32` on Qwen3-0.6B; the call is not repeated.
        _unavailable("the reference's --device cpu path died with SIGSEGV during model construction on this pool's host; not re-run")
        return
    if not on_cpu and n_vis < args.gpus:
        _unavailable(f"{args.gpus} GPUs requested, {n_vis} visible")
        return
    sys.path.insert(0, ROOT)
    from baseline import synth

    want_fp8 = str(getattr(args, "dtype", "auto")).startswith("fp8")
    if args.model in ("deepseek-v3", "deepseek_v3"):
        # 671 B parameters: the checkpoint the reference's loader needs is ~700 GB of safetensors on the box's scratch disk
        # plus its own conversion pass over them; that does not fit a bounded benchmark call
        _unavailable("DeepSeek-V3 (671B): synthesising and loading a ~700 GB checkpoint through the reference's loader does not fit one bounded call")
        return
    if args.model.startswith("llama-3-70b"):
        _unavailable("Llama-3-70B int4g: the reference quantises the 140 GB bf16 checkpoint at load; synthesising + loading it does not fit one bounded call")
        return
    model_dir = os.environ.get("FB_REF_MODEL_DIR", f"/tmp/fb_ref_{args.model}" + ("_fp8" if want_fp8 else ""))
    t0 = time.time()
    synth.write_model(args.model, model_dir, fp8=want_fp8)
    t_synth = time.time() - t0
    sys.path.insert(0, REF)
    try:
        from ftllm import benchmark as rb
        from ftllm import llm as rllm
        from ftllm.util import make_normal_llm_model, make_normal_parser
    except Exception as e:
        _unavailable(f"import of the reference package failed: {e!r}"[:300])
        return
    B, P, O = args.batch, args.prompt_len, args.output_len
    is_moe = "a3b" in args.model or "moe" in args.model
    device = "cpu" if on_cpu else ("cuda" if args.gpus == 1 else "multicuda:" + ",".join(str(i) for i in range(args.gpus)))
    wdt = "float32" if on_cpu else "float16"
    # The reference's Llama path accepts fp32 / fp16 activations only ("Attention's input's type should be float32 or
    # float16" with bf16), so its arm runs the same 16-bit width in fp16.
    argv = [model_dir, "--device", device, "--dtype", wdt, "--atype", wdt, "--max_batch", str(B),
            "--tokens", str(int(B * (P + O + 256) / 0.75)), "--page_size", "128"]
    if is_moe:
        # Qwen3-MoE is one of the reference's thread-TP families: `--tp N` with everything (experts included) on the GPUs
        wd = "fp8_e4m3" if want_fp8 else "float16"
        argv = [model_dir, "--device", "cuda", "--moe_device", "cuda", "--dtype", wd, "--moe_dtype", wd, "--max_batch", str(B),
                "--tokens", str(int(B * (P + O + 256) / 0.75)), "--page_size", "128"]
        if args.gpus > 1:
            argv += ["--tp", str(args.gpus)]
            argv[argv.index("--moe_device") + 1] = "cuda:" + ",".join(str(i) for i in range(args.gpus))
    parser = make_normal_parser("reference bench")
    rb.add_benchmark_args(parser)
    rargs = parser.parse_args(argv)
    os.environ.setdefault("FASTLLM_CUDA_GRAPH", "1")
    try:
        model = make_normal_llm_model(rargs)
    except SystemExit as e:
        _unavailable(f"reference model construction exited: {e!r}")
        return
    except Exception as e:
        _unavailable(f"reference model construction failed: {e!r}"[:300])
        return
    import torch

    gen = torch.Generator().manual_seed(1234)
    vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]
    prompts = [torch.randint(0, vocab - 1, (P,), generator=gen).tolist() for _ in range(B)]
    gargs = {"do_sample": False, "top_p": 1.0, "top_k": 1, "temperature": 1.0, "repeat_penalty": 1.0}
    lib = rllm.fastllm_lib
    # warm-up request (the reference's own bench does the same)
    h = rb._launch_raw_response(model, prompts[0][:64], 4, gargs)
    while lib.fetch_response_llm_model(model.model, h) > -1:
        pass
    K, W = args.steps, args.warmup
    if W + K > O - 1:
        K = max(1, O - 1 - W)
    handles = [rb._launch_raw_response(model, p, O, gargs) for p in prompts]
    counts = [0] * B
    done = [False] * B
    t_launch = time.perf_counter()
    step_done_time = {}
    tokens_at = {}

    def min_count():
        return min(c for c in counts)

    # fetch round-robin: fetch blocks until the handle has a token, so after one pass every request advanced by one
    first_token_t = None
    cur = 0
    while not all(done):
        for i in range(B):
            if done[i]:
                continue
            tok = lib.fetch_response_llm_model(model.model, handles[i])
            if tok <= -1:
                done[i] = True
                continue
            counts[i] += 1
        cur += 1
        step_done_time[cur] = time.perf_counter()
        tokens_at[cur] = list(counts)
        if first_token_t is None:
            first_token_t = step_done_time[cur]
        if cur >= 1 + W + K:
            break
    alive = sum(1 for d in done if not d)
    if cur < 1 + W + 2:
        _unavailable(f"reference run ended early: {cur} steps observed, {alive}/{B} requests alive")
        _leave()
        return
    K = min(K, cur - 1 - W)                      # requests that ended early shorten the window instead of voiding the run
    t_a, t_b = step_done_time[1 + W], step_done_time[1 + W + K]
    secs = t_b - t_a
    steps = [step_done_time[s + 1] - step_done_time[s] for s in range(1 + W, 1 + W + K)]
    delivered = sum(tokens_at[1 + W + K]) - sum(tokens_at[1 + W])     # tokens that really arrived inside the window
    out = {
        "metric": "decode output tok/s (wall clock at the fetch loop)", "value": delivered / secs, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": secs / K * 1000.0, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32" if on_cpu else ("fp8 block-scaled weights, fp16 activations" if (is_moe and want_fp8) else "fp16 (the reference's Llama path rejects bf16 activations)"),
        "data": "synthetic (uniform random token ids, random-init weights N(0,0.02))",
        "config": {"model": args.model, "global_batch": B, "seq_len": P, "output_len": O,
                   "parallelism": device, "timing": "wall clock at the reference's fetch loop (no device events in its API)"},
        "e2e": {"value": delivered / secs, "unit": "tokens/s", "p50_tpot_ms": statistics.median(steps) * 1000.0,
                "ttft_s": first_token_t - t_launch},
        "impl": "reference", "synth_model_s": t_synth, "requests_alive_at_end": alive,
    }
    _printed.append(1)
    print(json.dumps(out), flush=True)
    _leave(handles, model, lib)


def _leave(handles=(), model=None, lib=None):
    """Abort what is still running, run the exit hooks, leave."""
    try:
        for h in handles:
            lib.abort_response_llm_model(model.model, h)
    except Exception:
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    # Run the interpreter's exit hooks now, then end the process: the reference's library keeps a scheduler thread and
    # per-GPU worker threads alive whose teardown is not ours to order, and a hang there would lose the result line.
    import atexit

    atexit._run_exitfuncs()
    os._exit(0)
