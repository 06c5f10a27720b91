"""``ftllm`` command line: run / chat / server / serve / webui / bench / export / download / config
(reference: tools/fastllm_pytools/cli.py:97-167)."""
from __future__ import annotations

import argparse
import json
import sys
import time


def _chat_loop(model, args):
    history = []
    print("fastllm_b200 chat — type 'clear' to reset, 'stop' to quit.")
    while True:
        try:
            q = input("\nUser: ")
        except EOFError:
            break
        if q.strip() == "stop":
            break
        if q.strip() == "clear":
            history = []
            continue
        print("AI: ", end="", flush=True)
        out = ""
        from .util import sampling_kwargs

        for piece in model.stream_response(q, history=history, **sampling_kwargs(args)):
            out += piece
            print(piece, end="", flush=True)
        print()
        history.append((q, out))


def _bench(model, args):
    from .engine import GenerationConfig

    ids = (model.encode(args.prompt_unit) * (args.input_tokens // max(1, len(model.encode(args.prompt_unit))) + 1))[:args.input_tokens]
    eng = model.engine
    gen = GenerationConfig(max_new_tokens=args.output_tokens, ignore_eos=True)
    prof = None
    if getattr(args, "profile", False) and eng.model.on_cuda:
        from .ops import _lib

        eng.runner.graph_ok = False          # events cannot be recorded inside a graph replay
        prof = _lib.start_profile()
    for _ in range(args.warmup):
        eng.generate([ids], GenerationConfig(max_new_tokens=8, ignore_eos=True))
    t0 = time.perf_counter()
    hs = [eng.launch(ids, gen) for _ in range(args.batch)]
    reqs = [eng.requests[h] for h in hs]
    first = None
    while any(not r.finished() for r in reqs):
        eng.step()
        if first is None and all(r.output_ids for r in reqs):
            first = time.perf_counter()
    t1 = time.perf_counter()
    out = sum(len(r.output_ids) for r in reqs)
    res = {"input_tokens": len(ids), "output_tokens": args.output_tokens, "batch": args.batch, "total_time_s": t1 - t0,
           "ttft_s": (first or t1) - t0, "tpot_ms": (t1 - (first or t0)) / max(1, args.output_tokens - 1) * 1e3,
           "batch_tokens_per_second": out / (t1 - t0), "batch_decode_tokens_per_second": (out - args.batch) / max(1e-9, t1 - (first or t0))}
    print(json.dumps(res, indent=1))
    if prof is not None:
        from .ops import _lib

        print(prof.format())
        _lib.stop_profile()
    return res


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    cmds = {"run", "chat", "tui", "server", "serve", "webui", "bench", "benchmark", "export", "download", "config"}
    if not argv or argv[0] == "tui":
        # no arguments: the deployment form, as with the reference (tools/fastllm_pytools/cli.py:113-118)
        from . import tui

        return tui.main(plain="--plain" in argv)
    cmd = argv.pop(0) if argv and argv[0] in cmds else "chat"
    from .util import make_normal_llm_model, make_normal_parser

    p = make_normal_parser(f"ftllm {cmd}")
    if cmd in ("server", "serve", "webui"):
        from .serving.server import add_server_args

        add_server_args(p)
    if cmd in ("bench", "benchmark"):
        p.add_argument("--input_tokens", type=int, default=64)
        p.add_argument("--output_tokens", type=int, default=256)
        p.add_argument("--batch", type=int, default=1)
        p.add_argument("--warmup", type=int, default=1)
        p.add_argument("--prompt_unit", type=str, default="FastLLM benchmark context block. ")
        p.add_argument("--profile", action="store_true", help="print a per-kernel device-time table (runs decode without CUDA graphs)")
    if cmd == "export":
        p.add_argument("-o", "--output", type=str, required=True)
    if cmd == "download":
        p.add_argument("--repo", type=str, default="")
        p.add_argument("--local-dir", dest="local_dir", type=str, default="")
        p.add_argument("--revision", type=str, default="")
        p.add_argument("--include", type=str, nargs="*", default=None)
        p.add_argument("--exclude", type=str, nargs="*", default=None)
        p.add_argument("--hf_token", type=str, default="")
        p.add_argument("--hf_username", type=str, default="")
        p.add_argument("-j", "--workers", dest="workers", type=int, default=8)
        # accepted for scripts written against the reference's downloader (which shells out to aria2c / wget); this one
        # downloads with its own worker threads
        p.add_argument("--tool", choices=["aria2c", "wget"], default="aria2c")
        p.add_argument("-x", dest="threads_per_file", type=int, default=4)
        p.add_argument("--dataset", action="store_true", help="the repository is a dataset")
    args = p.parse_args(argv)
    if cmd == "config":
        print(json.dumps({k: v for k, v in vars(args).items() if v not in (None, "", -1, False)}, indent=1))
        return 0
    if cmd == "download":
        from .download import download

        print(download(args.repo or args.model or args.path, args.cache_dir or None, args.local_dir or None, args.revision or None,
                       args.include, args.exclude, args.hf_token or None, args.workers, dataset=args.dataset))
        return 0
    if cmd == "export":
        from .loader import flm
        from .util import apply_config_file

        args = apply_config_file(args)
        if args.output.endswith(".flm"):
            flm.export_hf_to_flm(args.path, args.output, "float16" if args.dtype == "auto" else args.dtype)
        else:
            from .loader.export import export_quantized_hf

            export_quantized_hf(args.path, args.output, "float16" if args.dtype == "auto" else args.dtype, args.moe_dtype or None)
        print("exported to", args.output)
        return 0
    if cmd in ("server", "serve"):
        from .serving.server import serve

        serve(args)
        return 0
    if cmd == "webui":
        from .serving.webui import run_webui

        run_webui(args)
        return 0
    model = make_normal_llm_model(args)
    if cmd in ("bench", "benchmark"):
        _bench(model, args)
    else:
        _chat_loop(model, args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
