"""Command-line flag set and model factory shared by every entry point.

Same flags as the reference (tools/fastllm_pytools/util.py:478-567 ``make_normal_parser``) so that existing
command lines keep working; ``make_normal_llm_model`` (util.py:586-1089) maps them onto ``llm.model``: device /
``--tp`` normalisation, MoE defaults, ``quantization_config`` -> dtype, threads, KV limits.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def make_normal_parser(des: str = "fastllm_b200", add_help: bool = True) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=des, add_help=add_help)
    p.add_argument("model", nargs="?", help="model path: HF folder, .flm / .gguf file, or a JSON config file")
    p.add_argument("-p", "--path", type=str, default="")
    p.add_argument("-t", "--threads", type=int, default=-1)
    p.add_argument("-l", "--low", action="store_true")
    p.add_argument("--dtype", type=str, default="auto")
    p.add_argument("--moe_dtype", type=str, default="")
    p.add_argument("--moe_atype", type=str, default="")
    p.add_argument("--atype", type=str, default="auto")
    p.add_argument("--kv_cache_dtype", type=str, default="auto")
    p.add_argument("--cuda_embedding", action="store_true")
    p.add_argument("--kv_cache_limit", type=str, default="auto")
    p.add_argument("--max_batch", type=int, default=-1)
    p.add_argument("--chunked_prefill_size", type=int, default=-1)
    p.add_argument("--device", type=str)
    p.add_argument("--tp", type=str, default="")
    p.add_argument("--moe_device", type=str, default="")
    p.add_argument("--moe_device_layers", type=int, default=-1)
    p.add_argument("--moe_experts", type=int, default=-1)
    p.add_argument("--cache_history", type=str, default="")
    p.add_argument("--cache_fast", type=str, default="")
    p.add_argument("--enable_thinking", type=str, default="")
    p.add_argument("--cuda_shared_expert", "--cuda_se", type=str, default="true")
    p.add_argument("--enable_amx", "--amx", type=str, default="false")
    p.add_argument("--tokens", type=int, default=-1)
    p.add_argument("--page_size", type=int, default=-1)
    p.add_argument("--prefix_cache", "--prefix-cache", dest="prefix_cache", type=str, default="")
    p.add_argument("--gpu_mem_ratio", type=float, default=0.9)
    p.add_argument("--max_context_length", type=int, default=-1)
    p.add_argument("--cuda_graph", type=str, default="true")
    p.add_argument("--custom", type=str, default="")
    p.add_argument("--lora", type=str, default="")
    p.add_argument("--cache_dir", type=str, default="")
    p.add_argument("--dtype_config", type=str, default="")
    p.add_argument("--ori", type=str, default="")
    p.add_argument("--tool_call_parser", type=str, default="auto")
    p.add_argument("--chat_template", type=str, default="")
    # sampling defaults of the interactive commands (reference: chat.py / tui.py)
    p.add_argument("--top_p", type=float, default=None)
    p.add_argument("--top_k", type=int, default=None)
    p.add_argument("--temperature", type=float, default=None)
    p.add_argument("--repeat_penalty", type=float, default=None)
    # accepted for command-line compatibility; these name mechanisms this build does not have (a weight slab allocator, an
    # external Triton compile server, speculative draft models, linear-attention state snapshots): they change nothing here
    p.add_argument("--cuda_slab", type=str, default="")
    p.add_argument("--triton", type=str, default="")
    p.add_argument("--mtp", type=str, default="")
    p.add_argument("--dspark", type=str, default="")
    p.add_argument("--speculative_algorithm", type=str, default="")
    p.add_argument("--speculative_draft_model_path", type=str, default="")
    p.add_argument("--speculative_dspark_block_size", type=int, default=0)
    p.add_argument("--speculative_dspark_confidence_threshold", type=float, default=0.0)
    p.add_argument("--prefix_cache_snapshot_interval_pages", type=int, default=0)
    p.add_argument("--prefix_cache_snapshot_max_per_request", type=int, default=0)
    p.add_argument("--prefix_cache_snapshot_max_records", type=int, default=0)
    return p


def sampling_kwargs(args) -> dict:
    """Generation keyword arguments from the --top_p / --top_k / --temperature / --repeat_penalty flags (unset flags omitted)."""
    kw = {}
    for name in ("top_p", "top_k", "temperature", "repeat_penalty"):
        v = getattr(args, name, None)
        if v is not None:
            kw[name] = v
    return kw


def parse_tp(tp: str) -> list[int]:
    """``"4"`` -> first four GPUs, ``"0,2"`` -> those GPUs, ``"auto"`` -> all visible GPUs, ``""`` -> no TP."""
    tp = (tp or "").strip().lower()
    if not tp:
        return []
    if tp == "auto":
        return list(range(torch.cuda.device_count()))
    if "," in tp:
        return [int(x) for x in tp.split(",") if x.strip()]
    n = int(tp)
    return [0] if n == 0 else list(range(n))


def parse_device(device: str | None):
    """``cuda`` / ``cuda:1`` / ``cpu`` / ``multicuda:0,1[:ratio]`` / ``{'cuda:0':3,'cuda:1':2}`` -> (kind, gpu ids, raw map)."""
    if not device:
        return ("cuda" if torch.cuda.is_available() else "cpu"), [], None
    d = device.strip()
    if d.startswith("{"):
        m = json.loads(d.replace("'", '"'))
        return "cuda", [int(k.split(":")[1]) for k in m if k.startswith("cuda:")], m
    if d.startswith("multicuda"):
        ids = []
        spec = d.split(":", 1)[1] if ":" in d else ""
        for part in spec.split(","):
            part = part.strip()
            if part and part.split(":")[0].isdigit():
                ids.append(int(part.split(":")[0]))
        return "cuda", ids or list(range(torch.cuda.device_count())), None
    if d.startswith("cuda"):
        return "cuda", [int(d.split(":")[1])] if ":" in d else [], None
    return d, [], None


def apply_config_file(args):
    """A positional ``model`` that is a JSON file supplies defaults for every flag (reference: ``ftllm config``)."""
    path = args.path or args.model or ""
    if path.endswith(".json") and os.path.isfile(path):
        cfg = json.load(open(path))
        for k, v in cfg.items():
            if hasattr(args, k) and getattr(args, k) in (None, "", -1, "auto", False):
                setattr(args, k, v)
        path = cfg.get("path", cfg.get("model", ""))
    args.path = path
    return args


def make_normal_llm_model(args):
    from . import llm

    args = apply_config_file(args)
    algo = str(getattr(args, "speculative_algorithm", "") or "").lower()
    mtp_flag = getattr(args, "mtp", "")
    if algo in ("ngram", "prompt_lookup", "lookup", "mtp", "nextn", "eagle") or mtp_flag:
        # "mtp": drafts from the checkpoint's multi-token-prediction head (the engine falls back to prompt-lookup drafts when
        # the model has none, runs tensor-parallel or keeps recurrent state)
        llm._settings["speculative"] = "mtp" if (algo in ("mtp", "nextn", "eagle") or mtp_flag) else "ngram"
        n = getattr(args, "speculative_dspark_block_size", 0) or (int(mtp_flag) if str(mtp_flag).isdigit() else 0)
        if n:
            llm._settings["speculative_tokens"] = int(n)
        elif llm._settings["speculative"] == "mtp":
            llm._settings["speculative_tokens"] = 1
    elif algo in ("draft", "draft_model") or (not algo and getattr(args, "speculative_draft_model_path", "")):
        # a separate smaller model of the same vocabulary proposes the tokens (--speculative_draft_model_path)
        if not getattr(args, "speculative_draft_model_path", ""):
            raise SystemExit("--speculative_algorithm draft needs --speculative_draft_model_path <model folder>")
        llm._settings["speculative"] = "draft"
        llm._settings["draft_model_path"] = args.speculative_draft_model_path
        n = getattr(args, "speculative_dspark_block_size", 0)
        if n and n > 0:
            llm._settings["speculative_tokens"] = int(n)
    elif algo:
        print(f"[fastllm_b200] --speculative_algorithm {algo}: 'ngram' (prompt-lookup drafts), 'mtp' (the checkpoint's draft head) and "
              "'draft' (a separate draft model) exist in this build; decoding normally", file=sys.stderr)
    if getattr(args, "dspark", ""):
        print("[fastllm_b200] --dspark: the DeepSeek-V4 block-draft scheme is not part of this build "
              "(use --speculative_algorithm draft / mtp / ngram); decoding normally", file=sys.stderr)
    if not args.path:
        raise SystemExit("no model given: pass a model path (HF folder, .flm or .gguf)")
    if args.threads and args.threads > 0:
        llm.set_cpu_threads(args.threads)
    else:
        llm.set_cpu_threads(max(1, min(32, (os.cpu_count() or 4) - 2)))
    kind, gpu_ids, raw_map = parse_device(args.device)
    if raw_map:                      # layer-split placement over several GPUs of this process
        llm.set_device_map(raw_map)
        gpu_ids = gpu_ids[:1]
    tp_ids = parse_tp(args.tp) or (gpu_ids if len(gpu_ids) > 1 else [])
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.max_batch and args.max_batch > 0:
        llm.set_max_batch(args.max_batch)
    if args.tokens and args.tokens > 0:
        llm.set_max_tokens(args.tokens)
    if args.chunked_prefill_size and args.chunked_prefill_size > 0:
        llm.set_chunked_prefill_size(args.chunked_prefill_size)
    if args.max_context_length and args.max_context_length > 0:
        llm.set_max_context_length(args.max_context_length)
    if args.page_size and args.page_size > 0:
        llm.set_page_size(args.page_size)
    if getattr(args, "moe_device", ""):
        llm.set_device_map(args.moe_device, is_moe=True)
        llm._settings["moe_device_layers"] = int(getattr(args, "moe_device_layers", -1))
    llm.set_gpu_mem_ratio(args.gpu_mem_ratio)
    llm.set_cuda_graph(str(args.cuda_graph).lower() != "false")
    if args.prefix_cache:
        llm.set_prefix_cache(str(args.prefix_cache).lower() == "true")
    # Several GPUs: this process becomes rank 0 and spawns one worker process per further GPU (`--tp N`,
    # `--device multicuda:0,1`); inside a job started by an outer launcher (torchrun) the ranks attach instead.
    tp = None
    device = "cpu" if kind == "cpu" else (f"cuda:{gpu_ids[0]}" if len(gpu_ids) == 1 else "cuda")
    if world > 1:
        tp = "env"
    elif len(tp_ids) > 1:
        tp = [f"cuda:{i}" for i in tp_ids] if kind != "cpu" else ["cpu"] * len(tp_ids)
    cfg_path = os.path.join(args.path, "config.json")
    if os.path.isfile(cfg_path):
        mt = json.load(open(cfg_path)).get("model_type", "")
        if mt in ("bert", "xlm-roberta", "roberta"):
            from .models.embedding import EncoderModel

            return EncoderModel(args.path, device)
    m = llm.model(args.path, dtype=args.dtype, kv_cache_dtype=args.kv_cache_dtype, moe_dtype=args.moe_dtype, lora=args.lora,
                  dtype_config=args.dtype_config, ori_model_path=args.ori, chat_template=args.chat_template,
                  tool_call_parser=args.tool_call_parser, device=device, tp=tp, graph=(getattr(args, "custom", "") or None))
    if m.is_worker:
        # a non-zero rank of an outer launcher's job: it has served until rank 0 shut the group down
        raise SystemExit(0)
    m.torch_model.source_path = args.path
    return m
