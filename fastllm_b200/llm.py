"""Public Python API: ``llm.model(path, ...)`` with ``response`` / ``stream_response`` / handle-based streaming.

Mirrors the surface of the reference's ``ftllm.llm`` (tools/fastllm_pytools/llm.py: ``model.__init__`` :1083,
``response`` :1929, ``stream_response`` :1947, ``launch_stream_response`` :2082, ``abort_handle`` :2402,
``stream_response_handle`` :2429, ``response_logits`` :1900, module-level ``set_device_map`` etc. :589-640), on
top of the in-process engine instead of a ctypes bridge to a separate runtime.
"""
from __future__ import annotations

import asyncio
import os
import threading
from pathlib import Path
from typing import Iterable

import torch

from .engine import EngineConfig, GenerationConfig, LLMEngine
from .graph import ComputeGraph  # noqa: F401  (custom model files import it from here, as with the reference)
from .models.decoder import TPInfo
from .tokenizer import StreamDecoder, Tokenizer

# ---- module-level settings (reference: set_device_map / set_cpu_threads / ... before creating a model) ----
_settings = {"device": None, "device_map": None, "moe_device_map": None, "threads": None, "max_batch": 256, "max_tokens": None,
             "gpu_mem_ratio": 0.9, "chunked_prefill_size": 8192, "max_context": 8192, "page_size": 128, "cuda_graph": True,
             "prefix_cache": True, "speculative": "", "speculative_tokens": 4, "draft_model_path": "", "draft_dtype": ""}

fastllm_data_type_dict = {"": 0, "auto": 100003, "int2g": 11, "int4g": 9, "int4": 8, "int8": 3, "float16": 7, "fp16": 7, "half": 7,
                          "bfloat16": 1, "bf16": 1, "float32": 0, "fp8": 10, "float8": 10, "fp8_e4m3": 10}


def set_device_map(device_map, is_moe: bool = False):
    """``"cuda"``, ``"cuda:1"``, ``"cpu"``, a list of devices or a ``{device: layers}`` dict (layer split)."""
    _settings["moe_device_map" if is_moe else "device_map"] = device_map


def set_cpu_threads(n: int):
    """Worker threads of the native CPU backend (and of PyTorch's own CPU ops)."""
    from .ops import cpu

    _settings["threads"] = n
    torch.set_num_threads(max(1, n))
    if cpu.available():
        cpu.set_threads(max(1, n))


def get_cpu_threads() -> int:
    from .ops import cpu

    return cpu.get_threads() if cpu.available() else torch.get_num_threads()


def set_max_batch(n: int):
    _settings["max_batch"] = n


def set_max_tokens(n: int):
    _settings["max_tokens"] = n


def set_gpu_mem_ratio(r: float):
    _settings["gpu_mem_ratio"] = r


def set_chunked_prefill_size(n: int):
    _settings["chunked_prefill_size"] = n


def set_max_context_length(n: int):
    _settings["max_context"] = n


def set_page_size(n: int):
    if n not in (-1, 128):
        raise ValueError("this build uses 128-token KV pages (one page = one tensor-core tile)")


def set_cuda_graph(on: bool):
    _settings["cuda_graph"] = bool(on)


def set_prefix_cache(on: bool):
    _settings["prefix_cache"] = bool(on)


# ---- the rest of the reference's module-level switches (tools/fastllm_pytools/llm.py:290-640) -------------------------------
def set_model_load_progress_callback(callback):
    """``callback(stage, current, total, completed_bytes, total_bytes)`` during model load (None removes it)."""
    from .serving import progress

    progress.set_callback(callback)


def report_model_load_progress(stage, current=0, total=0, completed_bytes=0, total_bytes=0):
    from .serving import progress

    progress.emit(str(stage), int(current), int(total), completed_bytes=int(completed_bytes), total_bytes=int(total_bytes))


def export_llm_model_fromhf(path: str, output: str, dtype: str = "float16", moe_dtype: str = "", lora: str = "", dtype_config: str = ""):
    """Quantise an HF folder into a reloadable HF-layout export (the ``ftllm export`` command)."""
    from .loader.export import export_quantized_hf

    if lora or dtype_config:
        raise NotImplementedError("export takes dtype / moe_dtype; adapters and dtype_config rules apply at load time")
    export_quantized_hf(path, output, "float16" if dtype == "auto" else dtype, moe_dtype or None)


def softmax(a):
    import numpy as np

    a = np.asarray(a, dtype=np.float64)
    e = np.exp(a - a.max())
    return e / e.sum()


def has_device(device_type: str) -> bool:
    d = str(device_type).lower()
    if d == "cpu":
        return True
    if d == "cuda":
        return torch.cuda.is_available()
    if d == "multicuda":
        return torch.cuda.is_available() and torch.cuda.device_count() > 1
    if d in ("numa", "disk"):
        return True          # host placements of the routed experts (``--moe_device``)
    return False


def print_ins_info():
    """Instruction sets the native CPU backend was built for / runs with."""
    from .ops import cpu

    print("cpu backend:", cpu.isa() if cpu.available() else "not built", "| cuda:", torch.cuda.is_available())


def set_cpu_kvcache(cpu_kvcache):
    """KV pages in host memory.  The tensor-core attention kernels read HBM pages only: the switch is recorded and models on a
    GPU keep their cache on the device (a CPU model's cache is in host memory anyway)."""
    _settings["cpu_kvcache"] = bool(cpu_kvcache)


def get_cpu_kvcache():
    return bool(_settings.get("cpu_kvcache", False))


def set_cpu_historycache(cpu_historycache):
    """Prefix-cache history in host memory: recorded; cached prefix pages stay in the device page pool."""
    _settings["cpu_historycache"] = bool(cpu_historycache)


def get_cpu_historycache():
    return bool(_settings.get("cpu_historycache", False))


def set_cuda_embedding(cuda_embedding):
    _settings["cuda_embedding"] = bool(cuda_embedding)          # the embedding table always lives with the model's first layer


def set_cuda_slab(mb: int):
    _settings["cuda_slab_mb"] = int(mb)                          # device memory comes from PyTorch's caching allocator


def disable_cuda_malloc():
    """Steady-state decode allocates nothing new (static CUDA-graph buffers); kept for interface compatibility."""
    _settings["cuda_malloc_disabled"] = True


def set_enable_amx(enable_amx):
    """Switch the CPU backend's reduced-precision-activation kernels (AMX tiles, AVX-512 VNNI / BF16) on or off; what the CPU
    does not have stays off.  (Reference: ``--enable_amx``, fastllm.EnableAMX.)"""
    _settings["enable_amx"] = bool(enable_amx)
    from .ops import cpu

    if cpu.available():
        cpu.set_accel(7 if enable_amx else 0)


def set_cuda_shared_expert(cuda_shared_expert):
    _settings["cuda_shared_expert"] = bool(cuda_shared_expert)   # shared experts stay on the GPU under ``--moe_device cpu``


def set_cpu_low_mem(low_mem):
    _settings["cpu_low_mem"] = bool(low_mem)


def get_cpu_low_mem():
    return bool(_settings.get("cpu_low_mem", False))


def set_layered_moe_device_map(device_map):
    """Placement of the routed experts (``"cpu"``, ``"disk"``, a list or ``{device: weight}``); same as
    ``set_device_map(device_map, is_moe=True)``."""
    if isinstance(device_map, (list, tuple)) and device_map:
        device_map = str(device_map[0])
    elif isinstance(device_map, dict) and device_map:
        device_map = str(next(iter(device_map)))
    _settings["moe_device_map"] = device_map


def set_moe_device_layers(layers: int):
    """Only the first ``layers`` MoE layers use the expert placement (negative: all)."""
    _settings["moe_device_layers"] = int(layers)


def GraphNode(name: str, type: str = "data", value=None):
    d = {"name": name, "type": type}
    if value:
        d["value"] = value
    return d


def FloatGraphNode(v):
    if isinstance(v, (int, str)):
        v = float(v)
    if isinstance(v, float):
        return GraphNode("", "constant.float", v)
    if isinstance(v, dict):
        v["type"] = "config.float"
    return v


def IntGraphNode(v):
    if isinstance(v, float):
        v = int(v)
    if isinstance(v, int):
        return GraphNode("", "constant.int", v)
    if isinstance(v, dict):
        v["type"] = "config.int"
    return v


def _resolve_device():
    dm = _settings["device_map"]
    if isinstance(dm, str):
        d = dm.replace("multicuda", "cuda")
        return d.split(",")[0] if ":" in d else d
    if isinstance(dm, (list, tuple)) and dm:
        return str(dm[0])
    if isinstance(dm, dict) and dm:
        return str(next(iter(dm)))
    return "cuda" if torch.cuda.is_available() else "cpu"


def _parallel_devices(tp, device=None) -> list[str]:
    """Devices of a parallel group from the ``tp`` argument: a count, ``"auto"``, ``"0,2"``, a list of ids / device strings."""
    if tp == "env":
        return []
    if isinstance(tp, str):
        from .util import parse_tp

        tp = parse_tp(tp)
    if isinstance(tp, int):
        tp = list(range(tp))
    out = []
    for d in tp or []:
        out.append(d if isinstance(d, str) else (f"cuda:{int(d)}" if (device or "cuda").startswith("cuda") else "cpu"))
    return out


class model:
    """A loaded model plus its serving engine (started lazily on first request)."""

    def __init__(self, path: str, id: int = -99999, dtype: str = "auto", kv_cache_dtype: str = "auto", moe_dtype: str = "",
                 system_prompt: str = "", eos_token: Iterable[str] | None = None, tokenizer_type: str = "auto",
                 model_json: str = "", graph=None, lora: str = "", dtype_config: str = "", ori_model_path: str = "",
                 chat_template: str = "", tool_call_parser: str = "auto", device: str | None = None, tp=None,
                 engine_config: EngineConfig | None = None, _model=None, _defer_fused: bool = False):
        """``tp``: ``None`` (one device); a GPU count, ``"auto"``, a list of GPU ids / device strings -- the model is
        then sharded over those devices, this process being rank 0 and one spawned worker process per further
        device (``parallel/launcher.py``); ``"env"`` inside a job whose ranks an outer launcher started (RANK /
        WORLD_SIZE set: rank 0 returns a normal model object, the other ranks serve inside this call and come back
        with ``is_worker`` set when rank 0 shuts down); or a ready ``TPInfo`` (one rank of an SPMD program)."""
        from .loader import hf as hf_loader

        self._group = None
        self.is_worker = False
        if tp is not None and not isinstance(tp, TPInfo):
            devices = _parallel_devices(tp, device)
            if tp == "env" or len(devices) > 1:
                kwargs = dict(path=path, dtype=dtype, kv_cache_dtype=kv_cache_dtype, moe_dtype=moe_dtype, system_prompt=system_prompt,
                              eos_token=list(eos_token) if eos_token else None, tokenizer_type=tokenizer_type, model_json=model_json,
                              graph=graph if isinstance(graph, str) else None, lora=lora, dtype_config=dtype_config,
                              ori_model_path=ori_model_path, chat_template=chat_template, tool_call_parser=tool_call_parser)
                self._init_parallel(kwargs, devices, engine_config, attach=(tp == "env"))
                return
            tp, device = None, (devices[0] if devices else device)
        self.path = path
        self.system_prompt = system_prompt
        self.tool_call_parser = tool_call_parser
        dev = device or _resolve_device()
        tpl = Path(chat_template).read_text(encoding="utf-8") if chat_template and os.path.exists(chat_template) else (chat_template or None)
        self.tokenizer = Tokenizer(path if path and os.path.isdir(path) else None, prefer_native=(tokenizer_type == "native"),
                                   chat_template=tpl)
        self.hf_tokenizer = self.tokenizer.hf
        if _model is not None:
            self.torch_model = _model
        elif graph is not None:
            from . import graph as G

            cls = G.load_custom_file(graph) if isinstance(graph, str) else graph
            self.torch_model = G.load_graph_model(path, cls, device=dev)
        elif path and path.endswith(".flm"):
            from .loader import flm

            self.torch_model = flm.load_model(path, device=dev, tp=tp)
        elif path and path.endswith(".gguf"):
            from .loader import gguf

            self.torch_model = gguf.load_model(path, device=dev, ori=ori_model_path or None, tp=tp)
            meta = self.torch_model.gguf_meta
            if ori_model_path and os.path.isdir(ori_model_path):
                self.tokenizer = Tokenizer(ori_model_path, prefer_native=(tokenizer_type == "native"), chat_template=tpl)
                self.hf_tokenizer = self.tokenizer.hf
            elif self.tokenizer.hf is None and self.tokenizer.native is None:
                from .tokenizer import NativeBPE

                tj = gguf.tokenizer_json_from_meta(meta)
                if tj is not None:
                    self.tokenizer.native = NativeBPE(tj)
                if self.tokenizer.chat_template is None and isinstance(meta.get("tokenizer.chat_template"), str):
                    self.tokenizer.chat_template = meta["tokenizer.chat_template"]
        else:
            md = _settings.get("moe_device_map")
            self.torch_model = hf_loader.load_model(path, device=dev, wdtype=dtype or "auto", moe_wdtype=moe_dtype or None, tp=tp,
                                                    moe_device=("disk" if (isinstance(md, str) and md.startswith("disk")) else
                                                                "numa" if (isinstance(md, str) and md.startswith("numa")) else
                                                                "cpu" if (isinstance(md, str) and md.startswith("cpu")) else None),
                                                    moe_device_layers=int(_settings.get("moe_device_layers", -1) or -1),
                                                    dtype_config=dtype_config or None, lora=lora or None,
                                                    device_map=_settings["device_map"] if isinstance(_settings.get("device_map"), dict) else None)
        self._image_options = {}
        pp = os.path.join(path, "preprocessor_config.json") if os.path.isdir(str(path)) else ""
        if pp and os.path.exists(pp) and getattr(self.torch_model, "vision", None) is not None:
            import json as _json

            with open(pp, "r", encoding="utf-8") as f:
                d = _json.load(f)
            size = d.get("size") if isinstance(d.get("size"), dict) else {}
            self._image_options = dict(mean=tuple(d.get("image_mean") or (0.5, 0.5, 0.5)), std=tuple(d.get("image_std") or (0.5, 0.5, 0.5)),
                                       min_pixels=d.get("min_pixels") or size.get("shortest_edge"),
                                       max_pixels=d.get("max_pixels") or size.get("longest_edge"))
        if kv_cache_dtype not in ("auto", "", None):
            self.torch_model.set_kv_cache_dtype(kv_cache_dtype)
        cfg = self.torch_model.cfg
        eos = set(cfg.eos_token_ids) | set(self.tokenizer.eos_ids())
        for t in eos_token or []:
            ids = self.tokenizer.encode(t)
            if len(ids) == 1:
                eos.add(ids[0])
        self.eos_token_ids = sorted(eos)
        ec = engine_config or EngineConfig(max_batch=_settings["max_batch"], max_context=min(_settings["max_context"], cfg.max_position),
                                           chunked_prefill_size=_settings["chunked_prefill_size"], gpu_mem_ratio=_settings["gpu_mem_ratio"],
                                           max_tokens=_settings["max_tokens"], use_cuda_graph=_settings["cuda_graph"],
                                           prefix_cache=_settings["prefix_cache"], speculative=_settings.get("speculative", ""),
                                           speculative_tokens=int(_settings.get("speculative_tokens", 4)))
        draft = None
        dpath = _settings.get("draft_model_path") or ""
        if ec.speculative == "draft" and dpath and (tp is None or tp.size == 1):
            # a smaller model of the same vocabulary proposes tokens (its KV pools sit beside the target's, same page ids)
            draft = hf_loader.load_model(dpath, device=dev, dtype=self.torch_model.dtype, wdtype=_settings.get("draft_dtype") or dtype or "auto",
                                         tp=None)
        self.engine = LLMEngine(self.torch_model, ec, eos_token_ids=self.eos_token_ids, draft_model=draft)
        if tp is not None and tp.size > 1 and tp.comm is not None and not _defer_fused and self.torch_model.on_cuda:
            from .parallel import symm

            tp.comm.fused = symm.try_create(tp.comm, cfg, min(256, ec.max_batch), max_big_m=symm.prefill_rows(ec))
        self.default_generation_config = {"repetition_penalty": 1.0, "top_p": 0.8, "top_k": 1, "temperature": 1.0}
        gc = Path(path) / "generation_config.json" if path and os.path.isdir(path) else None
        if gc is not None and gc.exists():
            import json

            g = json.loads(gc.read_text())
            for k in ("repetition_penalty", "top_p", "top_k", "temperature"):
                if g.get(k) is not None:
                    self.default_generation_config[k] = g[k]
        self._lock = threading.Lock()

    def _init_parallel(self, kwargs: dict, devices: list[str], engine_config, attach: bool):
        """Become rank 0 of a tensor-parallel group (or, for the other ranks of an outer launcher's job, serve in it)."""
        import dataclasses

        from .parallel.launcher import TPGroup

        spec = {"kind": "hf", "kwargs": {k: v for k, v in kwargs.items() if v not in (None, "")}, "settings": dict(_settings)}
        if engine_config is not None:
            spec["engine"] = dataclasses.asdict(engine_config)
        if attach:
            group, _eng, inner = TPGroup.attach(spec)
        else:
            group, _eng, inner = TPGroup.launch(spec, devices)
        self.__dict__.update(inner.__dict__)
        self._group = group
        self.is_worker = group is None

    def shutdown(self):
        """Stop the engine loop and, for a parallel model, release the worker ranks."""
        if getattr(self, "engine", None) is not None:
            self.engine.shutdown()
        if self._group is not None:
            self._group.shutdown()
            self._group = None

    # ---- text helpers -------------------------------------------------------------------------------
    def encode(self, text: str) -> list[int]:
        return self.tokenizer.encode(text)

    def decode(self, ids) -> str:
        return self.tokenizer.decode(list(ids))

    def apply_chat_template(self, messages, add_generation_prompt=True, tools=None, **kw) -> str:
        msgs = list(messages)
        if self.system_prompt and not any(m.get("role") == "system" for m in msgs):
            msgs = [{"role": "system", "content": self.system_prompt}] + msgs
        return self.tokenizer.apply_chat_template(msgs, add_generation_prompt=add_generation_prompt, tools=tools, **kw)

    def get_prompt(self, query: str, history=None) -> str:
        msgs = []
        for q, a in history or []:
            msgs += [{"role": "user", "content": q}, {"role": "assistant", "content": a}]
        msgs.append({"role": "user", "content": query})
        return self.apply_chat_template(msgs)

    def _to_ids(self, query, history=None) -> list[int]:
        if isinstance(query, (list, tuple)) and query and isinstance(query[0], int):
            return list(query)
        if isinstance(query, (list, tuple)):            # list of chat messages
            return self.encode(self.apply_chat_template(list(query)))
        return self.encode(self.get_prompt(query, history))

    def _gen_config(self, max_length=4096, do_sample=True, top_p=None, top_k=None, temperature=None, repeat_penalty=None,
                    stop_token_ids=None, min_length=0, **kw) -> GenerationConfig:
        d = self.default_generation_config
        top_k = d["top_k"] if top_k is None else top_k
        temperature = d["temperature"] if temperature is None else temperature
        sample = bool(do_sample) and top_k != 1 and temperature > 1e-6
        return GenerationConfig(max_new_tokens=max_length, min_new_tokens=min_length, do_sample=sample, top_k=top_k if sample else 1,
                                top_p=d["top_p"] if top_p is None else top_p, temperature=temperature,
                                repeat_penalty=d["repetition_penalty"] if repeat_penalty is None else repeat_penalty,
                                stop_token_ids=list(stop_token_ids or []), output_logits=bool(kw.get("output_logits", False)),
                                logprobs=int(kw.get("logprobs", 0) or 0), logits_processor=kw.get("logits_processor"))

    # ---- handle-level API ---------------------------------------------------------------------------
    def launch_stream_response(self, query, history=None, images=None, videos=None, **gen_kwargs) -> int:
        """``images``: paths, ``data:`` URLs, bytes or PIL images for a model with a vision tower; a text query gets them in
        front of the text, a message list may carry them as ``image_url`` / ``image`` content parts instead.  ``videos``: per
        video a list of frames, a frame directory, an animated GIF / WebP or a ``{"frames": [...], "fps": f}`` dict
        (``video_url`` / ``video`` parts in a message list); frames are sampled at about two per second and enter the prompt in
        groups, each behind its time stamp."""
        images = list(images or getattr(query, "images", None) or [])
        videos = list(videos or getattr(query, "videos", None) or [])
        groups = list(getattr(query, "video_groups", None) or [])       # a prompt whose video markup is expanded already
        if images or videos or (isinstance(query, (list, tuple)) and query and isinstance(query[0], dict)):
            from .models import vision

            # CogVLM places its image rows behind the first token itself: its prompts carry no placeholder markup
            marked = getattr(self.torch_model.cfg, "model_type", "") != "cogvlm"
            if isinstance(query, str) and marked:
                msgs = []
                for q, a in history or []:
                    msgs += [{"role": "user", "content": q}, {"role": "assistant", "content": a}]
                slots = "".join(vision.video_slot(k) for k in range(len(videos)))
                query = msgs + [{"role": "user", "content": vision.IMAGE_MARKER * len(images) + slots + query}]
            elif isinstance(query, (list, tuple)) and query and isinstance(query[0], dict):
                found_v = []
                query, found = vision.extract_images(query, found_v)
                images = images or found
                videos = videos or found_v
                if not marked:
                    query = [dict(m, content=m["content"].replace(vision.IMAGE_MARKER, "")) if isinstance(m.get("content"), str) else m
                             for m in query]
            if videos:
                query, groups = self.expand_videos(query, videos)
        ids = self._to_ids(query, history)
        mm = None
        if images or groups:
            from .models import vision

            ids, mm = vision.build_context(self.torch_model, ids, images, videos=groups or None, **getattr(self, "_image_options", {}))
        self.engine.start()
        return self.engine.launch(ids, self._gen_config(**gen_kwargs), mm=mm)

    def expand_videos(self, messages, videos):
        """Read and sample every video, cut its frames into temporal groups and put the groups' markup (time stamp + placeholder
        run each) in place of ``vision.video_slot(k)`` in the messages.  Returns (messages, per-video groups)."""
        from .models import vision

        tower = getattr(self.torch_model, "vision", None)
        if tower is None or getattr(self.torch_model, "video_token_id", None) is None:
            raise ValueError("this model takes no video inputs")
        opts = getattr(self, "_image_options", {})
        groups = []
        for k, v in enumerate(videos):
            frames, times = vision.load_video(v)
            g = vision.frames_to_patches(frames, times, tower.cfg, **opts)
            groups.append(g)
            messages = [dict(m, content=m["content"].replace(vision.video_slot(k), vision.video_markup(g)))
                        if isinstance(m.get("content"), str) else m for m in messages]
        return messages, groups

    def abort_handle(self, handle: int):
        self.engine.abort(handle)

    def stream_response_handle(self, handle: int, one_by_one: bool = True, skip_special_tokens: bool = True):
        sd = StreamDecoder(self.tokenizer, skip_special_tokens)
        while True:
            tok = self.engine.fetch(handle)
            if tok < 0:
                break
            piece = sd.push(tok)
            if piece:
                yield piece

    def stream_response_raw(self, input_tokens, **gen_kwargs):
        h = self.launch_stream_response(list(input_tokens), **gen_kwargs)
        while True:
            tok = self.engine.fetch(h)
            if tok < 0:
                break
            yield tok

    # ---- convenience API ----------------------------------------------------------------------------
    def stream_response(self, query, history=None, max_length=4096, do_sample=True, top_p=None, top_k=None, temperature=None,
                        repeat_penalty=None, one_by_one=True, stop_token_ids=None, images=None, videos=None, **kw):
        h = self.launch_stream_response(query, history, images=images, videos=videos, max_length=max_length, do_sample=do_sample, top_p=top_p,
                                        top_k=top_k, temperature=temperature, repeat_penalty=repeat_penalty,
                                        stop_token_ids=stop_token_ids)
        try:
            yield from self.stream_response_handle(h, one_by_one)
        except GeneratorExit:
            self.abort_handle(h)
            raise

    async def stream_response_async(self, query, history=None, **kw):
        loop = asyncio.get_running_loop()
        h = self.launch_stream_response(query, history, **kw)
        sd = StreamDecoder(self.tokenizer)
        try:
            while True:
                tok = await loop.run_in_executor(None, self.engine.fetch, h)
                if tok < 0:
                    break
                piece = sd.push(tok)
                if piece:
                    yield piece
        except (asyncio.CancelledError, GeneratorExit):
            self.abort_handle(h)
            raise

    def response(self, query, history=None, **kw) -> str:
        return "".join(self.stream_response(query, history, **kw))

    def response_logits(self, query, history=None):
        """Logits of the token that follows the prompt (fp32 tensor ``[vocab]``)."""
        ids = self._to_ids(query, history)
        self.engine.start()
        h = self.engine.launch(ids, GenerationConfig(max_new_tokens=1, output_logits=True, do_sample=True, top_k=2, temperature=1.0))
        req = self.engine.requests[h]
        while self.engine.fetch(h) >= 0:
            pass
        return req.last_logits

    def response_batch(self, queries, **kw) -> list[str]:
        hs = [self.launch_stream_response(q, **kw) for q in queries]
        return ["".join(self.stream_response_handle(h)) for h in hs]

    def add_cache(self, prompt) -> int:
        """Prefill ``prompt`` once so that its full pages sit in the prefix cache for later requests that start with it
        (reference: add_cache_llm_model, tools/src/pytools.cpp:1006).  Returns the number of prompt tokens."""
        ids = self._to_ids(prompt) if not (isinstance(prompt, list) and prompt and isinstance(prompt[0], int)) else list(prompt)
        self.engine.start()
        h = self.engine.launch(ids, GenerationConfig(max_new_tokens=1, ignore_eos=True))
        while self.engine.fetch(h) >= 0:
            pass
        return len(ids)

    def load_adapter(self, name: str, adapter_dir: str) -> int:
        """Attach a PEFT LoRA adapter folder under ``name`` for run-time switching (``fastllm_b200/lora.py``)."""
        from . import lora

        n = lora.load_adapter(self.engine.model, name, adapter_dir)
        self._adapters = getattr(self, "_adapters", set()) | {name}
        return n

    def _switch_adapter(self, name):
        from . import lora

        lora.set_adapter(name)
        runner = self.engine.runner
        for slot in runner.slots.values():          # the captured decode graphs hold the previous operator sequence
            slot.graph = None

    def set_adapter(self, name: str):
        """Run with the adapter ``name`` (loaded by ``load_adapter``) from the next request on.
        Reference: tools/fastllm_pytools/llm.py:2709."""
        if name not in getattr(self, "_adapters", set()):
            raise KeyError(f"adapter '{name}' is not loaded: call load_adapter(name, adapter_dir) first "
                           f"(llm.model(path, lora=dir) merges an adapter at load instead)")
        self._switch_adapter(name)

    def disable_adapter(self):
        """Back to the base weights.  Reference: tools/fastllm_pytools/llm.py:2712."""
        self._switch_adapter(None)

    # ---- HF-style conveniences and run-time setters of the reference (tools/fastllm_pytools/llm.py:1338-2810) --------------
    def eval(self):
        return self

    def generate(self, inputs, max_length: int = 4096, do_sample: bool = True, top_p=None, top_k=None, temperature=None,
                 repeat_penalty=None, stop_token_ids=None, **kw):
        """Token-id lists in, token-id lists out (prompt + generated ids, like ``transformers`` ``generate``)."""
        rows = inputs.tolist() if hasattr(inputs, "tolist") else list(inputs)
        if rows and isinstance(rows[0], int):
            rows = [rows]
        hs = [self.launch_stream_response([int(t) for t in r], max_length=max_length, do_sample=do_sample, top_p=top_p, top_k=top_k,
                                          temperature=temperature, repeat_penalty=repeat_penalty, stop_token_ids=stop_token_ids)
              for r in rows]
        outs = []
        for r, h in zip(rows, hs):
            out = list(r)
            while True:
                tok = self.engine.fetch(h)
                if tok < 0:
                    break
                out.append(tok)
            outs.append(out)
        return outs

    def chat(self, tokenizer, query: str, history=None, max_length: int = 8192, do_sample=True, top_p=0.8, top_k=1, temperature=1.0,
             repeat_penalty=1.0, stop_token_ids=None, **kwargs):
        """ChatGLM-style: returns ``(response, history + [(query, response)])``; ``tokenizer`` is accepted for compatibility."""
        history = list(history or [])
        text = self.response(query, history, max_length=max_length, do_sample=do_sample, top_p=top_p, top_k=top_k,
                             temperature=temperature, repeat_penalty=repeat_penalty, stop_token_ids=stop_token_ids)
        return text, history + [(query, text)]

    def stream_chat(self, tokenizer, query: str, history=None, past_key_values=None, max_length: int = 8192, do_sample=True, top_p=0.8,
                    top_k=1, temperature=1.0, repeat_penalty=1.0, return_past_key_values=False, stop_token_ids=None, **kwargs):
        history = list(history or [])
        text = ""
        for piece in self.stream_response(query, history, max_length=max_length, do_sample=do_sample, top_p=top_p, top_k=top_k,
                                          temperature=temperature, repeat_penalty=repeat_penalty, stop_token_ids=stop_token_ids):
            text += piece
            item = (text, history + [(query, text)])
            yield item + (None,) if return_past_key_values else item

    def trans_conversation(self, conversation):
        """Messages whose ``content`` is a list of typed parts are flattened to their text."""
        out = []
        for m in conversation:
            c = m.get("content")
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if isinstance(p, dict))
            out.append(dict(m, content=c))
        return out

    def get_input_token_len(self, conversation, add_generation_prompt=True, **kw) -> int:
        if isinstance(conversation, str):
            return len(self.encode(self.get_prompt(conversation)))
        return len(self.encode(self.apply_chat_template(self.trans_conversation(list(conversation)),
                                                        add_generation_prompt=add_generation_prompt)))

    def tokenizer_encode_string(self, content: str) -> list[int]:
        return self.encode(content)

    def tokenizer_decode_token(self, token_id: int) -> bytes:
        cache = getattr(self, "tokenizer_decode_token_cache", None)
        if cache is not None and token_id in cache:
            return cache[token_id]
        return self.tokenizer.decode_bytes([int(token_id)]) if hasattr(self.tokenizer, "decode_bytes") \
            else self.decode([int(token_id)]).encode("utf-8", errors="ignore")

    def build_tokenizer_decode_token_cache(self):
        if getattr(self, "tokenizer_decode_token_cache", None) is None:
            self.tokenizer_decode_token_cache = None
            self.tokenizer_decode_token_cache = {i: self.tokenizer_decode_token(i) for i in range(self.torch_model.cfg.vocab_size)}

    def token_healing(self, prompt: str):
        """Generate from ``prompt`` with its last token re-chosen among the tokens that start with that token's text (so a
        prompt cut in the middle of a word continues with the natural token)."""
        ids = self.encode(prompt)
        if len(ids) < 2:
            return self.response(ids)
        tail = self.decode(ids[-1:])
        logits = torch.as_tensor(self.response_logits(ids[:-1])).float()
        cand = [i for i in range(min(logits.numel(), self.torch_model.cfg.vocab_size)) if self.decode([i]).startswith(tail)] or [ids[-1]]
        best = max(cand, key=lambda i: float(logits[i]))
        return self.decode([best])[len(tail):] + self.response(ids[:-1] + [best])

    def _engine_cfg(self):
        return self.engine.cfg

    def set_max_batch(self, batch: int):
        self._engine_cfg().max_batch = max(1, int(batch))

    def get_max_batch(self) -> int:
        return int(self._engine_cfg().max_batch)

    def set_max_context_length(self, length: int):
        self._engine_cfg().max_context = int(length)

    def set_chunked_prefill_size(self, size: int):
        self._engine_cfg().chunked_prefill_size = max(128, int(size))

    def set_kv_cache_limit(self, limit: str):
        """``"8G"`` / ``"512M"`` / bytes: informational here -- the page pool is sized when the model is built
        (``gpu_mem_ratio`` / ``max_tokens``); the value is kept for ``get_kv_cache_token_limit`` callers."""
        s_ = str(limit).strip().lower()
        mul = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30}.get(s_[-1:], 1)
        self.kv_cache_limit_bytes = int(float(s_[:-1] if s_[-1:] in "kmg" else s_) * mul)

    def set_save_history(self, save: bool):
        self.save_history = bool(save)            # prefix reuse is the page trie's job (``set_prefix_cache``)

    def set_verbose(self, verbose: int):
        self.verbose = int(verbose)

    def set_atype(self, atype: str):
        want = {"float16": torch.float16, "half": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32, "auto": None}.get(str(atype))
        if want is not None and want != self.torch_model.dtype:
            raise ValueError(f"activations are {self.torch_model.dtype} since load time; pass dtype= to llm.model to choose another type")

    def set_moe_atype(self, moe_atype: str):
        self.set_atype(moe_atype)

    def set_kv_cache_dtype(self, kv_cache_dtype: str):
        if str(kv_cache_dtype) not in ("auto", ""):
            raise RuntimeError("the page pool exists already: pass kv_cache_dtype= to llm.model(...)")

    def set_moe_experts(self, experts: int):
        """Route every token to ``experts`` experts instead of the checkpoint's top-k."""
        self.torch_model.cfg.num_experts_per_tok = int(experts)
        for slot in self.engine.runner.slots.values():
            slot.graph = None

    def set_cuda_shared_expert(self, cuda_shared_expert: bool):
        set_cuda_shared_expert(cuda_shared_expert)

    def embedding_sentence(self, input: str, normalize: bool = True):
        """Sentence embedding of an encoder model (bert / xlm-roberta folders: ``models.embedding.EncoderModel``)."""
        from .models.embedding import embed_texts

        return embed_texts(self, [input], normalize=normalize)[0]

    def reranker_compute_score(self, pairs):
        """Relevance score of every ``(query, text)`` pair (sequence-classification encoder folders)."""
        from .models.embedding import rerank_scores

        return [rerank_scores(self, q, [t])[0] for q, t in pairs]

    def get_response_statistics(self, handle: int) -> dict:
        return self.engine.stats(handle)

    def warmup(self):
        list(self.stream_response_raw([1, 2, 3, 4], max_length=2, do_sample=False))

    def get_type(self) -> str:
        return self.torch_model.cfg.model_type

    def get_struct(self) -> str:
        return self.torch_model.cfg.model_type

    def get_max_input_len(self) -> int:
        return self.engine.cfg.max_context

    def get_kv_cache_token_limit(self) -> int:
        return self.engine.runner.kv.num_pages * self.engine.cfg.page_len

    def save(self, path: str, dtype: str = "auto"):
        from .loader import flm

        flm.save_model(self.torch_model, self.tokenizer, path, dtype)

    def release_memory(self):
        self.shutdown()
        self.engine = None
        self.torch_model = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def stop_token_ctypes(self, stop_token_ids):      # kept for scripts written against the reference package
        return (0, None) if stop_token_ids is None else (len(stop_token_ids), list(stop_token_ids))


def from_hf(hf_model, tokenizer=None, dtype: str = "float16", device: str | None = None):
    """Create a ``model`` from an in-memory Hugging Face model (reference: llm.from_hf, hf_model.py)."""
    from .loader.shard import finalize_model
    from .models.config import from_hf_dict
    from .models.decoder import DecoderModel

    cfg = from_hf_dict(hf_model.config.to_dict())
    sd = {k: v.detach() for k, v in hf_model.state_dict().items()}
    dev = device or _resolve_device()
    tdt = torch.float32 if dev == "cpu" else (torch.bfloat16 if dtype in ("bfloat16", "bf16") else torch.float16)
    m = DecoderModel(cfg, dev, tdt)
    from .loader.hf import canonical_name

    sd = {canonical_name(k): v for k, v in sd.items()}
    finalize_model(m, lambda: {k: v for k, v in sd.items() if not k.startswith("model.layers.")},
                   lambda i: {k: v for k, v in sd.items() if k.startswith(f"model.layers.{i}.")},
                   wdtype=dtype if dtype not in ("float16", "bfloat16", "float32") else "dense")
    obj = model.__new__(model)
    model.__init__(obj, "", _model=m, device=dev)
    if tokenizer is not None:
        obj.tokenizer.hf = tokenizer
        obj.hf_tokenizer = tokenizer
        if getattr(tokenizer, "chat_template", None):
            obj.tokenizer.chat_template = tokenizer.chat_template
        if tokenizer.eos_token_id is not None:
            obj.engine.eos.add(tokenizer.eos_token_id)
    return obj
