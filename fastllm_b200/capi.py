"""Flat facade of ``llm.model`` for the C ABI.

The native host library (``csrc/capi/fastllm_capi.cpp``, built as ``lib/libfastllm_b200.so``) embeds the interpreter and
calls the functions below; every argument and result is an int, float, str, bytes or list of ints, so the C++ side needs no
knowledge of the package's classes.  Models and requests are named by small integers, as in the reference's C ABI
(tools/src/pytools.cpp:183-205 ``ModelManager``, :369-420 the ``create_*`` family, :721-1000 launch / fetch).
"""
from __future__ import annotations

import json
import threading

_lock = threading.Lock()
_models: dict[int, object] = {}
_decoders: dict[tuple[int, int], object] = {}
_final_stats: dict[tuple[int, int], dict] = {}      # statistics of ended requests (the engine forgets them at the last fetch)
_next_id = 0


def _model(mid: int):
    m = _models.get(mid)
    if m is None:
        raise KeyError(f"no model with id {mid}")
    return m


def create_model(path: str, dtype: str = "auto", options_json: str = "") -> int:
    """Load a model folder (Hugging Face layout, ``.flm`` or GGUF file) and return its id.  ``options_json``: keyword
    arguments of ``llm.model`` (``kv_cache_dtype``, ``moe_dtype``, ``device``, ``tp``, ``lora`` ...) and the engine settings
    ``max_batch``, ``max_tokens``, ``gpu_mem_ratio``, ``chunked_prefill_size``, ``max_context_length``, ``page_size``,
    ``cuda_graph``, ``prefix_cache``, ``cpu_threads``."""
    global _next_id
    from . import llm

    opts = json.loads(options_json) if options_json else {}
    for name in ("max_batch", "max_tokens", "gpu_mem_ratio", "chunked_prefill_size", "max_context_length", "page_size", "cuda_graph",
                 "prefix_cache", "cpu_threads"):
        if name in opts:                          # process-wide engine settings (the reference's set_* calls before create)
            getattr(llm, "set_" + name)(opts.pop(name))
    m = llm.model(path, dtype=dtype or "auto", **opts)
    with _lock:
        mid = _next_id
        _next_id += 1
        _models[mid] = m
    return mid


def release(mid: int) -> None:
    with _lock:
        m = _models.pop(mid, None)
        for k in [k for k in _decoders if k[0] == mid]:
            _decoders.pop(k, None)
    if m is not None:
        m.release_memory()


def _gen_kwargs(max_length, min_length, do_sample, top_p, top_k, temperature, repeat_penalty, stop_ids):
    return dict(max_length=int(max_length) if max_length > 0 else 4096, min_length=int(min_length), do_sample=bool(do_sample),
                top_p=float(top_p) if top_p > 0 else None, top_k=int(top_k) if top_k > 0 else None,
                temperature=float(temperature) if temperature > 0 else None,
                repeat_penalty=float(repeat_penalty) if repeat_penalty > 0 else None, stop_token_ids=list(stop_ids or []))


def launch_tokens(mid: int, ids, max_length=0, min_length=0, do_sample=0, top_p=0.0, top_k=0, temperature=0.0, repeat_penalty=0.0,
                  stop_ids=None) -> int:
    return _model(mid).launch_stream_response([int(t) for t in ids],
                                              **_gen_kwargs(max_length, min_length, do_sample, top_p, top_k, temperature,
                                                            repeat_penalty, stop_ids))


def launch_text(mid: int, content: str, as_chat=1, max_length=0, min_length=0, do_sample=0, top_p=0.0, top_k=0, temperature=0.0,
                repeat_penalty=0.0, stop_ids=None) -> int:
    """``as_chat``: wrap ``content`` as one user turn of the model's chat template; otherwise it is the raw prompt."""
    m = _model(mid)
    q = content if as_chat else m.encode(content)
    return m.launch_stream_response(q, **_gen_kwargs(max_length, min_length, do_sample, top_p, top_k, temperature, repeat_penalty,
                                                     stop_ids))


def launch_request_json(mid: int, body: str) -> int:
    """A chat-completions style request body: ``messages`` (or ``prompt``), ``max_tokens``, ``temperature``, ``top_p``,
    ``top_k``, ``repetition_penalty``; the HTTP host passes the body through unparsed."""
    m = _model(mid)
    req = json.loads(body)
    temperature = req.get("temperature")
    kw = dict(max_length=int(req.get("max_tokens") or req.get("max_completion_tokens") or 4096),
              do_sample=temperature is None or float(temperature) > 1e-6, top_p=req.get("top_p"), top_k=req.get("top_k"),
              temperature=temperature, repeat_penalty=req.get("repetition_penalty") or req.get("repeat_penalty"))
    if "messages" in req:
        return m.launch_stream_response(list(req["messages"]), **kw)
    prompt = req.get("prompt", "")
    return m.launch_stream_response(m.encode(prompt if isinstance(prompt, str) else prompt[0]), **kw)


def request_wants_stream(body: str) -> int:
    try:
        return int(bool(json.loads(body).get("stream", False)))
    except (ValueError, AttributeError):
        return 0


def can_fetch(mid: int, handle: int) -> int:
    return int(_model(mid).engine.can_fetch(handle))


def _fetch(m, mid: int, handle: int) -> int:
    req = m.engine.requests.get(handle)
    tok = int(m.engine.fetch(handle))
    if tok < 0 and req is not None:
        if len(_final_stats) >= 4096:
            _final_stats.pop(next(iter(_final_stats)))
        _final_stats[(mid, handle)] = req.stats.as_dict()
    return tok


def fetch_token(mid: int, handle: int) -> int:
    """Next token id of the request (blocks until there is one); -1 once it has ended."""
    return _fetch(_model(mid), mid, handle)


def fetch_text(mid: int, handle: int):
    """Next piece of decoded text (complete UTF-8 only; may be empty while a multi-byte character is pending), ``None``
    once the request has ended."""
    from .tokenizer import StreamDecoder

    m = _model(mid)
    key = (mid, handle)
    sd = _decoders.get(key)
    if sd is None:
        sd = _decoders[key] = StreamDecoder(m.tokenizer)
    tok = _fetch(m, mid, handle)
    if tok < 0:
        _decoders.pop(key, None)
        return None
    return sd.push(tok)


def abort(mid: int, handle: int) -> None:
    _decoders.pop((mid, handle), None)
    _model(mid).abort_handle(handle)


def response_text(mid: int, content: str, as_chat=1, max_length=0, min_length=0, do_sample=0, top_p=0.0, top_k=0, temperature=0.0,
                  repeat_penalty=0.0, stop_ids=None) -> str:
    h = launch_text(mid, content, as_chat, max_length, min_length, do_sample, top_p, top_k, temperature, repeat_penalty, stop_ids)
    out = []
    while True:
        piece = fetch_text(mid, h)
        if piece is None:
            return "".join(out)
        out.append(piece)


def encode(mid: int, text: str):
    return [int(t) for t in _model(mid).encode(text)]


def decode_token(mid: int, token: int) -> bytes:
    return bytes(_model(mid).tokenizer_decode_token(int(token)))


def apply_chat_template(mid: int, messages_json: str) -> str:
    return _model(mid).apply_chat_template(json.loads(messages_json))


def stats_json(mid: int, handle: int) -> str:
    """``prompt_tokens``, ``cached_tokens``, ``output_tokens``, ``ttft_s``, ``tpot_s`` of a running or ended request."""
    return json.dumps(_model(mid).get_response_statistics(handle) or _final_stats.get((mid, handle), {}))


def info_json(mid: int) -> str:
    m = _model(mid)
    return json.dumps({"type": m.get_type(), "vocab_size": int(m.torch_model.cfg.vocab_size), "max_input_len": int(m.get_max_input_len()),
                       "kv_cache_token_limit": int(m.get_kv_cache_token_limit()), "max_batch": int(m.get_max_batch())})


def set_option(mid: int, name: str, value: str) -> None:
    """Per-model setters of the reference's ABI by name: ``max_batch``, ``max_context_length``, ``chunked_prefill_size``,
    ``kv_cache_limit``, ``save_history``, ``verbose``, ``atype``, ``moe_atype``, ``kv_cache_dtype``, ``moe_experts``."""
    m = _model(mid)
    conv = {"max_batch": int, "max_context_length": int, "chunked_prefill_size": int, "kv_cache_limit": str,
            "save_history": lambda v: v not in ("0", "false", "False", ""), "verbose": int, "atype": str, "moe_atype": str,
            "kv_cache_dtype": str, "moe_experts": int}
    if name not in conv:
        raise KeyError(f"unknown option {name!r}")
    getattr(m, "set_" + name)(conv[name](value))
