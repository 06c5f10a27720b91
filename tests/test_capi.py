"""The C ABI (``lib/libfastllm_b200.so``) and the native hosts over it, on the CPU backend with a synthetic tiny model.

In-process: the library is loaded with ctypes into this interpreter and its results are compared with ``llm.model`` on the same
folder.  Out of process: ``fastllm_chat``, ``fastllm_benchmark`` and ``fastllm_apiserver`` start their own embedded interpreter.
"""
import ctypes
import json
import os
import socket
import subprocess
import sys
import time
import urllib.request
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "fastllm_b200" / "lib" / "libfastllm_b200.so"
BIN = ROOT / "fastllm_b200" / "bin"


@pytest.fixture(scope="module")
def built():
    from fastllm_b200 import build

    if build.build_capi() is None:
        pytest.skip("interpreter headers / shared library not available")
    return LIB


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from baseline import synth

    return synth.write_model("tiny-llama", str(tmp_path_factory.mktemp("capi") / "m"), dtype=torch.float32, std=0.05)


class GenCfg(ctypes.Structure):
    _fields_ = [("max_length", ctypes.c_int), ("min_length", ctypes.c_int), ("do_sample", ctypes.c_int), ("top_k", ctypes.c_int),
                ("top_p", ctypes.c_float), ("temperature", ctypes.c_float), ("repeat_penalty", ctypes.c_float),
                ("stop_token_cnt", ctypes.c_int), ("stop_token_ids", ctypes.POINTER(ctypes.c_int))]


def _take(lib, p):
    s = ctypes.cast(p, ctypes.c_char_p).value.decode()
    lib.fastllm_free(p)
    return s


def test_c_abi_in_process(built, folder):
    from fastllm_b200 import llm

    lib = ctypes.CDLL(str(built))
    lib.fastllm_last_error.restype = ctypes.c_char_p
    for fn in ("fetch_response_str_llm_model", "response_str_llm_model", "get_info_llm_model", "get_response_statistics_llm_model",
               "apply_chat_template"):
        getattr(lib, fn).restype = ctypes.c_void_p
    lib.fastllm_free.argtypes = [ctypes.c_void_p]
    assert lib.create_llm_model_fromhf(b"/no/such/folder", b"auto", b'{"device": "cpu"}') == -1
    assert lib.fastllm_last_error()

    mid = lib.create_llm_model_fromhf(folder.encode(), b"float32", b'{"device": "cpu"}')
    assert mid >= 0, lib.fastllm_last_error()
    info = json.loads(_take(lib, lib.get_info_llm_model(mid)))
    assert info["type"] == "llama" and info["vocab_size"] > 0

    ref = llm.model(folder, dtype="float32", device="cpu")
    text = "hello world"
    want_ids = ref.encode(text)
    buf = (ctypes.c_int * 64)()
    n = lib.token_encode_string(mid, text.encode(), 64, buf)
    assert list(buf[:n]) == want_ids
    out = ctypes.create_string_buffer(64)
    k = lib.token_decode(mid, want_ids[0], 64, out)
    assert out.raw[:k] == bytes(ref.tokenizer_decode_token(want_ids[0]))

    prompt = [3, 9, 27, 81, 5]
    want = list(ref.stream_response_raw(prompt, max_length=8, do_sample=False))
    cfg = GenCfg(max_length=8, top_k=1)
    h = lib.launch_response_llm_model(mid, len(prompt), (ctypes.c_int * len(prompt))(*prompt), ctypes.byref(cfg))
    assert h >= 0, lib.fastllm_last_error()
    got = []
    while True:
        t = lib.fetch_response_llm_model(mid, h)
        if t < 0:
            break
        got.append(t)
    assert t == -1 and got == want
    stats = json.loads(_take(lib, lib.get_response_statistics_llm_model(mid, h)))
    assert stats.get("prompt_tokens") == len(prompt)

    msgs = [{"role": "user", "content": "hi"}]
    assert _take(lib, lib.apply_chat_template(mid, json.dumps(msgs).encode())) == ref.apply_chat_template(msgs)
    want_text = ref.response("hi", max_length=6, do_sample=False)
    cfg = GenCfg(max_length=6, top_k=1)
    assert _take(lib, lib.response_str_llm_model(mid, b"hi", 1, ctypes.byref(cfg))) == want_text
    h = lib.launch_request_json_llm_model(mid, json.dumps({"messages": msgs, "max_tokens": 6, "temperature": 0}).encode())
    pieces = []
    while True:
        p = lib.fetch_response_str_llm_model(mid, h)
        if not p:
            break
        pieces.append(_take(lib, p))
    assert "".join(pieces) == want_text
    assert lib.set_option_llm_model(mid, b"no_such_option", b"1") == -1
    lib.release_memory(mid)
    ref.release_memory()


def _env():
    env = dict(os.environ)
    env["FASTLLM_PYTHON"] = sys.executable
    return env


def test_native_chat_and_benchmark(built, folder):
    r = subprocess.run([str(BIN / "fastllm_chat"), "-p", folder, "--dtype", "float32", "--device", "cpu", "--max_tokens", "6", "--temperature", "0"],
                       input="hi\nreset\nhi\nstop\n", capture_output=True, text=True, timeout=300, env=_env())
    assert r.returncode == 0, r.stderr[-2000:]
    replies = [l for l in r.stdout.splitlines() if l.startswith("assistant: ")]
    assert len(replies) == 2 and replies[0] == replies[1]       # same conversation after the reset, greedy
    r = subprocess.run([str(BIN / "fastllm_benchmark"), "-p", folder, "--dtype", "float32", "--device", "cpu", "-b", "3", "--prompt_len", "12", "-l", "5"],
                       capture_output=True, text=True, timeout=300, env=_env())
    assert r.returncode == 0, r.stderr[-2000:]
    assert "decode: 12 tokens" in r.stdout and "total: 15 output tokens" in r.stdout, r.stdout


def test_native_apiserver(built, folder):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    proc = subprocess.Popen([str(BIN / "fastllm_apiserver"), "-p", folder, "--dtype", "float32", "--device", "cpu", "--port", str(port),
                             "--api_key", "k", "--model_name", "tiny"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=_env())
    try:
        line = proc.stdout.readline()
        assert "listening" in line, proc.stderr.read()[-2000:]
        base = f"http://127.0.0.1:{port}"

        def call(path, body=None, key="k"):
            req = urllib.request.Request(base + path, data=json.dumps(body).encode() if body is not None else None,
                                         headers={"Authorization": f"Bearer {key}", "Content-Type": "application/json"})
            try:
                with urllib.request.urlopen(req, timeout=120) as r:
                    return r.status, r.read().decode()
            except urllib.error.HTTPError as e:
                return e.code, e.read().decode()

        assert call("/health")[0] == 200
        code, body = call("/v1/models")
        assert code == 200 and json.loads(body)["data"][0]["id"] == "tiny"
        assert call("/v1/models", key="wrong")[0] == 401
        assert call("/v1/nothing")[0] == 404
        assert "<textarea" in call("/")[1]
        req = {"messages": [{"role": "user", "content": "hi \"there\"\n"}], "max_tokens": 6, "temperature": 0}
        code, body = call("/v1/chat/completions", req)
        full = json.loads(body)
        assert code == 200 and full["object"] == "chat.completion" and full["usage"]["completion_tokens"] >= 1
        text = full["choices"][0]["message"]["content"]
        code, sse = call("/v1/chat/completions", dict(req, stream=True))
        events = [e[6:] for e in sse.split("\n\n") if e.startswith("data: ")]
        assert code == 200 and events[-1] == "[DONE]"
        streamed = "".join(json.loads(e)["choices"][0]["delta"].get("content", "") for e in events[:-1])
        assert streamed == text
        code, body = call("/v1/completions", {"prompt": "hello", "max_tokens": 4, "temperature": 0})
        assert code == 200 and json.loads(body)["object"] == "text_completion"
        assert call("/v1/chat/completions", {"messages": "nonsense"})[0] == 400
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()
