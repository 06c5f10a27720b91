"""Shared by the CPU and GPU tests of ``ftllm server --tp N``: start the real server command on a synthetic tiny model,
stream one chat completion over HTTP, stop the server and check that every rank process has gone."""
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_server_and_stream(model_dir: str, extra_args: list[str], timeout_s: float = 300.0):
    port = _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "fastllm_b200.cli", "server", model_dir, "--host", "127.0.0.1", "--port", str(port), *extra_args]
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)
    try:
        t0 = time.time()
        while True:
            if proc.poll() is not None:
                raise AssertionError("server exited early:\n" + proc.stdout.read()[-4000:])
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    if r.status == 200:
                        break
            except OSError:
                pass
            if time.time() - t0 > timeout_s:
                raise AssertionError("server did not come up")
            time.sleep(0.5)
        body = json.dumps({"model": "m", "stream": True, "max_tokens": 12, "temperature": 0,
                           "messages": [{"role": "user", "content": "hello there"}]}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body, headers={"Content-Type": "application/json"})
        chunks, finish = [], None
        with urllib.request.urlopen(req, timeout=120) as r:
            for line in r:
                line = line.decode().strip()
                if not line.startswith("data:"):
                    continue
                data = line[5:].strip()
                if data == "[DONE]":
                    break
                ev = json.loads(data)
                ch = ev["choices"][0]
                if ch.get("delta", {}).get("content"):
                    chunks.append(ch["delta"]["content"])
                finish = ch.get("finish_reason") or finish
        return chunks, finish
    finally:
        try:
            os.killpg(proc.pid, signal.SIGINT)
        except ProcessLookupError:
            pass
        try:
            proc.wait(timeout=60)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
            proc.wait()
