"""OpenAI-style API server (FastAPI).

Routes of the reference server (tools/fastllm_pytools/server.py:136-246): ``/v1/chat/completions``,
``/v1/responses`` (+ alias ``/v1/response``), ``/v1/messages`` (Anthropic), ``/v1/embed``, ``/v1/rerank``,
``/v1/models``, ``/v1/cancel``, ``/v1/active_conversations`` (dev mode), API-key middleware.  Added here:
``/v1/completions`` and a Prometheus ``/metrics`` endpoint.
"""
import argparse
import json
import time

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse


def build_app(model, model_name: str = "fastllm-b200", api_key: str = "", dev_mode: bool = False, think: bool = True):
    from .completion import Completion

    app = FastAPI(title="fastllm_b200 API server")
    comp = Completion(model, model_name, think=think)
    app.state.completion = comp
    started = time.time()

    @app.middleware("http")
    async def auth(request: Request, call_next):
        if api_key and request.url.path.startswith("/v1"):
            got = request.headers.get("authorization", "")
            xk = request.headers.get("x-api-key", "")
            if got != f"Bearer {api_key}" and xk != api_key:
                return JSONResponse({"error": {"message": "invalid API key", "type": "invalid_request_error"}}, status_code=401)
        return await call_next(request)

    def _bad(msg, code=400):
        return JSONResponse({"error": {"message": msg, "type": "invalid_request_error"}}, status_code=code)

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        req = await request.json()
        if not isinstance(req.get("messages"), list) or not req["messages"]:
            return _bad("'messages' must be a non-empty list")
        try:
            r = await comp.chat_completion(req, request.is_disconnected)
        except Exception as e:  # template / tokenizer / engine errors become a 4xx/5xx JSON, never a hung stream
            return _bad(f"{type(e).__name__}: {e}", 500)
        if req.get("stream"):
            return StreamingResponse(r, media_type="text/event-stream")
        return JSONResponse(r)

    @app.post("/v1/completions")
    async def completions(request: Request):
        return JSONResponse(await comp.text_completion(await request.json(), request.is_disconnected))

    @app.post("/v1/responses")
    @app.post("/v1/response")
    async def responses(request: Request):
        req = await request.json()
        try:
            r = await comp.responses(req, request.is_disconnected)
        except Exception as e:
            return _bad(f"{type(e).__name__}: {e}", 500)
        if req.get("stream"):
            return StreamingResponse(r, media_type="text/event-stream")
        return JSONResponse(r)

    @app.post("/v1/messages")
    async def messages(request: Request):
        req = await request.json()
        if "max_tokens" not in req:
            return _bad("'max_tokens' is required")
        try:
            r = await comp.anthropic_messages(req, request.is_disconnected)
        except Exception as e:
            return _bad(f"{type(e).__name__}: {e}", 500)
        if req.get("stream"):
            return StreamingResponse(r, media_type="text/event-stream")
        return JSONResponse(r)

    @app.post("/v1/embed")
    @app.post("/v1/embeddings")
    async def embed(request: Request):
        req = await request.json()
        inputs = req.get("inputs", req.get("input", []))
        inputs = [inputs] if isinstance(inputs, str) else inputs
        from ..models.embedding import embed_texts

        vecs = embed_texts(model, inputs, normalize=req.get("normalize", True))
        return JSONResponse({"object": "list", "model": model_name,
                             "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)]})

    @app.post("/v1/rerank")
    async def rerank(request: Request):
        req = await request.json()
        from ..models.embedding import rerank_scores

        scores = rerank_scores(model, req.get("query", ""), req.get("texts", req.get("documents", [])))
        order = sorted(range(len(scores)), key=lambda i: -scores[i])
        return JSONResponse({"results": [{"index": i, "relevance_score": scores[i]} for i in order]})

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "created": int(started), "owned_by": "fastllm_b200"}]}

    @app.post("/v1/cancel")
    async def cancel(request: Request):
        req = await request.json()
        rid = req.get("conversation_id") or req.get("id") or ""
        ent = comp.active.by_id.get(rid)
        if ent is None:
            return _bad("unknown conversation id", 404)
        model.abort_handle(ent["handle"])
        return {"status": "cancelled", "id": rid}

    @app.get("/v1/active_conversations")
    async def active():
        if not dev_mode:
            return _bad("dev mode is off", 403)
        return {"conversations": [dict(v, id=k) for k, v in comp.active.by_id.items()]}

    @app.get("/health")
    async def health():
        return {"status": "ok", "uptime_s": time.time() - started}

    @app.get("/metrics")
    async def metrics():
        t = comp.totals
        eng = model.engine
        pm = eng.pm.stats()
        lines = [
            "# TYPE fastllm_requests_total counter", f"fastllm_requests_total {t['requests']}",
            "# TYPE fastllm_prompt_tokens_total counter", f"fastllm_prompt_tokens_total {t['prompt_tokens']}",
            "# TYPE fastllm_completion_tokens_total counter", f"fastllm_completion_tokens_total {t['completion_tokens']}",
            "# TYPE fastllm_cached_prompt_tokens_total counter", f"fastllm_cached_prompt_tokens_total {t['cached_tokens']}",
            "# TYPE fastllm_running_requests gauge", f"fastllm_running_requests {len(eng.running)}",
            "# TYPE fastllm_waiting_requests gauge", f"fastllm_waiting_requests {len(eng.waiting)}",
            "# TYPE fastllm_kv_pages_free gauge", f"fastllm_kv_pages_free {pm['free']}",
            "# TYPE fastllm_kv_pages_cached gauge", f"fastllm_kv_pages_cached {pm['cached']}",
            "# TYPE fastllm_decode_steps_total counter", f"fastllm_decode_steps_total {eng.decode_steps}",
        ]
        return PlainTextResponse("\n".join(lines) + "\n")

    return app


def add_server_args(p: argparse.ArgumentParser):
    p.add_argument("--model_name", type=str, default="")
    p.add_argument("--host", type=str, default="0.0.0.0")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--api_key", type=str, default="")
    p.add_argument("--think", type=str, default="true")
    p.add_argument("--hide_input", action="store_true")
    p.add_argument("--dev_mode", action="store_true")
    p.add_argument("--startup-progress", dest="startup_progress", choices=["off", "ndjson"], default="off",
                   help="ndjson: FTLLM_PROGRESS events on stderr while the model loads")


def serve(args):
    import uvicorn

    from ..util import make_normal_llm_model
    from .progress import emit

    if getattr(args, "startup_progress", "off") == "ndjson":
        import os

        os.environ["FTLLM_PROGRESS"] = "1"
    emit("load", 0, 1)
    model = make_normal_llm_model(args)
    emit("load", 1, 1)
    model.warmup()
    emit("ready", 1, 1)
    name = args.model_name or (args.path.rstrip("/").split("/")[-1] if getattr(args, "path", "") else "fastllm-b200")
    app = build_app(model, name, args.api_key, args.dev_mode, str(args.think).lower() != "false")
    uvicorn.run(app, host=args.host, port=args.port, log_level="warning")
