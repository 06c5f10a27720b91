"""Request handling shared by the HTTP routes: prompt building, generation, streaming chunks, usage accounting.

Covers the reference's completion glue (tools/fastllm_pytools/openai_server/fastllm_completion.py:122-3502):
validation, chat-template rendering, SSE streaming, usage with cached-token counts, ``<think>`` splitting,
tool-call parsing (stream + non-stream), stop strings, abort on client disconnect.
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid

from ..tokenizer import StreamDecoder
from .toolcall import StreamSplitter, get_parser, split_reasoning


def _content_text(c):
    if isinstance(c, list):
        return "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type", "text") in ("text", "input_text", "output_text"))
    return c or ""


def normalize_messages(messages):
    out = []
    for m in messages:
        d = dict(m)
        d["content"] = _content_text(d.get("content"))
        out.append(d)
    return out


class PromptIds(list):
    """Token ids of a prompt plus the images and video frame groups its placeholder tokens stand for
    (``launch_stream_response`` picks them up)."""
    images: list = ()
    video_groups: list = ()


class ActiveRequests:
    """Bookkeeping for /v1/cancel and /v1/active_conversations."""

    def __init__(self):
        self.by_id: dict[str, dict] = {}

    def add(self, rid, handle, prompt_tokens):
        self.by_id[rid] = {"handle": handle, "created": time.time(), "prompt_tokens": prompt_tokens, "output_tokens": 0}

    def remove(self, rid):
        self.by_id.pop(rid, None)


class Completion:
    def __init__(self, model, model_name: str = "fastllm-b200", think: bool = True, hide_input: bool = True):
        self.model = model
        self.model_name = model_name
        self.think = think
        self.hide_input = hide_input
        self.active = ActiveRequests()
        self.totals = {"requests": 0, "prompt_tokens": 0, "completion_tokens": 0, "cached_tokens": 0}

    # ---------------------------------------------------------------------------------------------
    def build_prompt_ids(self, messages=None, prompt=None, tools=None, chat_template_kwargs=None):
        if messages is not None:
            images, groups = [], []
            if getattr(getattr(self.model, "torch_model", None), "vision", None) is not None:
                from ..models.vision import extract_images

                videos = []
                messages, images = extract_images(messages, videos)  # image / video parts -> placeholder markup + the media
                if videos:
                    messages, groups = self.model.expand_videos(messages, videos)
            text = self.model.apply_chat_template(normalize_messages(messages), add_generation_prompt=True, tools=tools,
                                                  **(chat_template_kwargs or {}))
            ids = PromptIds(self.model.encode(text))
            ids.images = images
            ids.video_groups = groups
            return ids, text
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            return list(prompt), None
        return self.model.encode(prompt or ""), prompt

    def gen_kwargs(self, req: dict) -> dict:
        temperature = req.get("temperature")
        top_k = req.get("top_k")
        do_sample = not (temperature is not None and temperature <= 1e-6)
        if top_k is None and do_sample and (temperature is not None or req.get("top_p") is not None):
            top_k = 50
        mx = req.get("max_completion_tokens") or req.get("max_tokens") or req.get("max_output_tokens") or 4096
        lp = 0
        if req.get("logprobs"):                 # chat API: logprobs=true (+ top_logprobs=n); completions API: logprobs=n
            lp = int(req.get("top_logprobs") or (req["logprobs"] if isinstance(req["logprobs"], int) and not isinstance(req["logprobs"], bool) else 1))
        return dict(max_length=int(mx), do_sample=do_sample, top_p=req.get("top_p"), top_k=top_k, temperature=temperature,
                    repeat_penalty=req.get("repetition_penalty") or req.get("frequency_penalty_as_repeat"),
                    stop_token_ids=req.get("stop_token_ids"), logprobs=max(0, min(lp, 20)),
                    logits_processor=self.tool_constraint(req))

    def tool_constraint(self, req: dict):
        """Name constraint for requests that declare tools: while the model writes a function name in its tool-call markup only
        continuations of a declared name can be sampled (on by default, ``"tool_call_constraint": false`` in the request or
        ``tool_choice: "none"`` turns it off)."""
        tools = req.get("tools")
        if not tools or req.get("tool_call_constraint") is False or req.get("tool_choice") == "none":
            return None
        from .toolcall_constraints import build_constraint

        try:
            name = get_parser(self.model.tool_call_parser, self.model.get_type()).name
            return build_constraint(self.model.tokenizer, name, tools)
        except Exception:
            return None

    def logprobs_content(self, r) -> list | None:
        """OpenAI ``choices[].logprobs.content`` entries of a finished request (None when logprobs were not requested)."""
        if r is None or not r.gen.logprobs:
            return None
        tok = self.model.tokenizer
        out = []
        for tid, (lp, top) in zip(r.output_ids, r.logprob_entries):
            piece = tok.decode([tid], skip_special_tokens=False)
            out.append({"token": piece, "logprob": lp, "bytes": list(piece.encode("utf-8")),
                        "top_logprobs": [{"token": tok.decode([i], skip_special_tokens=False), "logprob": v} for i, v in top]})
        return out

    async def generate(self, ids, gen_kwargs, stop=None, is_disconnected=None, rid=None, info: dict | None = None):
        """Async generator of (piece, finish_reason or None).  Aborts the engine request when the client goes away."""
        loop = asyncio.get_running_loop()
        m = self.model
        handle = m.launch_stream_response(ids, **gen_kwargs)
        rid = rid or uuid.uuid4().hex
        self.active.add(rid, handle, len(ids))
        req = m.engine.requests.get(handle)
        if info is not None:
            info["request"] = req
        sd = StreamDecoder(m.tokenizer)
        stops = [stop] if isinstance(stop, str) else list(stop or [])
        text = ""
        try:
            while True:
                tok = await loop.run_in_executor(None, m.engine.fetch, handle)
                if tok < 0:
                    break
                self.active.by_id.get(rid, {}).update(output_tokens=len(req.output_ids) if req else 0)
                piece = sd.push(tok)
                if not piece:
                    continue
                text += piece
                hit = next((s for s in stops if s and s in text), None)
                if hit is not None:
                    cut = text.index(hit)
                    keep = piece[:max(0, len(piece) - (len(text) - cut))]
                    if keep:
                        yield keep, None
                    m.abort_handle(handle)
                    yield "", "stop"
                    return
                yield piece, None
                if is_disconnected is not None and await is_disconnected():
                    m.abort_handle(handle)
                    return
            yield "", (req.finish_reason if req is not None and req.finish_reason in ("stop", "length") else "stop")
        except (asyncio.CancelledError, GeneratorExit):
            m.abort_handle(handle)
            raise
        finally:
            st = req.stats.as_dict() if req is not None else {}
            self.last_usage = {"prompt_tokens": len(ids), "completion_tokens": st.get("output_tokens", 0),
                               "total_tokens": len(ids) + st.get("output_tokens", 0),
                               "prompt_tokens_details": {"cached_tokens": st.get("cached_tokens", 0)}}
            self.totals["requests"] += 1
            self.totals["prompt_tokens"] += len(ids)
            self.totals["completion_tokens"] += st.get("output_tokens", 0)
            self.totals["cached_tokens"] += st.get("cached_tokens", 0)
            self.active.remove(rid)

    # ---------------------------------------------------------------------------------------------
    async def chat_completion(self, req: dict, is_disconnected=None):
        """Non-streaming: returns the response dict.  Streaming: returns an async generator of SSE ``data:`` lines."""
        tools = req.get("tools")
        ids, _ = self.build_prompt_ids(messages=req["messages"], tools=tools, chat_template_kwargs=req.get("chat_template_kwargs"))
        parser = get_parser(self.model.tool_call_parser, self.model.get_type()) if tools else None
        cid = "chatcmpl-" + uuid.uuid4().hex
        created = int(time.time())
        gk = self.gen_kwargs(req)
        if not req.get("stream"):
            text, finish = "", "stop"
            info: dict = {}
            async for piece, fin in self.generate(ids, gk, req.get("stop"), is_disconnected, cid, info):
                text += piece
                finish = fin or finish
            reasoning, content = split_reasoning(text) if self.think else (None, text)
            calls = []
            if parser is not None:
                content, calls = parser.parse(content)
            msg = {"role": "assistant", "content": content if (content or not calls) else None}
            if reasoning:
                msg["reasoning_content"] = reasoning
            if calls:
                msg["tool_calls"] = calls
                finish = "tool_calls"
            choice = {"index": 0, "message": msg, "finish_reason": finish}
            lpc = self.logprobs_content(info.get("request")) if gk.get("logprobs") else None
            if lpc is not None:
                choice["logprobs"] = {"content": lpc}
            return {"id": cid, "object": "chat.completion", "created": created, "model": req.get("model") or self.model_name,
                    "choices": [choice], "usage": self.last_usage}

        async def sse():
            def chunk(delta, finish=None, usage=None):
                d = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": req.get("model") or self.model_name,
                     "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
                if usage is not None:
                    d["usage"] = usage
                return "data: " + json.dumps(d, ensure_ascii=False) + "\n\n"

            yield chunk({"role": "assistant", "content": ""})
            sp = StreamSplitter(parser, reasoning=self.think)
            finish = "stop"
            async for piece, fin in self.generate(ids, gk, req.get("stop"), is_disconnected, cid):
                finish = fin or finish
                for kind, txt in sp.push(piece) if piece else []:
                    yield chunk({"reasoning_content": txt} if kind == "reasoning" else {"content": txt})
            rest, calls = sp.finish()
            if rest:
                yield chunk({"content": rest})
            for i, c in enumerate(calls):
                yield chunk({"tool_calls": [dict(c, index=i)]})
            include_usage = (req.get("stream_options") or {}).get("include_usage", True)
            yield chunk({}, "tool_calls" if calls else finish, self.last_usage if include_usage else None)
            yield "data: [DONE]\n\n"

        return sse()

    async def _events(self, req: dict, is_disconnected=None, rid=None):
        """Protocol-neutral stream of one chat request: ``("reasoning" | "content", text)`` pieces as they are decoded,
        ``("tool_call", call)`` for every parsed call, and a final ``("finish", reason)``.  The three streaming protocols
        (chat-completions chunks, Responses events, Anthropic events) are renderings of this stream."""
        tools = req.get("tools")
        ids, _ = self.build_prompt_ids(messages=req["messages"], tools=tools, chat_template_kwargs=req.get("chat_template_kwargs"))
        parser = get_parser(self.model.tool_call_parser, self.model.get_type()) if tools else None
        sp = StreamSplitter(parser, reasoning=self.think)
        finish = "stop"
        async for piece, fin in self.generate(ids, self.gen_kwargs(req), req.get("stop"), is_disconnected, rid):
            finish = fin or finish
            for kind, txt in sp.push(piece) if piece else []:
                yield kind, txt
        rest, calls = sp.finish()
        if rest:
            yield "content", rest
        for c in calls:
            yield "tool_call", c
        yield "finish", ("tool_calls" if calls else finish)

    async def text_completion(self, req: dict, is_disconnected=None):
        ids, _ = self.build_prompt_ids(prompt=req.get("prompt", ""))
        text, finish = "", "stop"
        async for piece, fin in self.generate(ids, self.gen_kwargs(req), req.get("stop"), is_disconnected):
            text += piece
            finish = fin or finish
        return {"id": "cmpl-" + uuid.uuid4().hex, "object": "text_completion", "created": int(time.time()),
                "model": req.get("model") or self.model_name,
                "choices": [{"index": 0, "text": text, "finish_reason": finish}], "usage": self.last_usage}

    # ---- OpenAI Responses API ---------------------------------------------------------------------
    async def responses(self, req: dict, is_disconnected=None):
        inp = req.get("input", "")
        msgs = []
        if req.get("instructions"):
            msgs.append({"role": "system", "content": req["instructions"]})
        if isinstance(inp, str):
            msgs.append({"role": "user", "content": inp})
        else:
            for it in inp:
                if it.get("type", "message") == "message":
                    msgs.append({"role": it.get("role", "user"), "content": _content_text(it.get("content"))})
        for t in req.get("tools") or []:          # Responses tools are flat; the chat template wants the nested form
            if t.get("type") == "function" and "function" not in t:
                t["function"] = {"name": t.get("name"), "description": t.get("description", ""), "parameters": t.get("parameters", {})}
        creq = dict(req, messages=msgs, stream=False, max_tokens=req.get("max_output_tokens"))
        if req.get("stream"):
            return self._responses_stream(creq, is_disconnected)
        r = await self.chat_completion(creq, is_disconnected)
        msg = r["choices"][0]["message"]
        output = []
        if msg.get("reasoning_content"):
            output.append({"type": "reasoning", "id": "rs_" + uuid.uuid4().hex[:16], "summary": [{"type": "summary_text", "text": msg["reasoning_content"]}]})
        if msg.get("content"):
            output.append({"type": "message", "id": "msg_" + uuid.uuid4().hex[:16], "role": "assistant", "status": "completed",
                           "content": [{"type": "output_text", "text": msg["content"], "annotations": []}]})
        for c in msg.get("tool_calls", []):
            output.append({"type": "function_call", "id": "fc_" + uuid.uuid4().hex[:16], "call_id": c["id"], "name": c["function"]["name"],
                           "arguments": c["function"]["arguments"], "status": "completed"})
        u = r["usage"]
        return {"id": "resp_" + uuid.uuid4().hex, "object": "response", "created_at": r["created"], "status": "completed", "model": r["model"],
                "output": output, "output_text": msg.get("content") or "",
                "usage": {"input_tokens": u["prompt_tokens"], "output_tokens": u["completion_tokens"], "total_tokens": u["total_tokens"],
                          "input_tokens_details": {"cached_tokens": u["prompt_tokens_details"]["cached_tokens"]}}}

    async def _responses_stream(self, creq: dict, is_disconnected=None):
        """Server-sent events of the Responses protocol (reference: tools/fastllm_pytools/server.py:152-168 streams
        ``/v1/responses``): response.created / in_progress, then per output item ``output_item.added`` ->
        deltas -> ``*.done`` -> ``output_item.done``, and ``response.completed`` with the whole response and usage."""
        rid = "resp_" + uuid.uuid4().hex
        created = int(time.time())
        model_name = creq.get("model") or self.model_name
        seq = 0

        def ev(kind, **body):
            nonlocal seq
            d = dict(type=kind, sequence_number=seq, **body)
            seq += 1
            return f"event: {kind}\ndata: " + json.dumps(d, ensure_ascii=False) + "\n\n"

        def shell(status, output=None, usage=None):
            return {"id": rid, "object": "response", "created_at": created, "status": status, "model": model_name,
                    "output": output or [], "usage": usage}

        yield ev("response.created", response=shell("in_progress"))
        yield ev("response.in_progress", response=shell("in_progress"))
        output = []
        cur = None          # the open item: {"kind", "item", "text"}

        def close_item():
            nonlocal cur
            out = []
            if cur is None:
                return out
            idx = len(output)
            it = cur["item"]
            if cur["kind"] == "content":
                part = {"type": "output_text", "text": cur["text"], "annotations": []}
                it["content"] = [part]
                it["status"] = "completed"
                out.append(ev("response.output_text.done", item_id=it["id"], output_index=idx, content_index=0, text=cur["text"]))
                out.append(ev("response.content_part.done", item_id=it["id"], output_index=idx, content_index=0, part=part))
            else:
                it["summary"] = [{"type": "summary_text", "text": cur["text"]}]
                out.append(ev("response.reasoning_summary_text.done", item_id=it["id"], output_index=idx, summary_index=0, text=cur["text"]))
            out.append(ev("response.output_item.done", output_index=idx, item=it))
            output.append(it)
            cur = None
            return out

        finish = "stop"
        async for kind, val in self._events(creq, is_disconnected, rid):
            if kind in ("content", "reasoning"):
                if cur is None or cur["kind"] != kind:
                    for line in close_item():
                        yield line
                    idx = len(output)
                    if kind == "content":
                        item = {"type": "message", "id": "msg_" + uuid.uuid4().hex[:16], "role": "assistant", "status": "in_progress", "content": []}
                        yield ev("response.output_item.added", output_index=idx, item=item)
                        yield ev("response.content_part.added", item_id=item["id"], output_index=idx, content_index=0,
                                 part={"type": "output_text", "text": "", "annotations": []})
                    else:
                        item = {"type": "reasoning", "id": "rs_" + uuid.uuid4().hex[:16], "summary": []}
                        yield ev("response.output_item.added", output_index=idx, item=item)
                    cur = {"kind": kind, "item": item, "text": ""}
                cur["text"] += val
                if kind == "content":
                    yield ev("response.output_text.delta", item_id=cur["item"]["id"], output_index=len(output), content_index=0, delta=val)
                else:
                    yield ev("response.reasoning_summary_text.delta", item_id=cur["item"]["id"], output_index=len(output), summary_index=0, delta=val)
            elif kind == "tool_call":
                for line in close_item():
                    yield line
                idx = len(output)
                item = {"type": "function_call", "id": "fc_" + uuid.uuid4().hex[:16], "call_id": val["id"], "name": val["function"]["name"],
                        "arguments": "", "status": "in_progress"}
                yield ev("response.output_item.added", output_index=idx, item=item)
                args = val["function"]["arguments"] or ""
                yield ev("response.function_call_arguments.delta", item_id=item["id"], output_index=idx, delta=args)
                yield ev("response.function_call_arguments.done", item_id=item["id"], output_index=idx, arguments=args)
                item = dict(item, arguments=args, status="completed")
                yield ev("response.output_item.done", output_index=idx, item=item)
                output.append(item)
            else:
                finish = val
        for line in close_item():
            yield line
        u = self.last_usage
        usage = {"input_tokens": u["prompt_tokens"], "output_tokens": u["completion_tokens"], "total_tokens": u["total_tokens"],
                 "input_tokens_details": {"cached_tokens": u["prompt_tokens_details"]["cached_tokens"]}}
        final = shell("incomplete" if finish == "length" else "completed", output, usage)
        final["output_text"] = "".join(p["text"] for it in output if it["type"] == "message" for p in it["content"])
        if finish == "length":
            final["incomplete_details"] = {"reason": "max_output_tokens"}
        yield ev("response.incomplete" if finish == "length" else "response.completed", response=final)

    async def _anthropic_stream(self, creq: dict, is_disconnected=None):
        """Server-sent events of the Anthropic Messages protocol (reference: tools/fastllm_pytools/server.py:169-180):
        message_start, then per content block start / deltas / stop, message_delta with the stop reason and output
        token count, message_stop."""
        mid = "msg_" + uuid.uuid4().hex[:24]
        model_name = creq.get("model") or self.model_name

        def ev(kind, **body):
            return f"event: {kind}\ndata: " + json.dumps(dict(type=kind, **body), ensure_ascii=False) + "\n\n"

        yield ev("message_start", message={"id": mid, "type": "message", "role": "assistant", "model": model_name, "content": [],
                                           "stop_reason": None, "stop_sequence": None, "usage": {"input_tokens": 0, "output_tokens": 0}})
        yield ev("ping")
        index = -1
        open_kind = None
        finish = "stop"
        async for kind, val in self._events(creq, is_disconnected, mid):
            if kind in ("content", "reasoning"):
                if open_kind != kind:
                    if open_kind is not None:
                        yield ev("content_block_stop", index=index)
                    index += 1
                    open_kind = kind
                    block = {"type": "text", "text": ""} if kind == "content" else {"type": "thinking", "thinking": ""}
                    yield ev("content_block_start", index=index, content_block=block)
                delta = {"type": "text_delta", "text": val} if kind == "content" else {"type": "thinking_delta", "thinking": val}
                yield ev("content_block_delta", index=index, delta=delta)
            elif kind == "tool_call":
                if open_kind is not None:
                    yield ev("content_block_stop", index=index)
                    open_kind = None
                index += 1
                yield ev("content_block_start", index=index, content_block={"type": "tool_use", "id": val["id"].replace("call_", "toolu_"),
                                                                            "name": val["function"]["name"], "input": {}})
                yield ev("content_block_delta", index=index, delta={"type": "input_json_delta", "partial_json": val["function"]["arguments"] or "{}"})
                yield ev("content_block_stop", index=index)
            else:
                finish = val
        if open_kind is not None:
            yield ev("content_block_stop", index=index)
        u = self.last_usage
        yield ev("message_delta", delta={"stop_reason": {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use"}.get(finish, "end_turn"),
                                         "stop_sequence": None},
                 usage={"input_tokens": u["prompt_tokens"], "output_tokens": u["completion_tokens"],
                        "cache_read_input_tokens": u["prompt_tokens_details"]["cached_tokens"]})
        yield ev("message_stop")

    # ---- Anthropic Messages API -------------------------------------------------------------------
    async def anthropic_messages(self, req: dict, is_disconnected=None):
        msgs = []
        sysm = req.get("system")
        if sysm:
            msgs.append({"role": "system", "content": _content_text(sysm) if not isinstance(sysm, str) else sysm})
        for m in req.get("messages", []):
            msgs.append({"role": m["role"], "content": _content_text(m.get("content"))})
        tools = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""), "parameters": t.get("input_schema", {})}}
                 for t in req.get("tools") or []] or None
        creq = dict(req, messages=msgs, stream=False, tools=tools, stop=req.get("stop_sequences"))
        if req.get("stream"):
            return self._anthropic_stream(creq, is_disconnected)
        r = await self.chat_completion(creq, is_disconnected)
        msg = r["choices"][0]["message"]
        content = []
        if msg.get("reasoning_content"):
            content.append({"type": "thinking", "thinking": msg["reasoning_content"]})
        if msg.get("content"):
            content.append({"type": "text", "text": msg["content"]})
        for c in msg.get("tool_calls", []):
            content.append({"type": "tool_use", "id": c["id"].replace("call_", "toolu_"), "name": c["function"]["name"],
                            "input": json.loads(c["function"]["arguments"] or "{}")})
        fin = r["choices"][0]["finish_reason"]
        u = r["usage"]
        return {"id": "msg_" + uuid.uuid4().hex[:24], "type": "message", "role": "assistant", "model": r["model"], "content": content,
                "stop_reason": {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use"}.get(fin, "end_turn"), "stop_sequence": None,
                "usage": {"input_tokens": u["prompt_tokens"], "output_tokens": u["completion_tokens"],
                          "cache_read_input_tokens": u["prompt_tokens_details"]["cached_tokens"]}}
