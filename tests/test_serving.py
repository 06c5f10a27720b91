"""Serving layer: tool-call parsers (golden strings per family), reasoning split, stream splitter, usage accounting
and routes with a tiny model on CPU (ASGI calls in-process, no sockets)."""
import asyncio
import json

import pytest
import torch

from fastllm_b200.serving import toolcall as tc


def test_hermes_and_reasoning():
    text = '<think>need weather</think>\nSure.<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    r, content = tc.split_reasoning(text)
    assert r == "need weather"
    content, calls = tc.get_parser("hermes").parse(content)
    assert content == "Sure." and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris"}


GOLDEN = [
    ("qwen3_coder", "<tool_call>\n<function=add>\n<parameter=a>\n1\n</parameter>\n<parameter=b>\n2\n</parameter>\n</function>\n</tool_call>", "add", {"a": 1, "b": 2}),
    ("deepseek_v3", "ok<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>f\n```json\n{\"x\": 3}\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>", "f", {"x": 3}),
    ("deepseek_v31", "<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>f<｜tool▁sep｜>{\"x\": 3}<｜tool▁call▁end｜><｜tool▁calls▁end｜>", "f", {"x": 3}),
    ("glm45", "<tool_call>f\n<arg_key>x</arg_key>\n<arg_value>3</arg_value>\n</tool_call>", "f", {"x": 3}),
    ("kimi_k2", "<|tool_calls_section_begin|><|tool_call_begin|>functions.f:0<|tool_call_argument_begin|>{\"x\": 3}<|tool_call_end|><|tool_calls_section_end|>", "f", {"x": 3}),
    ("minimax_m2", '<minimax:tool_call>\n<invoke name="f">\n<parameter name="x">3</parameter>\n</invoke>\n</minimax:tool_call>', "f", {"x": 3}),
    ("json", '{"name": "f", "parameters": {"x": 3}}', "f", {"x": 3}),
]


@pytest.mark.parametrize("parser,text,name,args", GOLDEN)
def test_parser_golden(parser, text, name, args):
    _, calls = tc.get_parser(parser).parse(text)
    assert len(calls) == 1 and calls[0]["function"]["name"] == name
    assert json.loads(calls[0]["function"]["arguments"]) == args


def test_stream_splitter_holds_back_markup():
    sp = tc.StreamSplitter(tc.get_parser("hermes"), reasoning=True)
    pieces = ["<thi", "nk>plan", "</th", "ink>\nHel", "lo <tool", '_call>{"name": "f", "argu', 'ments": {}}</tool_call>']
    out = []
    for p in pieces:
        out += sp.push(p)
    rest, calls = sp.finish()
    assert "".join(t for k, t in out if k == "reasoning") == "plan"
    assert "".join(t for k, t in out if k == "content") == "Hello "
    assert calls and calls[0]["function"]["name"] == "f"


@pytest.fixture(scope="module")
def client(tmp_path_factory):
    fastapi = pytest.importorskip("fastapi")
    httpx = pytest.importorskip("httpx")
    from baseline import synth
    from fastllm_b200 import llm
    from fastllm_b200.serving.server import build_app

    d = synth.write_model("tiny-llama", str(tmp_path_factory.mktemp("srv") / "m"), dtype=torch.float32, std=0.05)
    llm.set_device_map("cpu")
    m = llm.model(d, device="cpu")
    app = build_app(m, "tiny", api_key="k", dev_mode=True)

    def call(method, path, body=None, key="k"):
        async def go():
            tr = httpx.ASGITransport(app=app)
            async with httpx.AsyncClient(transport=tr, base_url="http://t") as c:
                h = {"Authorization": f"Bearer {key}"} if key else {}
                return await (c.post(path, json=body, headers=h) if method == "POST" else c.get(path, headers=h))
        return asyncio.run(go())

    yield call
    m.release_memory()


def test_chat_completion_and_usage(client):
    r = client("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "temperature": 0})
    assert r.status_code == 200
    j = r.json()
    assert j["object"] == "chat.completion" and j["choices"][0]["message"]["role"] == "assistant"
    u = j["usage"]
    assert u["completion_tokens"] <= 5 and u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"]
    assert "cached_tokens" in u["prompt_tokens_details"]


def test_stream_models_auth_metrics(client):
    r = client("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True, "temperature": 0})
    lines = [l for l in r.text.split("\n\n") if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]" and json.loads(lines[0][6:])["choices"][0]["delta"]["role"] == "assistant"
    assert json.loads(lines[-2][6:])["usage"]["completion_tokens"] >= 1
    assert client("GET", "/v1/models").json()["data"][0]["id"] == "tiny"
    assert client("GET", "/v1/models", key="").status_code == 401
    assert "fastllm_requests_total" in client("GET", "/metrics").text
    assert client("GET", "/v1/active_conversations").json()["conversations"] == []


def test_responses_and_anthropic(client):
    r = client("POST", "/v1/responses", {"input": "hello", "max_output_tokens": 4, "temperature": 0})
    assert r.json()["object"] == "response" and r.json()["usage"]["output_tokens"] >= 1
    r = client("POST", "/v1/messages", {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 4, "temperature": 0})
    assert r.json()["type"] == "message" and r.json()["stop_reason"] in ("end_turn", "max_tokens")
    assert client("POST", "/v1/messages", {"messages": []}).status_code == 400


def test_chat_completion_logprobs(client):
    r = client("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0,
                                                "logprobs": True, "top_logprobs": 3})
    j = r.json()
    content = j["choices"][0]["logprobs"]["content"]
    assert 1 <= len(content) <= 4
    for e in content:
        assert e["logprob"] <= 0 and len(e["top_logprobs"]) == 3
        # greedy decoding: the chosen token is the most likely one
        assert abs(e["logprob"] - e["top_logprobs"][0]["logprob"]) < 1e-5


def _sse_events(text):
    out = []
    for block in text.split("\n\n"):
        ev, data = None, None
        for ln in block.split("\n"):
            if ln.startswith("event: "):
                ev = ln[7:]
            elif ln.startswith("data: "):
                data = json.loads(ln[6:])
        if ev is not None:
            out.append((ev, data))
    return out


def test_responses_stream_events(client):
    r = client("POST", "/v1/responses", {"input": "hello", "max_output_tokens": 6, "temperature": 0, "stream": True})
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
    evs = _sse_events(r.text)
    kinds = [k for k, _ in evs]
    assert kinds[0] == "response.created" and kinds[1] == "response.in_progress"
    assert kinds[-1] in ("response.completed", "response.incomplete")
    assert [d["sequence_number"] for _, d in evs] == list(range(len(evs)))
    deltas = "".join(d["delta"] for k, d in evs if k == "response.output_text.delta")
    final = evs[-1][1]["response"]
    assert final["output_text"] == deltas and final["usage"]["output_tokens"] >= 1
    if deltas:
        assert "response.output_item.added" in kinds and "response.output_text.done" in kinds and "response.output_item.done" in kinds
    # same request without streaming gives the same text
    r2 = client("POST", "/v1/responses", {"input": "hello", "max_output_tokens": 6, "temperature": 0})
    assert r2.json()["output_text"] == deltas


def test_anthropic_stream_events(client):
    r = client("POST", "/v1/messages", {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0, "stream": True})
    assert r.status_code == 200
    evs = _sse_events(r.text)
    kinds = [k for k, _ in evs]
    assert kinds[0] == "message_start" and kinds[-1] == "message_stop" and kinds[-2] == "message_delta"
    assert evs[-2][1]["delta"]["stop_reason"] in ("end_turn", "max_tokens") and evs[-2][1]["usage"]["output_tokens"] >= 1
    text = "".join(d["delta"]["text"] for k, d in evs if k == "content_block_delta" and d["delta"]["type"] == "text_delta")
    r2 = client("POST", "/v1/messages", {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0})
    assert "".join(b["text"] for b in r2.json()["content"] if b["type"] == "text") == text
    assert kinds.count("content_block_start") == kinds.count("content_block_stop")


MORE_GOLDEN = [
    ("deepseek_v4", '查一下。\n<｜DSML｜tool_calls><｜DSML｜invoke name="plan_trip"><｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>'
                    '<｜DSML｜parameter name="note" string="true">靠窗</｜DSML｜parameter></｜DSML｜invoke></｜DSML｜tool_calls>',
     "plan_trip", {"days": 3, "note": "靠窗"}, "查一下。\n"),
    ("hy_v3", "<tool_calls><tool_call>f<tool_sep><arg_key>x</arg_key><arg_value>3</arg_value></tool_call></tool_calls>", "f", {"x": 3}, ""),
    ("hy_v3", "<tool_calls:a1><tool_call:a1>f<tool_sep:a1><arg_key:a1>x</arg_key:a1><arg_value:a1>3</arg_value:a1></tool_call:a1></tool_calls:a1>",
     "f", {"x": 3}, ""),
    ("kimi_k3", 'ok <|open|>tools<|sep|><|open|>call tool="f" index="1"<|sep|><|open|>argument key="x" type="json"<|sep|>3<|close|>argument<|sep|>'
                '<|close|>call<|sep|><|close|>tools<|sep|>', "f", {"x": 3}, "ok"),
    ("kimi_k3", '<|open|>call tool="f" index="2"<|sep|><|open|>json<|sep|>{"x": 3}<|close|>json<|sep|><|close|>call<|sep|>', "f", {"x": 3}, ""),
    ("poolside_v1", "<tool_call>f\n<arg_key>x</arg_key><arg_value>3</arg_value></tool_call>", "f", {"x": 3}, ""),
    ("glm47", "<tool_call>f\n<arg_key>x</arg_key>\n<arg_value>3</arg_value>\n</tool_call>", "f", {"x": 3}, ""),
]


@pytest.mark.parametrize("parser,text,name,args,content", MORE_GOLDEN)
def test_more_parser_golden(parser, text, name, args, content):
    got, calls = tc.get_parser(parser).parse(text)
    assert len(calls) == 1 and calls[0]["function"]["name"] == name
    assert json.loads(calls[0]["function"]["arguments"]) == args
    assert (got or "") == content
    # streamed in small pieces: no markup leaks into the content, the call comes out at the end
    sp = tc.StreamSplitter(tc.get_parser(parser), reasoning=False)
    out = []
    for i in range(0, len(text), 5):
        out += sp.push(text[i:i + 5])
    rest, calls2 = sp.finish()
    streamed = "".join(t for _, t in out) + (rest or "")
    assert len(calls2) == 1 and calls2[0]["function"]["name"] == name
    assert "tool_call" not in streamed and "DSML" not in streamed and "<|open|>" not in streamed


class _CharTok:
    """One token per character; decode joins."""

    chars = [chr(c) for c in range(32, 127)] + ["\n"]

    def vocab_size(self):
        return len(self.chars)

    def decode(self, ids, skip_special_tokens=False):
        return "".join(self.chars[i] for i in ids)

    def encode(self, s):
        return [self.chars.index(c) for c in s]


def test_tool_name_constraint_masks_to_declared_names():
    from fastllm_b200.serving.toolcall_constraints import ToolNameConstraint, build_constraint

    tok = _CharTok()
    c = ToolNameConstraint(tok, "hermes", ["get_weather", "get_time", "search"])
    assert c(tok.encode("Let me think. ")) is None                           # outside a name position: unconstrained
    pre = tok.encode('<tool_call>\n{"name": "')
    first = {tok.chars[i] for i in c(pre)}
    assert first == {"g", "s"}
    after = {tok.chars[i] for i in c(pre + tok.encode("get_"))}
    assert after == {"w", "t"}
    done = {tok.chars[i] for i in c(pre + tok.encode("search"))}
    assert done == {'"'}                                                     # a complete name can only be closed
    assert c(pre + tok.encode('search"')) is None                            # closed: unconstrained again
    tools = [{"type": "function", "function": {"name": "add"}}]
    assert build_constraint(tok, "qwen3_coder", tools)(tok.encode("<function=")) == [tok.chars.index("a")]
    assert build_constraint(tok, "json", tools) is None                      # no name position in that format


def test_engine_applies_logits_processor():
    """The sampler masks what the request's processor does not allow, greedy or sampled, on the scheduler rank."""
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.models import preset, random_init

    m = random_init(preset("tiny-llama"), "cpu", torch.float32, std=0.05)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=256), num_pages=16)
    allowed = [5, 9, 11]
    seen = []

    def proc(out_ids):
        seen.append(len(out_ids))
        return allowed if len(out_ids) % 2 == 0 else None

    outs = eng.generate([[1, 2, 3, 4]], GenerationConfig(max_new_tokens=8, ignore_eos=True, logits_processor=proc))[0]
    assert all(t in allowed for t in outs[0::2]) and len(outs) == 8 and seen[:3] == [0, 1, 2]
