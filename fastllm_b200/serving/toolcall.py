"""Tool-call and reasoning extraction from model output (stream and non-stream).

The reference carries one parser per model family (tools/fastllm_pytools/openai_server/tool_parsers/*, selected
in toolcall_parser.py; enabled set: hermes, qwen3_coder, deepseek_v3/v31, glm45/47, kimi_k2, minimax_m2, ...).
The formats below are the wire formats those families emit; each parser turns text into OpenAI ``tool_calls``
entries ``{"id", "type": "function", "function": {"name", "arguments": json-string}}`` plus the remaining content.
"""
from __future__ import annotations

import json
import re
import uuid


def _call(name: str, arguments) -> dict:
    if not isinstance(arguments, str):
        arguments = json.dumps(arguments, ensure_ascii=False)
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function", "function": {"name": name, "arguments": arguments}}


def _loads_lenient(s: str):
    try:
        return json.loads(s)
    except Exception:
        try:
            return json.loads(s.strip().rstrip(",").replace("'", '"'))
        except Exception:
            return None


class ToolParser:
    name = "base"
    start_markers: tuple = ()

    def parse(self, text: str):
        """-> (content without the tool-call markup, list of tool calls)"""
        return text, []

    def may_start(self, text: str) -> bool:
        """True if ``text`` ends in something that could be the beginning of tool-call markup (hold it back)."""
        for m in self.start_markers:
            for k in range(1, len(m) + 1):
                if text.endswith(m[:k]):
                    return True
            if m in text:
                return True
        return False


class HermesParser(ToolParser):
    """``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` (Qwen2.5/Qwen3, Hermes)."""
    name = "hermes"
    start_markers = ("<tool_call>",)
    _re = re.compile(r"<tool_call>\s*(.*?)\s*(?:</tool_call>|$)", re.S)

    def parse(self, text):
        calls = []
        for m in self._re.finditer(text):
            obj = _loads_lenient(m.group(1))
            if isinstance(obj, dict) and "name" in obj:
                calls.append(_call(obj["name"], obj.get("arguments", obj.get("parameters", {}))))
        content = self._re.sub("", text).strip() if calls else text
        return content, calls


class Qwen3CoderParser(ToolParser):
    """``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``"""
    name = "qwen3_coder"
    start_markers = ("<tool_call>", "<function=")
    _fn = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|$)", re.S)
    _par = re.compile(r"<parameter=([^>\s]+)>(.*?)(?:</parameter>|(?=<parameter=)|$)", re.S)

    def parse(self, text):
        calls = []
        for m in self._fn.finditer(text):
            args = {}
            for p in self._par.finditer(m.group(2)):
                v = p.group(2).strip("\n")
                j = _loads_lenient(v)
                args[p.group(1)] = j if (j is not None and not isinstance(j, str)) else v
            calls.append(_call(m.group(1), args))
        if not calls:
            return text, []
        content = re.sub(r"<tool_call>.*?(?:</tool_call>|$)", "", text, flags=re.S)
        content = self._fn.sub("", content).strip()
        return content, calls


class DeepSeekV3Parser(ToolParser):
    """``<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>NAME\\n```json\\n{...}\\n```<｜tool▁call▁end｜>...``"""
    name = "deepseek_v3"
    start_markers = ("<｜tool▁calls▁begin｜>",)
    _re = re.compile(r"<｜tool▁call▁begin｜>(?:function)?<｜tool▁sep｜>([^\n<]+)\n?(?:```json\n)?(.*?)(?:\n```)?<｜tool▁call▁end｜>", re.S)

    def parse(self, text):
        calls = [_call(m.group(1).strip(), _loads_lenient(m.group(2)) or m.group(2).strip()) for m in self._re.finditer(text)]
        if not calls:
            return text, []
        return text.split("<｜tool▁calls▁begin｜>")[0].strip(), calls


class DeepSeekV31Parser(DeepSeekV3Parser):
    """V3.1 drops the code fence: ``<｜tool▁call▁begin｜>NAME<｜tool▁sep｜>{json}<｜tool▁call▁end｜>``"""
    name = "deepseek_v31"
    _re = re.compile(r"<｜tool▁call▁begin｜>([^<]+?)<｜tool▁sep｜>(.*?)<｜tool▁call▁end｜>", re.S)


class Glm45Parser(ToolParser):
    """``<tool_call>NAME\\n<arg_key>K</arg_key>\\n<arg_value>V</arg_value>...</tool_call>``"""
    name = "glm45"
    start_markers = ("<tool_call>",)
    _re = re.compile(r"<tool_call>\s*([^\n<]+)\s*(.*?)</tool_call>", re.S)
    _kv = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)

    def parse(self, text):
        calls = []
        for m in self._re.finditer(text):
            args = {}
            for k, v in self._kv.findall(m.group(2)):
                j = _loads_lenient(v)
                args[k.strip()] = j if (j is not None and not isinstance(j, str)) else v
            calls.append(_call(m.group(1).strip(), args))
        return (self._re.sub("", text).strip(), calls) if calls else (text, [])


class KimiK2Parser(ToolParser):
    """``<|tool_calls_section_begin|><|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{json}<|tool_call_end|>``"""
    name = "kimi_k2"
    start_markers = ("<|tool_calls_section_begin|>", "<|tool_call_begin|>")
    _re = re.compile(r"<\|tool_call_begin\|>\s*(?:functions\.)?([\w\-\.]+?)(?::\d+)?\s*<\|tool_call_argument_begin\|>(.*?)<\|tool_call_end\|>", re.S)

    def parse(self, text):
        calls = [_call(m.group(1), _loads_lenient(m.group(2)) or m.group(2).strip()) for m in self._re.finditer(text)]
        if not calls:
            return text, []
        return re.split(r"<\|tool_calls_section_begin\|>|<\|tool_call_begin\|>", text)[0].strip(), calls


class MinimaxM2Parser(ToolParser):
    """``<minimax:tool_call><invoke name="NAME"><parameter name="K">V</parameter></invoke></minimax:tool_call>``"""
    name = "minimax_m2"
    start_markers = ("<minimax:tool_call>",)
    _inv = re.compile(r'<invoke name="([^"]+)">(.*?)</invoke>', re.S)
    _par = re.compile(r'<parameter name="([^"]+)">(.*?)</parameter>', re.S)

    def parse(self, text):
        calls = []
        for m in self._inv.finditer(text):
            args = {}
            for k, v in self._par.findall(m.group(2)):
                j = _loads_lenient(v)
                args[k] = j if (j is not None and not isinstance(j, str)) else v.strip()
            calls.append(_call(m.group(1), args))
        return (text.split("<minimax:tool_call>")[0].strip(), calls) if calls else (text, [])


def _typed(v: str):
    j = _loads_lenient(v)
    return j if (j is not None and not isinstance(j, str)) else v


class DeepSeekV4Parser(ToolParser):
    """DSML: ``<｜DSML｜tool_calls><｜DSML｜invoke name="NAME"><｜DSML｜parameter name="K" string="true|false">V</｜DSML｜parameter>
    ...</｜DSML｜invoke></｜DSML｜tool_calls>``; ``string="false"`` values are JSON.  The tag prefix also appears spelled ``\\DSML\\``.
    (reference: openai_server/tool_parsers/deepseekv4_tool_parser.py:58-80)"""
    name = "deepseek_v4"
    start_markers = ("<｜DSML｜tool_calls>", "<\\DSML\\tool_calls>")
    _T = r"(?:｜DSML｜|\\DSML\\)"
    _block = re.compile(r"<" + _T + r"tool_calls>(.*?)(?:</" + _T + r"tool_calls>|$)", re.S)
    _inv = re.compile(r'<' + _T + r'invoke\s+name="([^"]+)"\s*>(.*?)</' + _T + r'invoke>', re.S)
    _par = re.compile(r'<' + _T + r'parameter\s+name="([^"]+)"\s+string="(true|false)"\s*>(.*?)</' + _T + r'parameter>', re.S)

    def parse(self, text):
        calls = []
        for b in self._block.finditer(text):
            for m in self._inv.finditer(b.group(1)):
                args = {}
                for k, is_str, v in self._par.findall(m.group(2)):
                    if is_str == "true":
                        args[k] = v
                    else:
                        j = _loads_lenient(v)
                        args[k] = v if j is None else j
                calls.append(_call(m.group(1), args))
        if not calls:
            return text, []
        content = self._block.sub("", text)
        return (content if content.strip() else ""), calls


class HYV3Parser(ToolParser):
    """Hunyuan V3: ``<tool_calls><tool_call>NAME<tool_sep><arg_key>K</arg_key><arg_value>V</arg_value>...</tool_call></tool_calls>``;
    the special tokens may carry a ``:suffix`` inside the angle brackets (``<tool_call:x>``), which is accepted on every tag.
    (reference: openai_server/tool_parsers/hy_v3_tool_parser.py:61-110, 140-160)"""
    name = "hy_v3"
    start_markers = ("<tool_calls", "<tool_call")
    _sfx = r"(?::[^>]*)?"
    _call_re = re.compile(r"<tool_call" + _sfx + r">(.*?)<tool_sep" + _sfx + r">(.*?)(?:</tool_call" + _sfx + r">|$)", re.S)
    _kv = re.compile(r"<arg_key" + _sfx + r">(.*?)</arg_key" + _sfx + r">\s*<arg_value" + _sfx + r">(.*?)</arg_value" + _sfx + r">", re.S)
    _strip = re.compile(r"<tool_calls" + _sfx + r">.*?(?:</tool_calls" + _sfx + r">|$)|<tool_call" + _sfx + r">.*?(?:</tool_call" + _sfx + r">|$)", re.S)

    def parse(self, text):
        calls = []
        for m in self._call_re.finditer(text):
            args = {k.strip(): _typed(v) for k, v in self._kv.findall(m.group(2))}
            calls.append(_call(m.group(1).strip(), args))
        return (self._strip.sub("", text).strip(), calls) if calls else (text, [])


class KimiK3Parser(ToolParser):
    """Kimi K3 XTML: ``<|open|>tools<|sep|><|open|>call tool="NAME" index="1"<|sep|><|open|>argument key="K" type="string|json"<|sep|>V
    <|close|>argument<|sep|>...<|close|>call<|sep|><|close|>tools<|sep|>``; attribute values escape ``"`` and ``&`` as entities; a call
    may carry one ``<|open|>json<|sep|>{...}<|close|>json<|sep|>`` block instead of arguments.  Call ids are ``NAME:index-1``.
    (reference: openai_server/tool_parsers/kimi_k3_tool_parser.py:63-200)"""
    name = "kimi_k3"
    start_markers = ("<|open|>tools", "<|open|>call")
    _O, _C, _S = r"<\|open\|>", r"<\|close\|>", r"<\|sep\|>"
    _UNTIL = r"(?:(?!" + _S + r").)*?"
    _call_re = re.compile(_O + r"\s*call\s+(?P<attrs>" + _UNTIL + r")" + _S + r"(?P<body>.*?)" + _C + r"\s*call\s*" + _S, re.S)
    _arg_re = re.compile(_O + r"\s*argument\s+(?P<attrs>" + _UNTIL + r")" + _S + r"(?P<value>.*?)" + _C + r"\s*argument\s*" + _S, re.S)
    _json_re = re.compile(_O + r"\s*json(?:\s+" + _UNTIL + r")?" + _S + r"(?P<value>.*?)" + _C + r"\s*json\s*" + _S, re.S)
    _attr_re = re.compile(r'(?P<key>\w+)="(?P<value>[^"]*)"')
    _head_re = re.compile(_O + r"\s*(?:tools\s*" + _S + r"|call[\s<])")

    def _attrs(self, t):
        return {m["key"]: m["value"].replace("&quot;", '"').replace("&amp;", "&") for m in self._attr_re.finditer(t)}

    def parse(self, text):
        calls = []
        for m in self._call_re.finditer(text):
            a = self._attrs(m["attrs"])
            if not a.get("tool"):
                continue
            args = {}
            for am in self._arg_re.finditer(m["body"]):
                aa = self._attrs(am["attrs"])
                v = am["value"]
                if aa.get("type", "string") != "string":
                    j = _loads_lenient(v)
                    v = v if j is None else j
                args[aa.get("key", "")] = v
            if not args:
                jm = self._json_re.search(m["body"])
                j = _loads_lenient(jm["value"]) if jm else None
                if isinstance(j, dict):
                    args = j
            c = _call(a["tool"], args)
            if a.get("index", "").isdigit():
                c["id"] = f"{a['tool']}:{int(a['index']) - 1}"
            calls.append(c)
        if not calls:
            return text, []
        hm = self._head_re.search(text)
        return (text[:hm.start()].strip() if hm else ""), calls


class PoolsideV1Parser(Glm45Parser):
    """Poolside: the GLM-4.5 key/value form, ``<tool_call>NAME\\n<arg_key>K</arg_key><arg_value>V</arg_value>...</tool_call>``; a call
    without arguments is ``<tool_call>NAME</tool_call>``; keys never contain ``<``.
    (reference: openai_server/tool_parsers/poolside_v1_tool_parser.py:50-70)"""
    name = "poolside_v1"
    _re = re.compile(r"<tool_call>\s*([^\n<]+?)\s*\n?\s*((?:<arg_key>.*?)?)</tool_call>", re.S)
    _kv = re.compile(r"<arg_key>([^<]*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)


class JsonParser(ToolParser):
    """Bare JSON object / array of ``{"name", "arguments"|"parameters"}`` (Llama-3.1 style)."""
    name = "json"
    start_markers = ('{"name"', '[{"name"')

    def parse(self, text):
        obj = _loads_lenient(text.strip().removeprefix("<|python_tag|>"))
        items = obj if isinstance(obj, list) else [obj]
        calls = [_call(o["name"], o.get("arguments", o.get("parameters", {}))) for o in items if isinstance(o, dict) and "name" in o]
        return ("", calls) if calls else (text, [])


PARSERS = {p.name: p for p in (HermesParser, Qwen3CoderParser, DeepSeekV3Parser, DeepSeekV31Parser, DeepSeekV4Parser, Glm45Parser,
                               KimiK2Parser, KimiK3Parser, HYV3Parser, PoolsideV1Parser, MinimaxM2Parser, JsonParser)}
PARSERS["glm47"] = Glm45Parser
PARSERS["llama3_json"] = JsonParser

_AUTO = {"qwen2": "hermes", "qwen3": "hermes", "qwen3_moe": "hermes", "deepseek_v3": "deepseek_v3", "deepseek_v32": "deepseek_v31",
         "kimi_k2": "kimi_k2", "kimi_k3": "kimi_k3", "glm4_moe": "glm45", "glm_moe_dsa": "glm47", "minimax_m2": "minimax_m2", "llama": "json",
         "deepseek_v4": "deepseek_v4", "hy_v3": "hy_v3", "hunyuan_v1_dense": "hermes", "hunyuan_v1_moe": "hermes", "laguna": "poolside_v1",
         "qwen3_next": "hermes", "qwen3_5": "qwen3_coder", "qwen3_5_moe": "qwen3_coder"}


def get_parser(name: str = "auto", model_type: str = "") -> ToolParser:
    if name in ("auto", "", None):
        name = _AUTO.get(model_type, "hermes")
    cls = PARSERS.get(name)
    if cls is None:
        raise ValueError(f"unknown tool_call_parser '{name}' (available: {sorted(PARSERS)})")
    return cls()


# ---------------------------------------------------------------------------------------------------
def split_reasoning(text: str, start: str = "<think>", end: str = "</think>"):
    """-> (reasoning_content or None, content).  A missing opening tag (template already emitted it) is accepted."""
    if end in text:
        head, tail = text.split(end, 1)
        head = head.split(start, 1)[-1] if start in head else head
        return head.strip(), tail.lstrip("\n")
    if text.lstrip().startswith(start):
        return text.lstrip()[len(start):].strip(), ""
    return None, text


class StreamSplitter:
    """Incremental reasoning / content / tool-call separation for SSE streaming.

    ``push(piece)`` returns a list of ``(kind, text)`` with kind in {"reasoning", "content"}; text that might be
    the start of tool-call markup is held back, ``finish()`` parses whatever was held into tool calls.
    """

    def __init__(self, parser: ToolParser | None, reasoning: bool = True, in_think: bool = False):
        self.parser = parser
        self.reasoning = reasoning
        self.in_think = in_think
        self.buf = ""
        self.held = ""

    def push(self, piece: str):
        out = []
        self.buf += piece
        if self.reasoning:
            if not self.in_think and "<think>" in self.buf and not self.held:
                pre, self.buf = self.buf.split("<think>", 1)
                if pre.strip():
                    out.append(("content", pre))
                self.in_think = True
            if self.in_think:
                if "</think>" in self.buf:
                    r, self.buf = self.buf.split("</think>", 1)
                    if r:
                        out.append(("reasoning", r))
                    self.in_think = False
                    self.buf = self.buf.lstrip("\n")
                else:
                    keep = 0
                    for k in range(1, len("</think>")):
                        if self.buf.endswith("</think>"[:k]):
                            keep = k
                    emit = self.buf[:len(self.buf) - keep] if keep else self.buf
                    if emit:
                        out.append(("reasoning", emit))
                    self.buf = self.buf[len(emit):]
                    return out
            elif any(self.buf.endswith("<think>"[:k]) for k in range(1, len("<think>"))) and not self.held:
                return out
        if self.parser is not None and (self.held or self.parser.may_start(self.buf)):
            # find where the markup (or its possible prefix) begins; everything before it is plain content
            cut = len(self.buf)
            for m in self.parser.start_markers:
                i = self.buf.find(m)
                if i >= 0:
                    cut = min(cut, i)
                else:
                    for k in range(len(m) - 1, 0, -1):
                        if self.buf.endswith(m[:k]):
                            cut = min(cut, len(self.buf) - k)
                            break
            if not self.held and cut > 0:
                out.append(("content", self.buf[:cut]))
            self.held += self.buf[cut:] if not self.held else self.buf
            self.buf = ""
            if self.held and not any(m in self.held or any(self.held.endswith(m[:k]) for k in range(1, len(m))) for m in self.parser.start_markers):
                out.append(("content", self.held))       # false alarm
                self.held = ""
            return out
        if self.buf:
            out.append(("content", self.buf))
            self.buf = ""
        return out

    def finish(self):
        """-> (trailing content, tool calls)"""
        rest = self.held + self.buf
        self.held = self.buf = ""
        if self.parser is None or not rest:
            return rest, []
        return self.parser.parse(rest)
