"""Own chat-template evaluator against the jinja2 package on templates in the style of the major model families."""
import pytest

from fastllm_b200 import chat_template, template_engine

jinja2 = pytest.importorskip("jinja2")

LLAMA31 = r"""{{- bos_token }}
{%- if custom_tools is defined %}
    {%- set tools = custom_tools %}
{%- endif %}
{%- if not tools_in_user_message is defined %}
    {%- set tools_in_user_message = true %}
{%- endif %}
{%- if not date_string is defined %}
    {%- set date_string = "26 Jul 2024" %}
{%- endif %}
{%- if not tools is defined %}
    {%- set tools = none %}
{%- endif %}
{#- This block extracts the system message, so we can slot it into the right place. #}
{%- if messages[0]['role'] == 'system' %}
    {%- set system_message = messages[0]['content']|trim %}
    {%- set messages = messages[1:] %}
{%- else %}
    {%- set system_message = "" %}
{%- endif %}
{{- "<|start_header_id|>system<|end_header_id|>\n\n" }}
{%- if tools is not none %}
    {{- "Environment: ipython\n" }}
{%- endif %}
{{- "Cutting Knowledge Date: December 2023\n" }}
{{- "Today Date: " + date_string + "\n\n" }}
{%- if tools is not none and not tools_in_user_message %}
    {{- "You have access to the following functions." }}
    {%- for t in tools %}
        {{- t | tojson(indent=4) }}
        {{- "\n\n" }}
    {%- endfor %}
{%- endif %}
{{- system_message }}
{{- "<|eot_id|>" }}
{%- if tools_in_user_message and not tools is none %}
    {%- if messages | length != 0 %}
        {%- set first_user_message = messages[0]['content']|trim %}
        {%- set messages = messages[1:] %}
    {%- else %}
        {{- raise_exception("Cannot put tools in the first user message when there's no first user message!") }}
{%- endif %}
    {{- '<|start_header_id|>user<|end_header_id|>\n\n' -}}
    {%- for t in tools %}
        {{- t | tojson(indent=4) }}
        {{- "\n\n" }}
    {%- endfor %}
    {{- first_user_message + "<|eot_id|>"}}
{%- endif %}
{%- for message in messages %}
    {%- if not (message.role == 'ipython' or message.role == 'tool' or 'tool_calls' in message) %}
        {{- '<|start_header_id|>' + message['role'] + '<|end_header_id|>\n\n'+ message['content'] | trim + '<|eot_id|>' }}
    {%- elif 'tool_calls' in message %}
        {%- if not message.tool_calls|length == 1 %}
            {{- raise_exception("This model only supports single tool-calls at once!") }}
        {%- endif %}
        {%- set tool_call = message.tool_calls[0].function %}
        {{- '<|start_header_id|>assistant<|end_header_id|>\n\n' -}}
        {{- '{"name": "' + tool_call.name + '", ' }}
        {{- '"parameters": ' }}
        {{- tool_call.arguments | tojson }}
        {{- "}" }}
        {{- "<|eot_id|>" }}
    {%- elif message.role == "tool" or message.role == "ipython" %}
        {{- "<|start_header_id|>ipython<|end_header_id|>\n\n" }}
        {%- if message.content is mapping or message.content is iterable %}
            {{- message.content | tojson }}
        {%- else %}
            {{- message.content }}
        {%- endif %}
        {{- "<|eot_id|>" }}
    {%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|start_header_id|>assistant<|end_header_id|>\n\n' }}
{%- endif %}
"""

QWEN3 = r"""{%- if tools %}
    {{- '<|im_start|>system\n' }}
    {%- if messages[0].role == 'system' %}
        {{- messages[0].content + '\n\n' }}
    {%- endif %}
    {{- "# Tools\n\nYou may call one or more functions.\n<tools>" }}
    {%- for tool in tools %}
        {{- "\n" }}
        {{- tool | tojson }}
    {%- endfor %}
    {{- "\n</tools>\n<|im_end|>\n" }}
{%- else %}
    {%- if messages[0].role == 'system' %}
        {{- '<|im_start|>system\n' + messages[0].content + '<|im_end|>\n' }}
    {%- endif %}
{%- endif %}
{%- set ns = namespace(multi_step_tool=true, last_query_index=messages|length - 1) %}
{%- for message in messages[::-1] %}
    {%- set index = (messages|length - 1) - loop.index0 %}
    {%- if ns.multi_step_tool and message.role == "user" and message.content is string and not(message.content.startswith('<tool_response>') and message.content.endswith('</tool_response>')) %}
        {%- set ns.multi_step_tool = false %}
        {%- set ns.last_query_index = index %}
    {%- endif %}
{%- endfor %}
{%- for message in messages %}
    {%- if message.content is string %}
        {%- set content = message.content %}
    {%- else %}
        {%- set content = '' %}
    {%- endif %}
    {%- if (message.role == "user") or (message.role == "system" and not loop.first) %}
        {{- '<|im_start|>' + message.role + '\n' + content + '<|im_end|>' + '\n' }}
    {%- elif message.role == "assistant" %}
        {%- set reasoning_content = '' %}
        {%- if message.reasoning_content is string %}
            {%- set reasoning_content = message.reasoning_content %}
        {%- else %}
            {%- if '</think>' in content %}
                {%- set reasoning_content = content.split('</think>')[0].rstrip('\n').split('<think>')[-1].lstrip('\n') %}
                {%- set content = content.split('</think>')[-1].lstrip('\n') %}
            {%- endif %}
        {%- endif %}
        {%- if loop.index0 > ns.last_query_index %}
            {%- if loop.last or (not loop.last and reasoning_content) %}
                {{- '<|im_start|>' + message.role + '\n<think>\n' + reasoning_content.strip('\n') + '\n</think>\n\n' + content.lstrip('\n') }}
            {%- else %}
                {{- '<|im_start|>' + message.role + '\n' + content }}
            {%- endif %}
        {%- else %}
            {{- '<|im_start|>' + message.role + '\n' + content }}
        {%- endif %}
        {%- if message.tool_calls %}
            {%- for tool_call in message.tool_calls %}
                {%- if (loop.first and content) or (not loop.first) %}
                    {{- '\n' }}
                {%- endif %}
                {%- if tool_call.function %}
                    {%- set tool_call = tool_call.function %}
                {%- endif %}
                {{- '<tool_call>\n{"name": "' }}
                {{- tool_call.name }}
                {{- '", "arguments": ' }}
                {%- if tool_call.arguments is string %}
                    {{- tool_call.arguments }}
                {%- else %}
                    {{- tool_call.arguments | tojson }}
                {%- endif %}
                {{- '}\n</tool_call>' }}
            {%- endfor %}
        {%- endif %}
        {{- '<|im_end|>\n' }}
    {%- elif message.role == "tool" %}
        {%- if loop.first or (messages[loop.index0 - 1].role != "tool") %}
            {{- '<|im_start|>user' }}
        {%- endif %}
        {{- '\n<tool_response>\n' }}
        {{- content }}
        {{- '\n</tool_response>' }}
        {%- if loop.last or (messages[loop.index0 + 1].role != "tool") %}
            {{- '<|im_end|>\n' }}
        {%- endif %}
    {%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|im_start|>assistant\n' }}
    {%- if enable_thinking is defined and enable_thinking is false %}
        {{- '<think>\n\n</think>\n\n' }}
    {%- endif %}
{%- endif %}
"""

DEEPSEEK = r"""{% if not add_generation_prompt is defined %}{% set add_generation_prompt = false %}{% endif %}{% set ns = namespace(is_first=false, is_tool=false, is_output_first=true, system_prompt='', is_first_sp=true) %}{%- for message in messages %}{%- if message['role'] == 'system' %}{%- if ns.is_first_sp %}{% set ns.system_prompt = ns.system_prompt + message['content'] %}{% set ns.is_first_sp = false %}{%- else %}{% set ns.system_prompt = ns.system_prompt + '\n\n' + message['content'] %}{%- endif %}{%- endif %}{%- endfor %}{{ bos_token }}{{ ns.system_prompt }}{%- for message in messages %}{%- if message['role'] == 'user' %}{%- set ns.is_tool = false -%}{{'<|User|>' + message['content']}}{%- endif %}{%- if message['role'] == 'assistant' and 'tool_calls' in message and message['tool_calls'] is not none %}{%- set ns.is_first = false %}{%- for tool in message['tool_calls'] %}{%- if not ns.is_first %}{{'<|Assistant|><|tool_calls_begin|><|tool_call_begin|>' + tool['type'] + '<|tool_sep|>' + tool['function']['name'] + '\n' + '```json' + '\n' + tool['function']['arguments'] + '\n' + '```' + '<|tool_call_end|>'}}{%- set ns.is_first = true -%}{%- else %}{{'\n' + '<|tool_call_begin|>' + tool['type'] + '<|tool_sep|>' + tool['function']['name'] + '\n' + '```json' + '\n' + tool['function']['arguments'] + '\n' + '```' + '<|tool_call_end|>'}}{%- endif %}{%- endfor %}{{'<|tool_calls_end|><|end_of_sentence|>'}}{%- endif %}{%- if message['role'] == 'assistant' and (message['tool_calls'] is not defined or message['tool_calls'] is none) %}{%- if ns.is_tool %}{{'<|tool_outputs_end|>' + message['content'] + '<|end_of_sentence|>'}}{%- set ns.is_tool = false -%}{%- else %}{% set content = message['content'] %}{% if '</think>' in content %}{% set content = content.split('</think>')[-1] %}{% endif %}{{'<|Assistant|>' + content + '<|end_of_sentence|>'}}{%- endif %}{%- endif %}{%- if message['role'] == 'tool' %}{%- set ns.is_tool = true -%}{%- if ns.is_output_first %}{{'<|tool_outputs_begin|><|tool_output_begin|>' + message['content'] + '<|tool_output_end|>'}}{%- set ns.is_output_first = false %}{%- else %}{{'\n<|tool_output_begin|>' + message['content'] + '<|tool_output_end|>'}}{%- endif %}{%- endif %}{%- endfor -%}{% if ns.is_tool %}{{'<|tool_outputs_end|>'}}{% endif %}{% if add_generation_prompt and not ns.is_tool %}{{'<|Assistant|><think>\n'}}{% endif %}"""

MISTRAL = r"""{{ bos_token }}{% for message in messages %}{% if (message['role'] == 'user') != (loop.index0 % 2 == 0) %}{{ raise_exception('Conversation roles must alternate user/assistant/user/assistant/...') }}{% endif %}{% if message['role'] == 'user' %}{{ '[INST] ' + message['content'] + ' [/INST]' }}{% elif message['role'] == 'assistant' %}{{ message['content'] + eos_token}}{% else %}{{ raise_exception('Only user and assistant roles are supported!') }}{% endif %}{% endfor %}"""

GEMMA = r"""{{ bos_token }}{% if messages[0]['role'] == 'system' %}{{ raise_exception('System role not supported') }}{% endif %}{% for message in messages %}{% if (message['role'] == 'assistant') %}{% set role = 'model' %}{% else %}{% set role = message['role'] %}{% endif %}{{ '<start_of_turn>' + role + '\n' + message['content'] | trim + '<end_of_turn>\n' }}{% endfor %}{% if add_generation_prompt %}{{'<start_of_turn>model\n'}}{% endif %}"""

MACROS = r"""{%- macro render_content(content, do_count=false) -%}
  {%- if content is string -%}{{ content }}
  {%- else -%}
    {%- for item in content -%}
      {%- if 'image' in item or item.type == 'image' -%}<|vision_start|><|image_pad|><|vision_end|>
      {%- elif 'text' in item -%}{{ item.text }}
      {%- endif -%}
    {%- endfor -%}
  {%- endif -%}
{%- endmacro -%}
{% for m in messages if m.role != 'skip' %}
[{{ loop.index }}/{{ loop.length }}{{ ' first' if loop.first }}{{ ' last' if loop.last else '' }}] {{ m.role | upper }}: {{ render_content(m.content) }}
{% else %}
no messages
{% endfor %}
{%- set names = messages | map(attribute='role') | unique | sort | join(', ') %}
roles: {{ names }}
{% for k, v in {'b': 2, 'a': 1} | dictsort %}{{ k }}={{ v }};{% endfor %}
{{ messages | selectattr('role', 'equalto', 'user') | list | length }} user / {{ messages | rejectattr('role', 'eq', 'user') | list | length }} other
{% for i in range(10) %}{% if i == 2 %}{% continue %}{% endif %}{% if i > 4 %}{% break %}{% endif %}{{ i }}{% endfor %}
{{ 7 // 2 }} {{ 7 % 3 }} {{ 2 ** 5 }} {{ (1, 2)[1] }} {{ [1, 2, 3][-1] }} {{ 'abc'[1:] }} {{ 3 if false else 4 }} {{ 'x' ~ 1 ~ none }}
{{ "%s-%d" | format("a", 3) }} {{ 3.14159 | round(2) }} {{ '  hi ' | trim | capitalize }} {{ [3, 1, 2] | sort | first }} {{ undefined_thing | default('dflt') }}
{% set joined %}{{ 'block' }} set{% endset %}{{ joined | upper }}
{% raw %}{{ not evaluated }}{% endraw %}
"""

MSGS = [
    {"role": "system", "content": " You are a helpful assistant. "},
    {"role": "user", "content": "What's the weather in Paris?"},
    {"role": "assistant", "content": "<think>\nneed a tool\n</think>\n\nLet me check.",
     "tool_calls": [{"type": "function", "function": {"name": "get_weather", "arguments": {"city": "Paris", "unit": "c"}}}]},
    {"role": "tool", "content": "{\"temp\": 21}"},
    {"role": "assistant", "content": "It is 21 °C in Paris — sunny."},
    {"role": "user", "content": "Merci ✓"},
]
TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "Get the weather", "parameters":
          {"type": "object", "properties": {"city": {"type": "string"}, "unit": {"type": "string", "enum": ["c", "f"]}}, "required": ["city"]}}}]
PLAIN = [m for m in MSGS if m["role"] in ("user",) or (m["role"] == "assistant" and "tool_calls" not in m)]


def _both(template, **kw):
    want = chat_template._environment().from_string(template).render(**kw)
    got = template_engine.render(template, **kw)
    assert got == want
    return got


@pytest.mark.parametrize("tools", [None, TOOLS])
@pytest.mark.parametrize("gen", [True, False])
def test_llama31_style(tools, gen):
    kw = dict(messages=MSGS, add_generation_prompt=gen, bos_token="<|begin_of_text|>")
    if tools:
        kw["tools"] = tools
    out = _both(LLAMA31, **kw)
    assert out.startswith("<|begin_of_text|><|start_header_id|>system")


@pytest.mark.parametrize("tools", [None, TOOLS])
@pytest.mark.parametrize("thinking", [None, False])
def test_qwen3_style(tools, thinking):
    kw = dict(messages=MSGS, add_generation_prompt=True, tools=tools)
    if thinking is not None:
        kw["enable_thinking"] = thinking
    out = _both(QWEN3, **kw)
    assert out.endswith("<|im_start|>assistant\n" if thinking is None else "</think>\n\n")


def test_deepseek_style_namespace_and_string_arguments():
    msgs = [dict(m) for m in MSGS]
    msgs[2] = dict(msgs[2], tool_calls=[{"type": "function", "function": {"name": "get_weather", "arguments": "{\"city\": \"Paris\"}"}}])
    _both(DEEPSEEK, messages=msgs, add_generation_prompt=True, bos_token="<bos>")
    _both(DEEPSEEK, messages=PLAIN, bos_token="<bos>")


def test_mistral_and_gemma_style_and_raised_exceptions():
    _both(MISTRAL, messages=PLAIN, bos_token="<s>", eos_token="</s>")
    _both(GEMMA, messages=PLAIN, add_generation_prompt=True, bos_token="<bos>")
    with pytest.raises(template_engine.TemplateError, match="System role not supported"):
        template_engine.render(GEMMA, messages=MSGS, bos_token="<bos>")
    with pytest.raises(template_engine.TemplateError, match="alternate"):
        template_engine.render(MISTRAL, messages=MSGS[1:], bos_token="<s>", eos_token="</s>")


def test_macros_loops_filters_and_expressions():
    msgs = [{"role": "user", "content": [{"type": "text", "text": "look: "}, {"type": "image", "image": "x.png"}]},
            {"role": "skip", "content": "hidden"}, {"role": "assistant", "content": "a cat"}, {"role": "user", "content": "ok"}]
    _both(MACROS, messages=msgs)
    _both(MACROS, messages=[])


def test_chat_template_render_uses_own_engine(monkeypatch):
    import builtins

    real = builtins.__import__

    def no_jinja(name, *a, **k):
        if name.startswith("jinja2"):
            raise ImportError(name)
        return real(name, *a, **k)

    want = chat_template._environment().from_string(QWEN3).render(messages=MSGS, add_generation_prompt=True, tools=TOOLS)
    monkeypatch.setattr(builtins, "__import__", no_jinja)
    assert chat_template.render(QWEN3, MSGS, True, tools=TOOLS) == want
