"""Chat-template rendering (Hugging Face ``chat_template`` Jinja dialect).

The reference ships its own Jinja lexer/parser/evaluator in C++ (include/template.h, src/template.cpp) so
that templates work without third-party packages; here ``template_engine`` is that evaluator (lexer, parser,
interpreter, the helpers HF templates rely on: ``raise_exception``, ``strftime_now``, ``tojson``, ``namespace``).
A template that uses a construct it does not know is handed to the sandboxed ``jinja2`` environment when that
package is installed.  Without a template a ChatML layout is used.
"""
from __future__ import annotations

import datetime
import json


def _fallback(messages, add_generation_prompt=True, **_):
    out = []
    for m in messages:
        c = m.get("content", "")
        if isinstance(c, list):
            c = "".join(p.get("text", "") for p in c if isinstance(p, dict))
        out.append(f"<|im_start|>{m['role']}\n{c}<|im_end|>\n")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
    return "".join(out)


_env = None


def _environment():
    global _env
    if _env is None:
        import jinja2
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(msg):
            raise jinja2.exceptions.TemplateError(msg)

        def tojson(x, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
            return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
        env.filters["tojson"] = tojson
        env.globals["raise_exception"] = raise_exception
        env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
        _env = env
    return _env


def render(template: str | None, messages, add_generation_prompt: bool = True, tools=None, **kw) -> str:
    if not template:
        return _fallback(messages, add_generation_prompt)
    from . import template_engine

    try:
        t = _compiled.get(template)
        if t is None:
            t = _compiled[template] = template_engine.Template(template)
            if len(_compiled) > 32:
                _compiled.pop(next(iter(_compiled)))
        return t.render(messages=messages, add_generation_prompt=add_generation_prompt, tools=tools, **kw)
    except template_engine.TemplateError as e:
        own_error = e
    except (TypeError, ValueError, KeyError, IndexError, AttributeError) as e:
        own_error = e
    try:
        t = _environment().from_string(template)
    except ImportError:
        raise own_error
    return t.render(messages=messages, add_generation_prompt=add_generation_prompt, tools=tools, **kw)


_compiled: dict = {}
