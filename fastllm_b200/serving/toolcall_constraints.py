"""Constrained generation for tool calls: while the model is writing a function name, only tokens that keep the
name a prefix of one of the declared tools are allowed.

The reference exposes a per-request tool-call constraint hook into its sampler
(tools/fastllm_pytools/openai_server/toolcall_constraints.py builds the name constraint per wire format,
``set_tool_call_constraint_llm_model`` in tools/src/pytools.cpp:352 installs it).  Here the constraint is a
logits processor on the request (``GenerationConfig.logits_processor``): the engine calls it with the tokens
generated so far and masks every token it does not return.

A wire format is described by the text that precedes a function name and the character that ends it:

    hermes        <tool_call>\\n{"name": "          ... "
    qwen3_coder   <function=                        ... >
    deepseek_v4   <｜DSML｜invoke name="             ... "
    minimax_m2    <invoke name="                    ... "
    glm45 / 47    <tool_call>                       ... \\n
    kimi_k2       <|tool_call_begin|>functions.     ... :
"""
from __future__ import annotations

import re

FORMATS = {
    "hermes": (r'<tool_call>\s*\{\s*"name"\s*:\s*"', '"'),
    "qwen3_coder": (r"<function=", ">"),
    "deepseek_v4": (r'<(?:｜DSML｜|\\DSML\\)invoke\s+name="', '"'),
    "minimax_m2": (r'<invoke name="', '"'),
    "glm45": (r"<tool_call>", "\n"),
    "glm47": (r"<tool_call>", "\n"),
    "poolside_v1": (r"<tool_call>", "\n"),
    "kimi_k2": (r"<\|tool_call_begin\|>\s*functions\.", ":"),
    "kimi_k3": (r'<\|open\|>\s*call\s+tool="', '"'),
}


class ToolNameConstraint:
    """``__call__(output_ids) -> allowed token ids or None`` (None = no restriction at this position)."""

    def __init__(self, tokenizer, parser_name: str, tool_names, tail_tokens: int = 48):
        if parser_name not in FORMATS:
            raise ValueError(f"no name constraint for tool-call format '{parser_name}'")
        trig, self.end = FORMATS[parser_name]
        self._trigger = re.compile("(?:" + trig + r")([^" + re.escape(self.end) + r"<]*)\Z", re.S)
        self.names = sorted(set(tool_names))
        self.tok = tokenizer
        self.tail = tail_tokens
        self._pieces = None          # token id -> decoded text, built on first use
        self.activations = 0

    def _vocab_pieces(self):
        if self._pieces is None:
            n = self.tok.vocab_size()
            self._pieces = [self.tok.decode([i], skip_special_tokens=False) for i in range(n)]
        return self._pieces

    def partial_name(self, text: str):
        m = self._trigger.search(text)
        return None if m is None else m.group(1)

    def allowed_after(self, partial: str) -> list[int]:
        """Tokens whose text keeps ``partial`` inside the declared names: either it extends the name without leaving every
        candidate, or it completes a candidate and goes on with the terminator."""
        cands = [n for n in self.names if n.startswith(partial)]
        ok = []
        for tid, piece in enumerate(self._vocab_pieces()):
            if not piece:
                continue
            for n in cands:
                rest = n[len(partial):]
                if rest and (rest.startswith(piece) or (piece.startswith(rest) and piece[len(rest):].startswith(self.end))):
                    ok.append(tid)
                    break
                if not rest and piece.startswith(self.end):
                    ok.append(tid)
                    break
        return ok

    def __call__(self, output_ids):
        if not self.names or not output_ids:
            return None
        text = self.tok.decode(list(output_ids[-self.tail:]), skip_special_tokens=False)
        partial = self.partial_name(text)
        if partial is None:
            return None
        allowed = self.allowed_after(partial)
        if not allowed:
            return None              # the tokenizer cannot spell any declared name from here: do not dead-lock the request
        self.activations += 1
        return allowed


def build_constraint(tokenizer, parser_name: str, tools) -> ToolNameConstraint | None:
    """Constraint for an OpenAI ``tools`` list, or None when the format has no name position to constrain."""
    names = [t.get("function", t).get("name") for t in tools or [] if isinstance(t, dict)]
    names = [n for n in names if n]
    if not names or parser_name not in FORMATS:
        return None
    return ToolNameConstraint(tokenizer, parser_name, names)
