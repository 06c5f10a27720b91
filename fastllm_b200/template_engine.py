"""Own evaluator for the Jinja dialect of Hugging Face chat templates: lexer, recursive-descent parser, tree-walking
interpreter.  No third-party dependency; ``chat_template.render`` uses it first and falls back to the ``jinja2`` package
only for constructs it does not know.

Covered: ``{{ }}`` / ``{% %}`` / ``{# #}`` with ``-`` whitespace control plus ``trim_blocks`` / ``lstrip_blocks``;
statements ``if / elif / else``, ``for`` (tuple targets, inline ``if``, ``else``, ``loop.*``, ``recursive`` excluded),
``set`` (also ``ns.attr`` targets and block form), ``macro`` / ``call``-less invocation, ``break`` / ``continue``, ``raw``,
``filter`` blocks, ``generation`` (transparent); expressions with literals, attribute / subscript / slice access, calls
with keyword arguments, arithmetic, ``~``, comparisons, ``in``, boolean logic, conditional expressions, filters and tests.
Python string / dict / list methods are reachable the way the sandboxed environment of the original allows.

Counterpart of the reference's C++ template engine (include/template.h, src/template.cpp: JinjaToken / JinjaAST / JinjaVar),
which covers a smaller subset.
"""
from __future__ import annotations

import datetime
import json
import re


class TemplateError(Exception):
    pass


class Undefined:
    """Missing name / key / attribute: falsy, prints as nothing, iterates as empty, stays undefined under access."""
    __slots__ = ("name",)

    def __init__(self, name=""):
        self.name = name

    def __bool__(self):
        return False

    def __str__(self):
        return ""

    def __iter__(self):
        return iter(())

    def __len__(self):
        return 0

    def __eq__(self, other):
        return isinstance(other, Undefined)

    def __hash__(self):
        return 0

    def __getattr__(self, k):
        if k.startswith("__"):
            raise AttributeError(k)
        return Undefined(k)

    def __getitem__(self, k):
        return Undefined(str(k))

    def __call__(self, *a, **k):
        raise TemplateError(f"'{self.name}' is undefined")


class _Namespace:
    def __init__(self, **kw):
        self.__dict__.update(kw)


class _Break(Exception):
    pass


class _Continue(Exception):
    pass


# ---------------------------------------------------------------------------------------------------
# lexer
# ---------------------------------------------------------------------------------------------------
_TAG_RE = re.compile(r"\{\{|\{%|\{#")
_EXPR_TOKEN = re.compile(r"""
    \s*(?:
      (?P<num>\d+\.\d+(?:[eE][+-]?\d+)?|\d+(?:[eE][+-]?\d+)?)
    | (?P<str>'(?:\\.|[^'\\])*'|"(?:\\.|[^"\\])*")
    | (?P<name>[A-Za-z_][A-Za-z0-9_]*)
    | (?P<op>==|!=|<=|>=|//|\*\*|[-+*/%~<>()\[\]{},.:|=])
    )""", re.X | re.S)
_ESC = {"n": "\n", "t": "\t", "r": "\r", "\\": "\\", "'": "'", '"': '"', "0": "\0", "a": "\a", "b": "\b", "f": "\f", "v": "\v"}


def _unescape(s: str) -> str:
    out, i = [], 0
    while i < len(s):
        c = s[i]
        if c == "\\" and i + 1 < len(s):
            n = s[i + 1]
            if n in _ESC:
                out.append(_ESC[n]); i += 2; continue
            if n == "u" and i + 5 < len(s) + 1:
                out.append(chr(int(s[i + 2:i + 6], 16))); i += 6; continue
            if n == "x":
                out.append(chr(int(s[i + 2:i + 4], 16))); i += 4; continue
            out.append(c + n); i += 2; continue
        out.append(c); i += 1
    return "".join(out)


def _lex(src: str, trim_blocks: bool, lstrip_blocks: bool):
    """-> list of ("data", text) | ("var", expr_src) | ("block", stmt_src)."""
    out = []
    pos = 0
    strip_next = False          # previous tag ended with '-': strip leading whitespace of the next data
    trim_nl = False             # previous block tag (trim_blocks): drop one leading newline of the next data
    while True:
        m = _TAG_RE.search(src, pos)
        data = src[pos:m.start()] if m else src[pos:]
        if strip_next:
            data = data.lstrip()
        elif trim_nl and data.startswith("\n"):
            data = data[1:]
        elif trim_nl and data.startswith("\r\n"):
            data = data[2:]
        strip_next = trim_nl = False
        if not m:
            if data:
                out.append(("data", data))
            break
        kind = m.group()
        close = {"{{": "}}", "{%": "%}", "{#": "#}"}[kind]
        start = m.end()
        if kind == "{%" and re.match(r"-?\s*raw\s*-?%\}", src[start:]):
            # raw block: everything up to endraw is data
            head = re.match(r"(-?)\s*raw\s*(-?)%\}", src[start:])
            endm = re.search(r"\{%(-?)\s*endraw\s*(-?)%\}", src[start + head.end():])
            if not endm:
                raise TemplateError("unclosed raw block")
            if head.group(1) == "-":
                data = data.rstrip()
            elif lstrip_blocks:
                data = _lstrip_line(data)
            if data:
                out.append(("data", data))
            raw = src[start + head.end():start + head.end() + endm.start()]
            if head.group(2) == "-":
                raw = raw.lstrip()
            if endm.group(1) == "-":
                raw = raw.rstrip()
            out.append(("data", raw))
            pos = start + head.end() + endm.end()
            strip_next = endm.group(2) == "-"
            trim_nl = trim_blocks and not strip_next
            continue
        end = _find_close(src, start, close)
        if end < 0:
            raise TemplateError(f"unclosed '{kind}'")
        inner = src[start:end]
        lstrip_here = inner.startswith("-")
        no_lstrip = inner.startswith("+")
        if lstrip_here or no_lstrip:
            inner = inner[1:]
        rstrip_after = inner.endswith("-")
        keep_after = inner.endswith("+") and kind != "{{"
        if rstrip_after or keep_after:
            inner = inner[:-1]
        if lstrip_here:
            data = data.rstrip()
        elif lstrip_blocks and kind != "{{" and not no_lstrip:
            data = _lstrip_line(data)
        if data:
            out.append(("data", data))
        if kind == "{{":
            out.append(("var", inner))
        elif kind == "{%":
            out.append(("block", inner.strip()))
        pos = end + 2
        strip_next = rstrip_after
        trim_nl = trim_blocks and kind != "{{" and not rstrip_after and not keep_after
    return out


def _lstrip_line(data: str) -> str:
    """lstrip_blocks: blanks between the last newline and a block tag disappear (only if nothing else is on that line)."""
    i = len(data)
    while i > 0 and data[i - 1] in " \t":
        i -= 1
    if i == 0 or data[i - 1] == "\n":
        return data[:i]
    return data


def _find_close(src: str, start: int, close: str) -> int:
    """Position of the closing delimiter, skipping string literals."""
    i, n = start, len(src)
    if close == "#}":
        return src.find(close, start)
    while i < n:
        c = src[i]
        if c in "'\"":
            j = i + 1
            while j < n and src[j] != c:
                j += 2 if src[j] == "\\" else 1
            i = j + 1
            continue
        if src.startswith(close, i):
            return i
        i += 1
    return -1


def _tokens(expr: str):
    out, pos, n = [], 0, len(expr)
    while pos < n:
        if expr[pos:].strip() == "":
            break
        m = _EXPR_TOKEN.match(expr, pos)
        if not m:
            raise TemplateError(f"bad expression near '{expr[pos:pos + 20]}'")
        pos = m.end()
        if m.group("num") is not None:
            t = m.group("num")
            out.append(("num", float(t) if ("." in t or "e" in t or "E" in t) else int(t)))
        elif m.group("str") is not None:
            out.append(("str", _unescape(m.group("str")[1:-1])))
        elif m.group("name") is not None:
            out.append(("name", m.group("name")))
        else:
            out.append(("op", m.group("op")))
    out.append(("eof", None))
    return out


# ---------------------------------------------------------------------------------------------------
# expression parser: nodes are tuples ("kind", ...)
# ---------------------------------------------------------------------------------------------------
class _P:
    def __init__(self, toks):
        self.t, self.i = toks, 0

    def peek(self):
        return self.t[self.i]

    def next(self):
        tok = self.t[self.i]
        self.i += 1
        return tok

    def at(self, kind, val=None):
        k, v = self.t[self.i]
        return k == kind and (val is None or v == val)

    def accept(self, kind, val=None):
        if self.at(kind, val):
            return self.next()
        return None

    def expect(self, kind, val=None):
        if not self.at(kind, val):
            raise TemplateError(f"expected {val or kind}, got {self.peek()[1]!r}")
        return self.next()

    # expression := or_expr ["if" or_expr ["else" expression]]
    def expression(self, allow_cond=True):
        e = self.or_()
        if allow_cond and self.at("name", "if"):
            self.next()
            c = self.or_()
            alt = ("const", Undefined())
            if self.accept("name", "else"):
                alt = self.expression()
            e = ("cond", c, e, alt)
        return e

    def or_(self):
        e = self.and_()
        while self.accept("name", "or"):
            e = ("or", e, self.and_())
        return e

    def and_(self):
        e = self.not_()
        while self.accept("name", "and"):
            e = ("and", e, self.not_())
        return e

    def not_(self):
        if self.accept("name", "not"):
            return ("not", self.not_())
        return self.compare()

    def compare(self):
        e = self.add()
        while True:
            if self.at("op") and self.peek()[1] in ("==", "!=", "<", ">", "<=", ">="):
                op = self.next()[1]
                e = ("cmp", op, e, self.add())
            elif self.at("name", "in"):
                self.next()
                e = ("in", e, self.add())
            elif self.at("name", "not") and self.t[self.i + 1] == ("name", "in"):
                self.next(); self.next()
                e = ("not", ("in", e, self.add()))
            else:
                return e

    def add(self):
        e = self.concat()
        while self.at("op") and self.peek()[1] in ("+", "-"):
            op = self.next()[1]
            e = ("bin", op, e, self.concat())
        return e

    def concat(self):
        e = self.mul()
        while self.accept("op", "~"):
            e = ("bin", "~", e, self.mul())
        return e

    def mul(self):
        e = self.pow_()
        while self.at("op") and self.peek()[1] in ("*", "/", "//", "%"):
            op = self.next()[1]
            e = ("bin", op, e, self.pow_())
        return e

    def pow_(self):
        e = self.unary()
        while self.accept("op", "**"):
            e = ("bin", "**", e, self.unary())
        return e

    def unary(self):
        if self.at("op", "-"):
            self.next()
            return self.filters(("neg", self.unary_nofilter()))
        if self.at("op", "+"):
            self.next()
            return self.filters(self.unary_nofilter())
        return self.filters(self.postfix(self.primary()))

    def unary_nofilter(self):
        if self.at("op", "-"):
            self.next()
            return ("neg", self.unary_nofilter())
        return self.postfix(self.primary())

    def filters(self, e):
        while True:
            if self.accept("op", "|"):
                name = self.expect("name")[1]
                args, kwargs = [], []
                if self.accept("op", "("):
                    args, kwargs = self.call_args()
                e = ("filter", name, e, args, kwargs)
            elif self.at("name", "is"):
                self.next()
                neg = bool(self.accept("name", "not"))
                name = self.expect("name")[1]
                args = []
                if self.accept("op", "("):
                    args, _ = self.call_args()
                elif (self.peek()[0] in ("num", "str") or (self.at("name") and self.peek()[1] not in
                                                          ("and", "or", "else", "if", "not", "in", "is", "recursive"))):
                    args = [self.postfix(self.primary())]
                e = ("test", name, e, args)
                if neg:
                    e = ("not", e)
            else:
                return e

    def call_args(self):
        args, kwargs = [], []
        while not self.at("op", ")"):
            if self.at("name") and self.t[self.i + 1] == ("op", "="):
                k = self.next()[1]
                self.next()
                kwargs.append((k, self.expression()))
            elif self.at("op", "*"):
                self.next()
                args.append(("star", self.expression()))
            else:
                args.append(self.expression())
            if not self.accept("op", ","):
                break
        self.expect("op", ")")
        return args, kwargs

    def postfix(self, e):
        while True:
            if self.accept("op", "."):
                tok = self.next()
                if tok[0] == "num":
                    e = ("item", e, ("const", tok[1]))
                else:
                    e = ("attr", e, tok[1])
            elif self.accept("op", "["):
                e = ("item", e, self.subscript())
                self.expect("op", "]")
            elif self.accept("op", "("):
                args, kwargs = self.call_args()
                e = ("call", e, args, kwargs)
            else:
                return e

    def subscript(self):
        parts = []
        is_slice = False
        cur = None
        while True:
            if self.at("op", ":"):
                self.next()
                is_slice = True
                parts.append(cur)
                cur = None
            elif self.at("op", "]"):
                parts.append(cur)
                break
            else:
                cur = self.expression()
        if not is_slice:
            return parts[0]
        while len(parts) < 3:
            parts.append(None)
        return ("slice", parts[0], parts[1], parts[2])

    def primary(self):
        k, v = self.next()
        if k == "num":
            return ("const", v)
        if k == "str":
            s = v
            while self.at("str"):          # adjacent literals concatenate
                s += self.next()[1]
            return ("const", s)
        if k == "name":
            if v in ("true", "True"):
                return ("const", True)
            if v in ("false", "False"):
                return ("const", False)
            if v in ("none", "None"):
                return ("const", None)
            return ("name", v)
        if k == "op" and v == "(":
            if self.accept("op", ")"):
                return ("tuple", [])
            e = self.expression()
            if self.at("op", ","):
                items = [e]
                while self.accept("op", ","):
                    if self.at("op", ")"):
                        break
                    items.append(self.expression())
                self.expect("op", ")")
                return ("tuple", items)
            self.expect("op", ")")
            return e
        if k == "op" and v == "[":
            items = []
            while not self.at("op", "]"):
                items.append(self.expression())
                if not self.accept("op", ","):
                    break
            self.expect("op", "]")
            return ("list", items)
        if k == "op" and v == "{":
            items = []
            while not self.at("op", "}"):
                key = self.expression()
                self.expect("op", ":")
                items.append((key, self.expression()))
                if not self.accept("op", ","):
                    break
            self.expect("op", "}")
            return ("dict", items)
        raise TemplateError(f"unexpected token {v!r}")


# ---------------------------------------------------------------------------------------------------
# statement parser
# ---------------------------------------------------------------------------------------------------
def _parse(tokens):
    pos = 0

    def block(until):
        nonlocal pos
        body = []
        while pos < len(tokens):
            kind, text = tokens[pos]
            if kind == "data":
                body.append(("data", text)); pos += 1
            elif kind == "var":
                p = _P(_tokens(text))
                e = p.expression()
                p.expect("eof")
                body.append(("out", e)); pos += 1
            else:
                word = text.split(None, 1)[0] if text else ""
                if word in until:
                    return body, text
                pos += 1
                body.append(statement(word, text[len(word):].strip()))
        if until:
            raise TemplateError(f"missing {' / '.join(until)}")
        return body, None

    def statement(word, rest):
        nonlocal pos
        if word == "if":
            branches = []
            cond = _expr(rest)
            while True:
                body, end = block(("elif", "else", "endif"))
                pos += 1
                branches.append((cond, body))
                w = end.split(None, 1)[0]
                if w == "elif":
                    cond = _expr(end[4:].strip())
                elif w == "else":
                    body, end = block(("endif",))
                    pos += 1
                    branches.append((None, body))
                    break
                else:
                    break
            return ("if", branches)
        if word == "for":
            p = _P(_tokens(rest))
            targets = [p.expect("name")[1]]
            while p.accept("op", ","):
                targets.append(p.expect("name")[1])
            p.expect("name", "in")
            it = p.expression(allow_cond=False)
            cond = None
            if p.accept("name", "if"):
                cond = p.expression(allow_cond=False)
            p.accept("name", "recursive")
            p.expect("eof")
            body, end = block(("else", "endfor"))
            pos += 1
            orelse = []
            if end.split(None, 1)[0] == "else":
                orelse, _ = block(("endfor",))
                pos += 1
            return ("for", targets, it, cond, body, orelse)
        if word == "set":
            p = _P(_tokens(rest))
            first = p.expect("name")[1]
            target = ("name", first)
            if p.accept("op", "."):
                target = ("nsattr", first, p.expect("name")[1])
            names = [target]
            while p.accept("op", ","):
                names.append(("name", p.expect("name")[1]))
            if p.accept("op", "="):
                e = p.expression()
                if p.at("op", ","):          # a, b = x, y
                    items = [e]
                    while p.accept("op", ","):
                        items.append(p.expression())
                    e = ("tuple", items)
                p.expect("eof")
                return ("set", names, e)
            flt = None
            if p.at("op", "|"):
                flt = p.filters(("name", "\0body"))
            p.expect("eof")
            body, _ = block(("endset",))
            pos += 1
            return ("setblock", names[0], body, flt)
        if word == "macro":
            p = _P(_tokens(rest))
            name = p.expect("name")[1]
            p.expect("op", "(")
            params = []
            while not p.at("op", ")"):
                pn = p.expect("name")[1]
                default = None
                if p.accept("op", "="):
                    default = p.expression()
                params.append((pn, default))
                if not p.accept("op", ","):
                    break
            p.expect("op", ")")
            body, _ = block(("endmacro",))
            pos += 1
            return ("macro", name, params, body)
        if word == "filter":
            p = _P(_tokens(rest))
            flt = p.filters(("name", "\0body"))     # parses "name(args)|other" as filters over the block's text
            body, _ = block(("endfilter",))
            pos += 1
            return ("filterblock", flt, body)
        if word == "generation":
            body, _ = block(("endgeneration",))
            pos += 1
            return ("group", body)
        if word == "call":
            p = _P(_tokens(rest))
            e = p.expression()
            body, _ = block(("endcall",))
            pos += 1
            return ("callblock", e, body)
        if word == "break":
            return ("break",)
        if word == "continue":
            return ("continue",)
        if word == "do":
            return ("do", _expr(rest))
        raise TemplateError(f"unsupported statement '{word}'")

    body, _ = block(())
    return body


def _expr(text):
    p = _P(_tokens(text))
    e = p.expression()
    p.expect("eof")
    return e


# ---------------------------------------------------------------------------------------------------
# evaluation
# ---------------------------------------------------------------------------------------------------
class _Loop:
    def __init__(self, n, depth=1):
        self.length, self.index0, self.depth = n, -1, depth
        self._prev = self._next = Undefined()

    index = property(lambda s: s.index0 + 1)
    first = property(lambda s: s.index0 == 0)
    last = property(lambda s: s.index0 == s.length - 1)
    revindex = property(lambda s: s.length - s.index0)
    revindex0 = property(lambda s: s.length - s.index0 - 1)
    previtem = property(lambda s: s._prev)
    nextitem = property(lambda s: s._next)

    def cycle(self, *vals):
        return vals[self.index0 % len(vals)] if vals else Undefined()


_SAFE_METHODS = {
    str: {"strip", "lstrip", "rstrip", "startswith", "endswith", "split", "rsplit", "splitlines", "upper", "lower", "title",
          "capitalize", "replace", "join", "find", "rfind", "index", "count", "format", "isdigit", "isalpha", "isalnum",
          "isspace", "islower", "isupper", "removeprefix", "removesuffix", "zfill", "center", "ljust", "rjust", "partition",
          "rpartition", "encode", "casefold", "swapcase", "expandtabs"},
    dict: {"items", "keys", "values", "get", "copy", "update", "pop", "setdefault"},
    list: {"append", "extend", "pop", "index", "count", "copy", "insert", "remove", "reverse", "sort"},
    tuple: {"index", "count"},
}


def _getattr(obj, name):
    if isinstance(obj, Undefined):
        return Undefined(name)
    if isinstance(obj, dict):
        if name in obj and name not in _SAFE_METHODS[dict]:
            return obj[name]
        if name in _SAFE_METHODS[dict]:
            return obj[name] if (name in obj and not callable(getattr(dict, name, None))) else getattr(obj, name)
        return Undefined(name)
    for tp, names in _SAFE_METHODS.items():
        if isinstance(obj, tp):
            return getattr(obj, name) if name in names else Undefined(name)
    if isinstance(obj, (_Namespace, _Loop, _Macro)) or hasattr(obj, "__dict__"):
        if name.startswith("_"):
            return Undefined(name)
        v = getattr(obj, name, None)
        return Undefined(name) if v is None and not hasattr(obj, name) else v
    return Undefined(name)


def _getitem(obj, key):
    if isinstance(obj, Undefined):
        return Undefined(str(key))
    try:
        return obj[key]
    except (KeyError, IndexError, TypeError):
        if isinstance(key, str):
            return _getattr(obj, key)
        return Undefined(str(key))


def _tojson(x, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
    def default(o):
        if isinstance(o, Undefined):
            return None
        if isinstance(o, _Namespace):
            return o.__dict__
        raise TypeError(type(o).__name__)
    return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys, default=default)


def _to_str(v):
    if v is None:
        return "None"
    if v is True:
        return "True"
    if v is False:
        return "False"
    return str(v)


def _attr_getter(attr):
    parts = str(attr).split(".")

    def get(o):
        for p in parts:
            o = _getitem(o, int(p)) if p.isdigit() else _getattr(o, p)
        return o
    return get


class _Interp:
    def __init__(self):
        self.filters = {
            "tojson": _tojson, "trim": lambda s, chars=None: _to_str(s).strip(chars), "length": len, "count": len,
            "default": self._default, "d": self._default, "join": self._join, "upper": lambda s: _to_str(s).upper(),
            "lower": lambda s: _to_str(s).lower(), "title": lambda s: _to_str(s).title(),
            "capitalize": lambda s: _to_str(s).capitalize(), "first": lambda s: next(iter(s), Undefined()),
            "last": lambda s: (list(s) or [Undefined()])[-1], "list": list, "string": _to_str, "safe": lambda s: s,
            "int": self._int, "float": self._float, "abs": abs, "round": self._round, "items": lambda d: list(d.items()) if isinstance(d, dict) else [],
            "replace": lambda s, a, b, count=None: _to_str(s).replace(a, b) if count is None else _to_str(s).replace(a, b, count),
            "reverse": lambda s: s[::-1] if isinstance(s, (str, list, tuple)) else list(s)[::-1],
            "sort": self._sort, "unique": self._unique, "map": self._map, "select": self._select_f(True, False),
            "reject": self._select_f(False, False), "selectattr": self._select_f(True, True), "rejectattr": self._select_f(False, True),
            "sum": self._sum, "min": lambda s, **k: min(s) if s else Undefined(), "max": lambda s, **k: max(s) if s else Undefined(),
            "indent": self._indent, "dictsort": lambda d, **k: sorted(d.items(), key=lambda kv: _to_str(kv[0]).lower()),
            "batch": self._batch, "escape": self._escape, "e": self._escape, "wordcount": lambda s: len(_to_str(s).split()),
            "bool": bool, "attr": lambda o, n: _getattr(o, n), "striptags": lambda s: re.sub(r"<[^>]*>", "", _to_str(s)),
            "center": lambda s, w=80: _to_str(s).center(w), "truncate": self._truncate, "format": lambda s, *a, **k: _to_str(s) % (a or k),
            "fromjson": json.loads, "from_json": json.loads, "pprint": lambda x: repr(x), "groupby": self._groupby,
        }
        self.tests = {
            "defined": lambda v: not isinstance(v, Undefined), "undefined": lambda v: isinstance(v, Undefined),
            "none": lambda v: v is None, "string": lambda v: isinstance(v, str),
            "number": lambda v: isinstance(v, (int, float)) and not isinstance(v, bool),
            "integer": lambda v: isinstance(v, int) and not isinstance(v, bool), "float": lambda v: isinstance(v, float),
            "boolean": lambda v: isinstance(v, bool), "true": lambda v: v is True, "false": lambda v: v is False,
            "mapping": lambda v: isinstance(v, dict), "sequence": lambda v: isinstance(v, (list, tuple, str, dict)),
            "iterable": lambda v: isinstance(v, (list, tuple, str, dict)) or hasattr(v, "__iter__") and not isinstance(v, Undefined),
            "callable": callable, "even": lambda v: v % 2 == 0, "odd": lambda v: v % 2 == 1,
            "divisibleby": lambda v, n: v % n == 0, "equalto": lambda a, b: a == b, "eq": lambda a, b: a == b,
            "ne": lambda a, b: a != b, "lt": lambda a, b: a < b, "le": lambda a, b: a <= b, "gt": lambda a, b: a > b,
            "ge": lambda a, b: a >= b, "greaterthan": lambda a, b: a > b, "lessthan": lambda a, b: a < b,
            "in": lambda a, b: a in b, "lower": lambda v: _to_str(v).islower(), "upper": lambda v: _to_str(v).isupper(),
            "sameas": lambda a, b: a is b, "escaped": lambda v: False,
        }

    # -- filters with arguments --
    @staticmethod
    def _default(v, d="", boolean=False):
        return d if isinstance(v, Undefined) or (boolean and not v) else v

    @staticmethod
    def _join(seq, d="", attribute=None):
        if attribute is not None:
            g = _attr_getter(attribute)
            seq = [g(x) for x in seq]
        return _to_str(d).join(_to_str(x) for x in seq)

    @staticmethod
    def _int(v, default=0, base=10):
        try:
            return int(v, base) if isinstance(v, str) else int(v)
        except (TypeError, ValueError):
            try:
                return int(float(v))
            except (TypeError, ValueError):
                return default

    @staticmethod
    def _float(v, default=0.0):
        try:
            return float(v)
        except (TypeError, ValueError):
            return default

    @staticmethod
    def _round(v, precision=0, method="common"):
        import math

        f = 10 ** precision
        if method == "ceil":
            return math.ceil(v * f) / f
        if method == "floor":
            return math.floor(v * f) / f
        return round(v, precision)

    @staticmethod
    def _sort(seq, reverse=False, case_sensitive=False, attribute=None):
        g = _attr_getter(attribute) if attribute is not None else (lambda x: x)

        def key(x):
            v = g(x)
            return v.lower() if (isinstance(v, str) and not case_sensitive) else v
        return sorted(seq, key=key, reverse=reverse)

    @staticmethod
    def _unique(seq, case_sensitive=False, attribute=None):
        g = _attr_getter(attribute) if attribute is not None else (lambda x: x)
        seen, out = set(), []
        for x in seq:
            k = g(x)
            if isinstance(k, str) and not case_sensitive:
                k = k.lower()
            if k not in seen:
                seen.add(k); out.append(x)
        return out

    def _map(self, seq, *args, **kw):
        if "attribute" in kw:
            g = _attr_getter(kw["attribute"])
            d = kw.get("default")
            out = []
            for x in seq:
                v = g(x)
                out.append(d if (isinstance(v, Undefined) and d is not None) else v)
            return out
        if not args:
            return list(seq)
        f = self.filters[args[0]]
        return [f(x, *args[1:], **kw) for x in seq]

    def _select_f(self, keep, by_attr):
        def run(seq, *args, **kw):
            args = list(args)
            g = _attr_getter(args.pop(0)) if by_attr else (lambda x: x)
            if args:
                t = self.tests[args[0]]
                pred = lambda x: t(g(x), *args[1:])
            else:
                pred = lambda x: bool(g(x))
            return [x for x in seq if bool(pred(x)) == keep]
        return run

    @staticmethod
    def _sum(seq, attribute=None, start=0):
        g = _attr_getter(attribute) if attribute is not None else (lambda x: x)
        return sum((g(x) for x in seq), start)

    @staticmethod
    def _indent(s, width=4, first=False, blank=False):
        pad = " " * width if isinstance(width, int) else str(width)
        lines = _to_str(s).split("\n")
        out = []
        for i, ln in enumerate(lines):
            if (i == 0 and not first) or (not ln and not blank and i > 0):
                out.append(ln)
            else:
                out.append(pad + ln)
        return "\n".join(out)

    @staticmethod
    def _batch(seq, n, fill=None):
        seq = list(seq)
        out = [seq[i:i + n] for i in range(0, len(seq), n)]
        if out and fill is not None and len(out[-1]) < n:
            out[-1] += [fill] * (n - len(out[-1]))
        return out

    @staticmethod
    def _escape(s):
        return (_to_str(s).replace("&", "&amp;").replace("<", "&lt;").replace(">", "&gt;").replace("'", "&#39;").replace('"', "&#34;"))

    @staticmethod
    def _truncate(s, length=255, killwords=False, end="...", leeway=5):
        s = _to_str(s)
        if len(s) <= length + leeway:
            return s
        if killwords:
            return s[:length - len(end)] + end
        return s[:length - len(end)].rsplit(" ", 1)[0] + end

    @staticmethod
    def _groupby(seq, attribute):
        g = _attr_getter(attribute)
        groups = {}
        for x in seq:
            groups.setdefault(g(x), []).append(x)
        return sorted(groups.items(), key=lambda kv: _to_str(kv[0]))

    # -- expressions --
    def ev(self, n, sc):
        k = n[0]
        if k == "const":
            return n[1]
        if k == "name":
            for s in reversed(sc):
                if n[1] in s:
                    return s[n[1]]
            return Undefined(n[1])
        if k == "attr":
            return _getattr(self.ev(n[1], sc), n[2])
        if k == "item":
            obj = self.ev(n[1], sc)
            idx = n[2]
            if idx[0] == "slice":
                a, b, c = (None if p is None else self.ev(p, sc) for p in idx[1:])
                return Undefined() if isinstance(obj, Undefined) else obj[slice(a, b, c)]
            return _getitem(obj, self.ev(idx, sc))
        if k == "call":
            f = self.ev(n[1], sc)
            args = []
            for a in n[2]:
                if a[0] == "star":
                    args.extend(self.ev(a[1], sc))
                else:
                    args.append(self.ev(a, sc))
            kwargs = {kk: self.ev(v, sc) for kk, v in n[3]}
            if isinstance(f, Undefined):
                raise TemplateError(f"'{f.name}' is undefined")
            return f(*args, **kwargs)
        if k == "filter":
            f = self.filters.get(n[1])
            if f is None:
                raise TemplateError(f"no filter named '{n[1]}'")
            v = self.ev(n[2], sc)
            return f(v, *[self.ev(a, sc) for a in n[3]], **{kk: self.ev(x, sc) for kk, x in n[4]})
        if k == "test":
            t = self.tests.get(n[1])
            if t is None:
                raise TemplateError(f"no test named '{n[1]}'")
            return bool(t(self.ev(n[2], sc), *[self.ev(a, sc) for a in n[3]]))
        if k == "cond":
            return self.ev(n[2], sc) if self.ev(n[1], sc) else self.ev(n[3], sc)
        if k == "or":
            a = self.ev(n[1], sc)
            return a if a else self.ev(n[2], sc)
        if k == "and":
            a = self.ev(n[1], sc)
            return self.ev(n[2], sc) if a else a
        if k == "not":
            return not self.ev(n[1], sc)
        if k == "neg":
            return -self.ev(n[1], sc)
        if k == "in":
            a, b = self.ev(n[1], sc), self.ev(n[2], sc)
            if isinstance(b, Undefined):
                return False
            return a in b
        if k == "cmp":
            a, b = self.ev(n[2], sc), self.ev(n[3], sc)
            op = n[1]
            if op == "==":
                return a == b
            if op == "!=":
                return a != b
            if op == "<":
                return a < b
            if op == ">":
                return a > b
            if op == "<=":
                return a <= b
            return a >= b
        if k == "bin":
            a, b = self.ev(n[2], sc), self.ev(n[3], sc)
            op = n[1]
            if op == "~":
                return _to_str(a) + _to_str(b)
            if op == "+":
                if isinstance(a, Undefined) or isinstance(b, Undefined):
                    a = "" if isinstance(a, Undefined) and isinstance(b, str) else a
                    b = "" if isinstance(b, Undefined) and isinstance(a, str) else b
                return a + b
            if op == "-":
                return a - b
            if op == "*":
                return a * b
            if op == "/":
                return a / b
            if op == "//":
                return a // b
            if op == "%":
                return a % b
            return a ** b
        if k == "list":
            return [self.ev(x, sc) for x in n[1]]
        if k == "tuple":
            return tuple(self.ev(x, sc) for x in n[1])
        if k == "dict":
            return {self.ev(a, sc): self.ev(b, sc) for a, b in n[1]}
        raise TemplateError(f"bad node {k}")

    # -- statements --
    def run(self, body, sc, out):
        for n in body:
            k = n[0]
            if k == "data":
                out.append(n[1])
            elif k == "out":
                v = self.ev(n[1], sc)
                if not isinstance(v, Undefined):
                    out.append(_to_str(v))
            elif k == "if":
                for cond, b in n[1]:
                    if cond is None or self.ev(cond, sc):
                        self.run(b, sc, out)
                        break
            elif k == "for":
                self.run_for(n, sc, out)
            elif k == "set":
                val = self.ev(n[2], sc)
                names = n[1]
                if len(names) == 1:
                    self.assign(names[0], val, sc)
                else:
                    vals = list(val)
                    if len(vals) != len(names):
                        raise TemplateError("cannot unpack in set")
                    for t, v in zip(names, vals):
                        self.assign(t, v, sc)
            elif k == "setblock":
                buf = []
                self.run(n[2], sc + [{}], buf)
                val = "".join(buf)
                if n[3] is not None:
                    val = self.ev(n[3], sc + [{"\0body": val}])
                self.assign(n[1], val, sc)
            elif k == "macro":
                sc[-1][n[1]] = _Macro(self, n[1], n[2], n[3], list(sc))
            elif k == "filterblock":
                buf = []
                self.run(n[2], sc + [{}], buf)
                out.append(_to_str(self.ev(n[1], sc + [{"\0body": "".join(buf)}])))
            elif k == "group":
                self.run(n[1], sc, out)
            elif k == "callblock":
                call = n[1]
                if call[0] != "call":
                    raise TemplateError("call block needs a macro call")
                body = n[2]
                interp = self

                def caller(*a, _sc=list(sc)):
                    buf = []
                    interp.run(body, _sc + [{}], buf)
                    return "".join(buf)
                out.append(_to_str(self.ev(call, sc + [{"caller": caller}])))
            elif k == "do":
                self.ev(n[1], sc)
            elif k == "break":
                raise _Break()
            elif k == "continue":
                raise _Continue()
            else:
                raise TemplateError(f"bad statement {k}")

    @staticmethod
    def assign(target, val, sc):
        if target[0] == "nsattr":
            for s in reversed(sc):
                if target[1] in s:
                    ns = s[target[1]]
                    if not isinstance(ns, _Namespace):
                        raise TemplateError("attribute assignment needs a namespace object")
                    setattr(ns, target[2], val)
                    return
            raise TemplateError(f"'{target[1]}' is undefined")
        sc[-1][target[1]] = val

    def run_for(self, n, sc, out):
        _, targets, it, cond, body, orelse = n
        seq = self.ev(it, sc)
        if isinstance(seq, dict):
            seq = list(seq.keys())
        elif isinstance(seq, Undefined) or seq is None:
            seq = []
        else:
            seq = list(seq)

        def bind(frame, item):
            if len(targets) == 1:
                frame[targets[0]] = item
            else:
                vals = list(item)
                if len(vals) != len(targets):
                    raise TemplateError("cannot unpack loop item")
                for t, v in zip(targets, vals):
                    frame[t] = v

        if cond is not None:
            kept = []
            for item in seq:
                f = {}
                bind(f, item)
                if self.ev(cond, sc + [f]):
                    kept.append(item)
            seq = kept
        if not seq:
            self.run(orelse, sc + [{}], out)
            return
        depth = 1
        for s in reversed(sc):
            if "loop" in s and isinstance(s["loop"], _Loop):
                depth = s["loop"].depth + 1
                break
        loop = _Loop(len(seq), depth)
        for i, item in enumerate(seq):
            loop.index0 = i
            loop._prev = seq[i - 1] if i > 0 else Undefined()
            loop._next = seq[i + 1] if i + 1 < len(seq) else Undefined()
            frame = {"loop": loop}
            bind(frame, item)
            try:
                self.run(body, sc + [frame], out)
            except _Continue:
                continue
            except _Break:
                break


class _Macro:
    def __init__(self, interp, name, params, body, closure):
        self.interp, self.name, self.params, self.body, self.closure = interp, name, params, body, closure

    def __call__(self, *args, **kwargs):
        frame = {}
        caller = kwargs.pop("caller", None)
        for i, (pn, default) in enumerate(self.params):
            if i < len(args):
                frame[pn] = args[i]
            elif pn in kwargs:
                frame[pn] = kwargs.pop(pn)
            elif default is not None:
                frame[pn] = self.interp.ev(default, self.closure + [frame])
            else:
                frame[pn] = Undefined(pn)
        frame["varargs"] = list(args[len(self.params):])
        frame["kwargs"] = kwargs
        if caller is not None:
            frame["caller"] = caller
        out = []
        self.interp.run(self.body, self.closure + [frame], out)
        return "".join(out)


def _raise_exception(msg):
    raise TemplateError(msg)


def _namespace(*a, **kw):
    ns = _Namespace()
    for d in a:
        ns.__dict__.update(d)
    ns.__dict__.update(kw)
    return ns


class Template:
    """Compiled template: ``Template(source).render(**variables)``."""

    def __init__(self, source: str, trim_blocks: bool = True, lstrip_blocks: bool = True):
        self.body = _parse(_lex(source, trim_blocks, lstrip_blocks))
        self.interp = _Interp()

    def render(self, **variables) -> str:
        glob = {
            "raise_exception": _raise_exception, "namespace": _namespace, "range": lambda *a: list(range(*a)), "dict": dict,
            "strftime_now": lambda fmt: datetime.datetime.now().strftime(fmt), "lipsum": lambda *a, **k: "",
            "joiner": _joiner, "cycler": _cycler, "len": len, "str": _to_str, "int": int, "float": float, "list": list,
            "true": True, "false": False, "none": None,
        }
        out = []
        try:
            self.interp.run(self.body, [glob, dict(variables), {}], out)
        except (_Break, _Continue):
            raise TemplateError("break / continue outside a loop")
        return "".join(out)


def _joiner(sep=", "):
    state = {"first": True}

    def j():
        if state["first"]:
            state["first"] = False
            return ""
        return sep
    return j


def _cycler(*items):
    ns = _Namespace(items=items, pos=0)

    def nxt():
        v = items[ns.pos % len(items)]
        ns.pos += 1
        return v
    ns.next = nxt
    ns.reset = lambda: setattr(ns, "pos", 0)
    return ns


def render(source: str, **variables) -> str:
    return Template(source).render(**variables)
