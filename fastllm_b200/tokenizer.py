"""Tokenizer front end.

Order of preference, like the reference's Python layer (tools/fastllm_pytools/llm.py:1947-2070): the Hugging
Face tokenizer of the model folder when ``transformers`` / ``tokenizers`` can load it, else the native byte-level
BPE core (``csrc/runtime/bpe.cpp``) fed from ``tokenizer.json``.  Streaming decode holds back bytes that end in
an incomplete UTF-8 sequence (the U+FFFD hold-back of the reference).
"""
from __future__ import annotations

import ctypes
import json
from pathlib import Path

from .ops import _lib


class NativeBPE:
    """ctypes wrapper over the C++ byte-level BPE."""

    def __init__(self, tokenizer_json: str | Path | dict):
        L = _lib.runtime()
        L.fbtok_create.restype = ctypes.c_void_p
        L.fbtok_destroy.argtypes = [ctypes.c_void_p]
        L.fbtok_add_token.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        L.fbtok_add_merge.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
        L.fbtok_add_special.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        L.fbtok_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
        L.fbtok_decode.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        L.fbtok_vocab_size.argtypes = [ctypes.c_void_p]
        self.L = L
        self.h = ctypes.c_void_p(L.fbtok_create())
        tj = tokenizer_json if isinstance(tokenizer_json, dict) else json.loads(Path(tokenizer_json).read_text(encoding="utf-8"))
        model = tj.get("model", {})
        for tok, i in model.get("vocab", {}).items():
            b = tok.encode("utf-8")
            L.fbtok_add_token(self.h, b, len(b), int(i))
        for m in model.get("merges", []):
            l, r = (m.split(" ", 1) if isinstance(m, str) else m)
            lb, rb = l.encode("utf-8"), r.encode("utf-8")
            L.fbtok_add_merge(self.h, lb, len(lb), rb, len(rb))
        L.fbtok_set_pretokenizer.argtypes = [ctypes.c_void_p, ctypes.c_int]
        pre = json.dumps(tj.get("pre_tokenizer") or {})
        # Llama-3 / Qwen style patterns cap digit runs at three; everything else is treated as the GPT-2 pattern
        L.fbtok_set_pretokenizer(self.h, 0 if "{1,3}" in pre else 1)
        self.special = {}
        for a in tj.get("added_tokens", []):
            b = a["content"].encode("utf-8")
            L.fbtok_add_special(self.h, b, len(b), int(a["id"]))
            self.special[a["content"]] = int(a["id"])

    def __del__(self):
        try:
            self.L.fbtok_destroy(self.h)
        except Exception:
            pass

    def encode(self, text: str) -> list[int]:
        b = text.encode("utf-8")
        cap = max(16, len(b) + 8)
        out = (ctypes.c_int * cap)()
        n = self.L.fbtok_encode(self.h, b, len(b), out, cap)
        if n < 0:
            cap = -n
            out = (ctypes.c_int * cap)()
            n = self.L.fbtok_encode(self.h, b, len(b), out, cap)
        return list(out[:n])

    def decode_bytes(self, ids, skip_special_tokens=True) -> bytes:
        arr = (ctypes.c_int * len(ids))(*ids)
        cap = max(64, len(ids) * 16)
        buf = ctypes.create_string_buffer(cap)
        n = self.L.fbtok_decode(self.h, arr, len(ids), buf, cap, 1 if skip_special_tokens else 0)
        if n < 0:
            cap = -n
            buf = ctypes.create_string_buffer(cap)
            n = self.L.fbtok_decode(self.h, arr, len(ids), buf, cap, 1 if skip_special_tokens else 0)
        return buf.raw[:n]

    def decode(self, ids, skip_special_tokens=True) -> str:
        return self.decode_bytes(ids, skip_special_tokens).decode("utf-8", errors="replace")

    @property
    def vocab_size(self):
        return self.L.fbtok_vocab_size(self.h)


class NativeUnigram:
    """ctypes wrapper over the C++ Unigram core (``csrc/runtime/unigram.cpp``): the SentencePiece-style models of
    ``tokenizer.json`` (``model.type == "Unigram"``: T5, ALBERT, XLM-R, older Llama / Gemma exports).  The Metaspace
    convention is applied here: spaces become U+2581 before segmentation (with a leading one unless the file says
    otherwise) and back to spaces after decoding."""

    SPACE = "\u2581"

    def __init__(self, tokenizer_json: str | Path | dict):
        L = _lib.runtime()
        L.fbuni_create.restype = ctypes.c_void_p
        L.fbuni_destroy.argtypes = [ctypes.c_void_p]
        L.fbuni_add_piece.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_float]
        L.fbuni_finish.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        L.fbuni_add_special.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        L.fbuni_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
        L.fbuni_decode.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
        L.fbuni_vocab_size.argtypes = [ctypes.c_void_p]
        self.L = L
        self.h = ctypes.c_void_p(L.fbuni_create())
        tj = tokenizer_json if isinstance(tokenizer_json, dict) else json.loads(Path(tokenizer_json).read_text(encoding="utf-8"))
        model = tj.get("model", {})
        for piece, score in model.get("vocab", []):
            b = piece.encode("utf-8")
            L.fbuni_add_piece(self.h, b, len(b), float(score))
        L.fbuni_finish(self.h, int(model.get("unk_id") or 0), 1 if model.get("byte_fallback") else 0)
        self.special = {}
        for a in tj.get("added_tokens", []):
            b = a["content"].encode("utf-8")
            L.fbuni_add_special(self.h, b, len(b), int(a["id"]))
            self.special[a["content"]] = int(a["id"])
        pre = tj.get("pre_tokenizer") or {}
        metas = [pre] + list(pre.get("pretokenizers", [])) if isinstance(pre, dict) else []
        meta = next((m for m in metas if m.get("type") == "Metaspace"), {})
        scheme = meta.get("prepend_scheme", "always" if meta.get("add_prefix_space", True) else "never")
        self.prepend = scheme in ("always", "first")

    def __del__(self):
        try:
            self.L.fbuni_destroy(self.h)
        except Exception:
            pass

    def encode(self, text: str) -> list[int]:
        t = text.replace(" ", self.SPACE)
        if self.prepend and not t.startswith(self.SPACE):
            t = self.SPACE + t
        b = t.encode("utf-8")
        cap = max(16, len(b) + 8)
        out = (ctypes.c_int * cap)()
        n = self.L.fbuni_encode(self.h, b, len(b), out, cap)
        if n < 0:
            cap = -n
            out = (ctypes.c_int * cap)()
            n = self.L.fbuni_encode(self.h, b, len(b), out, cap)
        return list(out[:n])

    def decode_bytes(self, ids, skip_special_tokens=True) -> bytes:
        arr = (ctypes.c_int * len(ids))(*ids)
        cap = max(64, len(ids) * 24)
        buf = ctypes.create_string_buffer(cap)
        n = self.L.fbuni_decode(self.h, arr, len(ids), buf, cap, 1 if skip_special_tokens else 0)
        if n < 0:
            cap = -n
            buf = ctypes.create_string_buffer(cap)
            n = self.L.fbuni_decode(self.h, arr, len(ids), buf, cap, 1 if skip_special_tokens else 0)
        return buf.raw[:n]

    def decode(self, ids, skip_special_tokens=True) -> str:
        s = self.decode_bytes(ids, skip_special_tokens).decode("utf-8", errors="replace").replace(self.SPACE, " ")
        return s[1:] if (self.prepend and s.startswith(" ")) else s

    @property
    def vocab_size(self):
        return self.L.fbuni_vocab_size(self.h)


def native_tokenizer(tokenizer_json: str | Path | dict):
    """The native core that matches the file's model type (byte-level BPE or Unigram)."""
    tj = tokenizer_json if isinstance(tokenizer_json, dict) else json.loads(Path(tokenizer_json).read_text(encoding="utf-8"))
    return NativeUnigram(tj) if (tj.get("model") or {}).get("type") == "Unigram" else NativeBPE(tj)


class Tokenizer:
    """Uniform interface: encode / decode / apply_chat_template / streaming decode."""

    def __init__(self, path: str | Path | None = None, prefer_native: bool = False, chat_template: str | None = None):
        self.path = Path(path) if path else None
        self.hf = None
        self.native = None
        self.config = {}
        self.chat_template = chat_template
        if self.path is not None:
            cfg = self.path / "tokenizer_config.json"
            if cfg.exists():
                self.config = json.loads(cfg.read_text(encoding="utf-8"))
                self.chat_template = self.chat_template or self.config.get("chat_template")
            jt = self.path / "chat_template.jinja"
            if self.chat_template is None and jt.exists():
                self.chat_template = jt.read_text(encoding="utf-8")
            if not prefer_native:
                try:
                    from transformers import AutoTokenizer

                    self.hf = AutoTokenizer.from_pretrained(str(self.path), trust_remote_code=False)
                except Exception:
                    self.hf = None
            if self.hf is None and (self.path / "tokenizer.json").exists():
                self.native = native_tokenizer(self.path / "tokenizer.json")
        if isinstance(self.chat_template, list):       # some configs store named templates
            self.chat_template = next((t["template"] for t in self.chat_template if t.get("name") == "default"),
                                      self.chat_template[0]["template"])

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        if self.hf is not None:
            return self.hf.encode(text, add_special_tokens=add_special_tokens)
        if self.native is not None:
            return self.native.encode(text)
        return list(text.encode("utf-8"))

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        if self.hf is not None:
            return self.hf.decode(ids, skip_special_tokens=skip_special_tokens)
        if self.native is not None:
            return self.native.decode(ids, skip_special_tokens)
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    def vocab_size(self) -> int:
        if self.hf is not None:
            return len(self.hf)
        if self.native is not None:
            return int(self.native.vocab_size)
        return 256

    def eos_ids(self) -> list[int]:
        out = []
        if self.hf is not None and self.hf.eos_token_id is not None:
            out.append(self.hf.eos_token_id)
        elif self.native is not None:
            e = self.config.get("eos_token")
            e = e.get("content") if isinstance(e, dict) else e
            if e in self.native.special:
                out.append(self.native.special[e])
        return out

    def apply_chat_template(self, messages, add_generation_prompt=True, tools=None, **kw) -> str:
        from .chat_template import render

        tok_vars = {}
        for k in ("bos_token", "eos_token", "pad_token", "unk_token"):
            v = self.config.get(k)
            tok_vars[k] = v.get("content") if isinstance(v, dict) else (v or "")
        return render(self.chat_template, messages, add_generation_prompt=add_generation_prompt, tools=tools, **tok_vars, **kw)


class StreamDecoder:
    """Incremental detokenisation: emits only complete UTF-8 text, re-decoding a short tail window."""

    def __init__(self, tok: Tokenizer, skip_special_tokens: bool = True):
        self.tok, self.skip = tok, skip_special_tokens
        self.ids: list[int] = []
        self.emitted = 0          # characters of decode(self.ids) already returned
        self.prefix_ids = 0       # ids before this index are final (their text has been emitted)

    def push(self, token_id: int) -> str:
        self.ids.append(token_id)
        window = self.ids[self.prefix_ids:]
        text = self.tok.decode(window, self.skip)
        if text.endswith("�"):
            return ""             # incomplete multi-byte sequence: wait for the next token
        out = text[self.emitted:]
        self.emitted = len(text)
        if len(window) > 16:      # slide the window, keeping a few tokens of context for merge-sensitive decoders
            keep = 4
            base = self.tok.decode(self.ids[len(self.ids) - keep:], self.skip)
            self.prefix_ids = len(self.ids) - keep
            self.emitted = len(base)
        return out
