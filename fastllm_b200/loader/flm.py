"""Reader / writer of the ``.flm`` model file, byte-compatible with the reference.

Layout (reference: WeightMap::LoadFromFile / SaveLowBitModel, src/fastllm.cpp:3189-3554; Python writer
tools/fastllm_pytools/torch2flm.py:33-103); all integers are little-endian int32, strings are
``int32 length + bytes``:

    int32 version (2)
    int32 n_kv, then n_kv x (string key, string value)          flattened config.json + tokenizer flags
    int32 vocab_len, then per token: int32 len, len x int32 (one per byte), int32 id [, float score]
    [int32 n_special + strings]                                   if "tokenizer_has_special_tokens" == "1"
    int32 n_tensors, then per tensor:
        string name, int32 ndims, dims..., int32 DataType, payload
        FLOAT32(0) / BFLOAT16(1) / FLOAT16(7): raw data
        INT8(3) / INT4(4):        int32 axis, k x (float min, float max), data   (zero-point form)
        INT4_NOZERO(8):           int32 axis, k x (float min, float max), data   (min form)
        INT4_GROUP(9):            int32 axis, int32 group, int32 groupCnt, k*group x (float min, float max), data
    4-bit data packs two values per byte, first value in the HIGH nibble.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

FLOAT32, BFLOAT16, INT8, INT4, FLOAT16, INT4_NOZERO, INT4_GROUP = 0, 1, 3, 4, 7, 8, 9


class _Reader:
    def __init__(self, path):
        self.buf = np.memmap(path, dtype=np.uint8, mode="r")
        self.pos = 0

    def i32(self):
        v = struct.unpack_from("<i", self.buf, self.pos)[0]
        self.pos += 4
        return v

    def f32(self):
        v = struct.unpack_from("<f", self.buf, self.pos)[0]
        self.pos += 4
        return v

    def string(self):
        n = self.i32()
        s = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        return s.decode("utf-8", errors="replace")

    def raw(self, n):
        a = self.buf[self.pos:self.pos + n]
        self.pos += n
        return a


def _unpack4(data: np.ndarray, shape):
    hi, lo = data >> 4, data & 0xF
    return np.stack([hi, lo], axis=-1).reshape(shape)


def read_flm(path: str | Path, dtype=torch.float32):
    """Returns (config dict, tokenizer dict, name -> dense tensor).  Quantised tensors are de-quantised."""
    r = _Reader(path)
    version = r.i32()
    cfg = {}
    if version >= 1:
        for _ in range(r.i32()):
            k = r.string()
            cfg[k] = r.string()
    use_score = cfg.get("tokenizer_use_score") == "1"
    vocab = []
    for i in range(r.i32()):
        n = r.i32()
        tok = bytes(int(x) & 0xFF for x in np.frombuffer(r.raw(4 * n), dtype="<i4"))
        tid = r.i32()
        score = r.f32() if use_score else float(-i)
        vocab.append((tok, tid, score))
    specials = []
    if cfg.get("tokenizer_has_special_tokens") == "1":
        specials = [r.string() for _ in range(r.i32())]
    tensors = {}
    for _ in range(r.i32()):
        name = r.string()
        dims = [r.i32() for _ in range(r.i32())]
        dt = r.i32()
        count = int(np.prod(dims)) if dims else 1
        if dt == FLOAT32:
            t = torch.from_numpy(np.frombuffer(r.raw(4 * count), dtype="<f4").copy()).reshape(dims)
        elif dt == FLOAT16:
            t = torch.from_numpy(np.frombuffer(r.raw(2 * count), dtype="<f2").copy()).reshape(dims)
        elif dt == BFLOAT16:
            t = torch.from_numpy(np.frombuffer(r.raw(2 * count), dtype="<i2").copy()).view(torch.bfloat16).reshape(dims)
        elif dt in (INT8, INT4, INT4_NOZERO):
            axis = r.i32()
            k = 1 if axis == -1 else dims[axis]
            mm = np.frombuffer(r.raw(8 * k), dtype="<f4").reshape(k, 2).astype(np.float64)
            bit = 8 if dt == INT8 else 4
            scale = np.maximum((mm[:, 1] - mm[:, 0]) / ((1 << bit) - 1), 1e-30)
            data = np.asarray(r.raw(count if bit == 8 else count // 2))
            q = data.reshape(dims) if bit == 8 else _unpack4(data, dims)
            if dt == INT4_NOZERO:
                w = q.astype(np.float32) * scale[:, None].astype(np.float32) + mm[:, 0][:, None].astype(np.float32)
            else:
                zero = np.clip(np.round(-mm[:, 0] / scale), 0, (1 << bit) - 1)
                w = (q.astype(np.float32) - zero[:, None].astype(np.float32)) * scale[:, None].astype(np.float32)
            t = torch.from_numpy(w.astype(np.float32))
        elif dt == INT4_GROUP:
            axis, group, group_cnt = r.i32(), r.i32(), r.i32()
            k = (1 if axis == -1 else dims[axis]) * group
            mm = np.frombuffer(r.raw(8 * k), dtype="<f4").reshape(dims[0], group, 2)
            data = np.asarray(r.raw(count // 2))
            q = _unpack4(data, dims).astype(np.float32)
            scale = (mm[..., 1] - mm[..., 0]) / 15.0
            sc = np.repeat(scale, group_cnt, axis=1)[:, :dims[1]]
            mn = np.repeat(mm[..., 0], group_cnt, axis=1)[:, :dims[1]]
            t = torch.from_numpy(q * sc + mn)
        else:
            raise ValueError(f"unsupported .flm tensor dtype {dt} for {name}")
        tensors[name] = t.to(dtype) if t.is_floating_point() and dt not in (FLOAT32,) else t
    return cfg, {"vocab": vocab, "special_tokens": specials}, tensors


# ---------------------------------------------------------------------------------------------------
class _Writer:
    def __init__(self, f):
        self.f = f

    def i32(self, v):
        self.f.write(struct.pack("<i", int(v)))

    def f32(self, v):
        self.f.write(struct.pack("<f", float(v)))

    def string(self, s):
        b = s.encode("utf-8") if isinstance(s, str) else s
        self.i32(len(b))
        self.f.write(b)


def _write_tensor(w: _Writer, name: str, t: torch.Tensor, kind: str, group_cnt: int = 128):
    w.string(name)
    dims = list(t.shape)
    w.i32(len(dims))
    for d in dims:
        w.i32(d)
    tf = t.float()
    if kind == "float32" or t.dim() != 2:
        w.i32(FLOAT32)
        w.f.write(tf.contiguous().numpy().astype("<f4").tobytes())
    elif kind == "float16":
        w.i32(FLOAT16)
        w.f.write(tf.half().contiguous().numpy().tobytes())
    elif kind == "bfloat16":
        w.i32(BFLOAT16)
        w.f.write(tf.bfloat16().contiguous().view(torch.int16).numpy().tobytes())
    elif kind == "int8":
        w.i32(INT8)
        w.i32(0)
        mn = tf.amin(1).clamp(max=0.0)
        mx = tf.amax(1).clamp(min=0.0)
        scale = ((mx - mn) / 255.0).clamp(min=1e-30)
        zero = torch.round(-mn / scale).clamp(0, 255)
        q = torch.round(tf / scale[:, None] + zero[:, None]).clamp(0, 255).to(torch.uint8)
        w.f.write(torch.stack([mn, mx], 1).numpy().astype("<f4").tobytes())
        w.f.write(q.numpy().tobytes())
    elif kind.startswith("int4g"):
        n, k = dims
        groups = (k + group_cnt - 1) // group_cnt
        pad = groups * group_cnt - k
        tp = torch.nn.functional.pad(tf, (0, pad), mode="replicate") if pad else tf
        g = tp.reshape(n, groups, group_cnt)
        mn, mx = g.amin(2), g.amax(2)
        scale = ((mx - mn) / 15.0).clamp(min=1e-30)
        q = torch.round((g - mn[..., None]) / scale[..., None]).clamp(0, 15).to(torch.uint8).reshape(n, groups * group_cnt)[:, :k]
        w.i32(INT4_GROUP)
        w.i32(0)
        w.i32(groups)
        w.i32(group_cnt)
        w.f.write(torch.stack([mn, mx], 2).numpy().astype("<f4").tobytes())
        w.f.write(((q[:, 0::2] << 4) | q[:, 1::2]).contiguous().numpy().tobytes())
    elif kind == "int4":
        w.i32(INT4_NOZERO)
        w.i32(0)
        mn, mx = tf.amin(1), tf.amax(1)
        scale = ((mx - mn) / 15.0).clamp(min=1e-30)
        q = torch.round((tf - mn[:, None]) / scale[:, None]).clamp(0, 15).to(torch.uint8)
        w.f.write(torch.stack([mn, mx], 1).numpy().astype("<f4").tobytes())
        w.f.write(((q[:, 0::2] << 4) | q[:, 1::2]).contiguous().numpy().tobytes())
    else:
        raise ValueError(f"unsupported export dtype {kind}")


def _flatten(d, prefix=""):
    out = {}
    for k, v in d.items():
        if isinstance(v, dict):
            out.update(_flatten(v, prefix + k + "."))
        elif isinstance(v, (list, tuple)):
            out[prefix + k] = json.dumps(list(v))
        elif isinstance(v, bool):
            out[prefix + k] = "true" if v else "false"
        elif v is not None:
            out[prefix + k] = str(v)
    return out


def write_flm(path, config: dict, vocab, specials, tensors, dtype: str = "float16", chat_template: str | None = None):
    """``vocab``: iterable of (token bytes, id, score); ``tensors``: iterable of (name, tensor).  2-D weights whose
    name ends in ``.weight`` (except embeddings / norms / lm_head) are stored in ``dtype``; the rest as float32 / fp16."""
    kv = _flatten(config)
    vocab = list(vocab)
    kv["tokenizer_use_score"] = "1"
    if specials:
        kv["tokenizer_has_special_tokens"] = "1"
    if chat_template:
        kv["chat_template"] = chat_template
    with open(path, "wb") as f:
        w = _Writer(f)
        w.i32(2)
        w.i32(len(kv))
        for k, v in kv.items():
            w.string(k)
            w.string(v)
        w.i32(len(vocab))
        for tok, tid, score in vocab:
            w.i32(len(tok))
            f.write(np.asarray(list(tok), dtype="<i4").tobytes())
            w.i32(tid)
            w.f32(score)
        if specials:
            w.i32(len(specials))
            for s in specials:
                w.string(s)
        tensors = list(tensors)
        w.i32(len(tensors))
        for name, t in tensors:
            lin = t.dim() == 2 and name.endswith(".weight") and not any(x in name for x in ("embed", "norm", "lm_head", "mlp.gate.weight"))
            kind = dtype if lin else ("float16" if (t.dim() == 2 and dtype != "float32") else "float32")
            if lin and dtype.startswith("int4g"):
                _write_tensor(w, name, t, dtype, int(dtype[5:] or 128))
            else:
                _write_tensor(w, name, t, kind)


def export_hf_to_flm(hf_dir: str, out_path: str, dtype: str = "float16"):
    """Convert an HF folder to ``.flm`` (reference: ``ftllm export`` / torch2flm.tofile)."""
    from ..tokenizer import Tokenizer
    from . import safetensors as st

    hf_dir = Path(hf_dir)
    config = json.loads((hf_dir / "config.json").read_text())
    tok = Tokenizer(hf_dir, prefer_native=True)
    vocab, specials = [], []
    tj = hf_dir / "tokenizer.json"
    if tj.exists():
        t = json.loads(tj.read_text(encoding="utf-8"))
        nb = tok.native
        for token, tid in t.get("model", {}).get("vocab", {}).items():
            raw = nb.decode_bytes([tid], skip_special_tokens=False) if nb is not None else token.encode("utf-8")
            vocab.append((raw, tid, 1.0))
        for a in t.get("added_tokens", []):
            vocab.append((a["content"].encode("utf-8"), a["id"], 1.0))
            specials.append(a["content"])
        config["tokenizer_byte_as_char"] = "True"
    files, where = st.open_model_dir(hf_dir)
    names = sorted(where.keys())
    write_flm(out_path, config, vocab, specials, ((n, files[where[n]].get(n)) for n in names), dtype, tok.chat_template)
    for f in files:
        f.close()


def load_model(path: str, device="cuda", dtype=None, wdtype: str = "auto", tp=None):
    """Load a ``.flm`` file into a ``DecoderModel``."""
    from ..models.config import from_hf_dict
    from ..models.decoder import DecoderModel
    from .hf import canonical_name
    from .shard import finalize_model

    cfg_kv, _tok, tensors = read_flm(path, torch.float32)
    raw = {}
    for k, v in cfg_kv.items():          # un-flatten what the model config needs; values come back as strings
        cur = raw
        parts = k.split(".")
        for p in parts[:-1]:
            cur = cur.setdefault(p, {}) if isinstance(cur.get(p, {}), dict) else cur
        try:
            cur[parts[-1]] = json.loads(v)
        except Exception:
            cur[parts[-1]] = v
    cfg = from_hf_dict(raw)
    if dtype is None:
        dtype = torch.float32 if str(device) == "cpu" else torch.bfloat16
    m = DecoderModel(cfg, device, dtype, tp)
    sd = {canonical_name(k): v for k, v in tensors.items()}
    finalize_model(m, lambda: {k: v for k, v in sd.items() if not k.startswith("model.layers.")},
                   lambda i: {k: v for k, v in sd.items() if k.startswith(f"model.layers.{i}.")},
                   wdtype="dense" if wdtype == "auto" else wdtype)
    return m


def save_model(torch_model, tokenizer, path: str, dtype: str = "float16"):
    src = getattr(torch_model, "source_path", None)
    if not src:
        raise ValueError("saving needs the original HF folder: use export_hf_to_flm(hf_dir, out_path, dtype)")
    export_hf_to_flm(src, path, dtype)
