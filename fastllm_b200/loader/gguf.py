"""GGUF reader (v2 / v3): metadata, tensor directory, block de-quantisation, and model construction.

The reference loads GGUF through its vendored ggml tables and keeps the k-quant blocks for dp4a GEMV kernels
(src/model.cpp:2663+, src/devices/cuda/linear/fastllm-ggml-cuda.cu).  Here GGUF weights are de-quantised at load time to
the model dtype (or re-quantised to one of the tensor-core formats with ``wdtype``): no GGUF GEMM kernel exists.
``ori`` names a Hugging Face folder supplying ``config.json`` / tokenizer, like the reference's ``--ori`` flag; without it
the configuration is rebuilt from the GGUF metadata keys.

File layout: magic "GGUF", uint32 version, uint64 n_tensors, uint64 n_kv, the key/value list, the tensor directory
(name, n_dims, dims (innermost first), ggml type, offset), padding to ``general.alignment`` (default 32), tensor data.
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np
import torch

GGUF_MAGIC = 0x46554747
# value types of the metadata list
_U8, _I8, _U16, _I16, _U32, _I32, _F32, _BOOL, _STR, _ARR, _U64, _I64, _F64 = range(13)
_SCALAR = {_U8: "<B", _I8: "<b", _U16: "<H", _I16: "<h", _U32: "<I", _I32: "<i", _F32: "<f", _BOOL: "<?", _U64: "<Q", _I64: "<q", _F64: "<d"}

# ggml tensor types: id -> (name, values per block, bytes per block)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24),
    8: ("Q8_0", 32, 34), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176),
    14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 30: ("BF16", 1, 2),
}
TYPE_ID = {v[0]: k for k, v in GGML_TYPES.items()}


class GGUFFile:
    """Parsed header of one GGUF file; tensors are de-quantised lazily from a memory map."""

    def __init__(self, path: str | Path):
        self.path = str(path)
        self.buf = np.memmap(self.path, dtype=np.uint8, mode="r")
        self.pos = 0
        magic, self.version = self._unpack("<II")
        if magic != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        if self.version < 2:
            raise ValueError(f"{path}: GGUF version {self.version} is not supported (need >= 2)")
        n_tensors, n_kv = self._unpack("<QQ")
        self.meta: dict = {}
        for _ in range(n_kv):
            key = self._string()
            (vt,) = self._unpack("<I")
            self.meta[key] = self._value(vt)
        self.tensors: dict = {}
        for _ in range(n_tensors):
            name = self._string()
            (nd,) = self._unpack("<I")
            dims = self._unpack("<" + "Q" * nd)
            ttype, off = self._unpack("<IQ")
            self.tensors[name] = {"shape": tuple(reversed(dims)), "type": ttype, "offset": off}
        align = int(self.meta.get("general.alignment", 32))
        self.data_start = (self.pos + align - 1) // align * align

    # ---- low-level readers ----
    def _unpack(self, fmt):
        v = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += struct.calcsize(fmt)
        return v

    def _string(self):
        (n,) = self._unpack("<Q")
        s = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        return s.decode("utf-8", errors="replace")

    def _value(self, vt):
        if vt in _SCALAR:
            return self._unpack(_SCALAR[vt])[0]
        if vt == _STR:
            return self._string()
        if vt == _ARR:
            et, n = self._unpack("<IQ")
            if et in _SCALAR:
                fmt = _SCALAR[et]
                size = struct.calcsize(fmt)
                arr = np.frombuffer(self.buf[self.pos:self.pos + size * n], dtype=np.dtype(fmt)).copy()
                self.pos += size * n
                return arr
            return [self._value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {vt}")

    # ---- tensors ----
    def tensor(self, name: str, dtype=torch.float32) -> torch.Tensor:
        info = self.tensors[name]
        tname, per, nbytes = GGML_TYPES[info["type"]]
        n = int(np.prod(info["shape"]))
        size = n // per * nbytes
        start = self.data_start + info["offset"]
        raw = np.asarray(self.buf[start:start + size])
        arr = dequantize(raw, tname, n)
        return torch.from_numpy(arr.reshape(info["shape"])).to(dtype)


def _f16(a: np.ndarray) -> np.ndarray:
    return a.view("<f2").astype(np.float32)


def dequantize(raw: np.ndarray, tname: str, n: int) -> np.ndarray:
    """ggml block formats -> fp32 (flat).  Layouts follow the public ggml block definitions."""
    if tname == "F32":
        return raw.view("<f4").astype(np.float32)
    if tname == "F16":
        return _f16(raw)
    if tname == "BF16":
        return (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
    if tname in ("I8", "I16", "I32"):
        return raw.view({"I8": "i1", "I16": "<i2", "I32": "<i4"}[tname]).astype(np.float32)
    per, nbytes = next((p, b) for k, (t, p, b) in GGML_TYPES.items() if t == tname)
    blk = raw.reshape(-1, nbytes)
    if tname == "Q8_0":                      # fp16 d, 32 x int8
        d = _f16(blk[:, :2].copy()).reshape(-1, 1)
        return (d * blk[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)
    if tname in ("Q4_0", "Q4_1"):            # low nibbles are values 0..15, high nibbles values 16..31
        hdr = 2 if tname == "Q4_0" else 4
        d = _f16(blk[:, :2].copy()).reshape(-1, 1)
        q = blk[:, hdr:]
        v = np.concatenate([q & 0xF, q >> 4], axis=1).astype(np.float32)
        if tname == "Q4_0":
            return (d * (v - 8.0)).reshape(-1)
        m = _f16(blk[:, 2:4].copy()).reshape(-1, 1)
        return (d * v + m).reshape(-1)
    if tname in ("Q5_0", "Q5_1"):
        hdr = 2 if tname == "Q5_0" else 4
        d = _f16(blk[:, :2].copy()).reshape(-1, 1)
        qh = blk[:, hdr:hdr + 4].copy().view("<u4").reshape(-1, 1)
        q = blk[:, hdr + 4:]
        bits = ((qh >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8)
        v = np.concatenate([q & 0xF, q >> 4], axis=1) | (bits << 4)
        if tname == "Q5_0":
            return (d * (v.astype(np.float32) - 16.0)).reshape(-1)
        m = _f16(blk[:, 2:4].copy()).reshape(-1, 1)
        return (d * v.astype(np.float32) + m).reshape(-1)
    if tname == "Q8_K":
        d = blk[:, :4].copy().view("<f4").reshape(-1, 1)
        return (d * blk[:, 4:260].view(np.int8).astype(np.float32)).reshape(-1)
    return _dequant_k(blk, tname)


def _scale_min_k4(sc: np.ndarray):
    """12 packed bytes -> 8 six-bit scales and 8 six-bit mins (Q4_K / Q5_K)."""
    sc = sc.astype(np.uint8)
    d = np.empty((sc.shape[0], 8), dtype=np.float32)
    m = np.empty((sc.shape[0], 8), dtype=np.float32)
    d[:, :4] = sc[:, 0:4] & 63
    m[:, :4] = sc[:, 4:8] & 63
    d[:, 4:] = (sc[:, 8:12] & 0xF) | ((sc[:, 0:4] >> 6) << 4)
    m[:, 4:] = (sc[:, 8:12] >> 4) | ((sc[:, 4:8] >> 6) << 4)
    return d, m


def _dequant_k(blk: np.ndarray, tname: str) -> np.ndarray:
    nb = blk.shape[0]
    if tname in ("Q4_K", "Q5_K"):
        d = _f16(blk[:, 0:2].copy()).reshape(nb, 1)
        dmin = _f16(blk[:, 2:4].copy()).reshape(nb, 1)
        sc, mn = _scale_min_k4(blk[:, 4:16])
        if tname == "Q4_K":
            qs = blk[:, 16:144].reshape(nb, 4, 32)
            v = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)
        else:
            qh = blk[:, 16:48].reshape(nb, 1, 32)
            qs = blk[:, 48:176].reshape(nb, 4, 32)
            lo, hi = qs & 0xF, qs >> 4
            bit_lo = (qh >> (2 * np.arange(4, dtype=np.uint8)).reshape(1, 4, 1)) & 1
            bit_hi = (qh >> (2 * np.arange(4, dtype=np.uint8) + 1).reshape(1, 4, 1)) & 1
            v = np.stack([lo | (bit_lo << 4), hi | (bit_hi << 4)], axis=2).reshape(nb, 8, 32).astype(np.float32)
        out = (d * sc).reshape(nb, 8, 1) * v - (dmin * mn).reshape(nb, 8, 1)
        return out.reshape(-1)
    if tname == "Q6_K":
        ql = blk[:, 0:128].reshape(nb, 2, 64)
        qh = blk[:, 128:192].reshape(nb, 2, 32)
        sc = blk[:, 192:208].view(np.int8).astype(np.float32).reshape(nb, 2, 8)
        d = _f16(blk[:, 208:210].copy()).reshape(nb, 1, 1)
        q1 = (ql[:, :, :32] & 0xF) | (((qh >> 0) & 3) << 4)
        q2 = (ql[:, :, 32:] & 0xF) | (((qh >> 2) & 3) << 4)
        q3 = (ql[:, :, :32] >> 4) | (((qh >> 4) & 3) << 4)
        q4 = (ql[:, :, 32:] >> 4) | (((qh >> 6) & 3) << 4)
        q = np.stack([q1, q2, q3, q4], axis=2).astype(np.float32) - 32.0          # [nb, 2, 4, 32]
        # scale index = (l / 16) + 2 * quarter within each 128-value half
        scl = sc.reshape(nb, 2, 4, 2)
        scl = np.repeat(scl, 16, axis=3)                                            # [nb, 2, 4, 32]
        return (d.reshape(nb, 1, 1, 1) * scl * q).reshape(-1)
    if tname == "Q2_K":
        scales = blk[:, 0:16]
        qs = blk[:, 16:80].reshape(nb, 2, 1, 32)
        d = _f16(blk[:, 80:82].copy()).reshape(nb, 1)
        dmin = _f16(blk[:, 82:84].copy()).reshape(nb, 1)
        shifts = (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)
        q = ((qs >> shifts) & 3).astype(np.float32)                                # [nb, 2, 4, 32]
        dl = (d * (scales & 0xF).astype(np.float32)).reshape(nb, 2, 4, 2)
        ml = (dmin * (scales >> 4).astype(np.float32)).reshape(nb, 2, 4, 2)
        return (np.repeat(dl, 16, axis=3) * q - np.repeat(ml, 16, axis=3)).reshape(-1)
    if tname == "Q3_K":
        hm = blk[:, 0:32].reshape(nb, 1, 1, 32)
        qs = blk[:, 32:96].reshape(nb, 2, 1, 32)
        aux = blk[:, 96:108].copy().view("<u4").reshape(nb, 3).astype(np.uint32)
        d = _f16(blk[:, 108:110].copy()).reshape(nb, 1, 1, 1)
        k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
        tmp = aux[:, 2]
        a = np.empty((nb, 4), dtype=np.uint32)
        a[:, 0] = (aux[:, 0] & k2) | (((tmp >> 0) & k1) << 4)
        a[:, 1] = (aux[:, 1] & k2) | (((tmp >> 2) & k1) << 4)
        a[:, 2] = ((aux[:, 0] >> 4) & k2) | (((tmp >> 4) & k1) << 4)
        a[:, 3] = ((aux[:, 1] >> 4) & k2) | (((tmp >> 6) & k1) << 4)
        sc = a.view(np.uint8).reshape(nb, 16).view(np.int8).astype(np.float32) - 32.0
        shifts = (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)
        q = ((qs >> shifts) & 3).astype(np.float32)                                # [nb, 2, 4, 32]
        mbit = (np.arange(8, dtype=np.uint8)).reshape(1, 2, 4, 1)                  # mask bit = 4 * half + shift index
        hbit = (hm >> mbit) & 1
        q = q - np.where(hbit != 0, 0.0, 4.0)
        scl = np.repeat(sc.reshape(nb, 2, 4, 2), 16, axis=3)
        return (d * scl * q).reshape(-1)
    raise NotImplementedError(f"GGUF tensor type {tname} is not supported")


# GGUF tensor names -> canonical (Hugging Face llama-style) names
_TOP = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight", "output.weight": "lm_head.weight"}
_BLK = {
    "attn_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
    "attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight", "attn_v.weight": "self_attn.v_proj.weight",
    "attn_q.bias": "self_attn.q_proj.bias", "attn_k.bias": "self_attn.k_proj.bias", "attn_v.bias": "self_attn.v_proj.bias",
    "attn_output.weight": "self_attn.o_proj.weight", "attn_q_norm.weight": "self_attn.q_norm.weight",
    "attn_k_norm.weight": "self_attn.k_norm.weight", "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight", "ffn_gate_inp.weight": "mlp.gate.weight",
    "ffn_gate_shexp.weight": "mlp.shared_expert.gate_proj.weight", "ffn_up_shexp.weight": "mlp.shared_expert.up_proj.weight",
    "ffn_down_shexp.weight": "mlp.shared_expert.down_proj.weight", "ffn_gate_inp_shexp.weight": "mlp.shared_expert_gate.weight",
}
_EXPERT = {"ffn_gate_exps.weight": "gate_proj", "ffn_up_exps.weight": "up_proj", "ffn_down_exps.weight": "down_proj"}
_ARCH_TO_HF = {"llama": "llama", "qwen2": "qwen2", "qwen3": "qwen3", "qwen2moe": "qwen2_moe", "qwen3moe": "qwen3_moe",
               "internlm2": "llama", "baichuan": "llama", "mistral": "llama", "gemma": "gemma", "gemma2": "gemma2", "phi3": "phi3"}


def config_from_meta(meta: dict) -> dict:
    """GGUF metadata -> a ``config.json``-style dictionary."""
    arch = meta.get("general.architecture", "llama")
    g = lambda k, d=None: meta.get(f"{arch}.{k}", d)
    heads = int(g("attention.head_count", 32))
    hidden = int(g("embedding_length", 4096))
    cfg = {
        "model_type": _ARCH_TO_HF.get(arch, arch), "hidden_size": hidden, "num_hidden_layers": int(g("block_count", 32)),
        "num_attention_heads": heads, "num_key_value_heads": int(g("attention.head_count_kv", heads)),
        "intermediate_size": int(g("feed_forward_length", 4 * hidden)), "rms_norm_eps": float(g("attention.layer_norm_rms_epsilon", 1e-6)),
        "rope_theta": float(g("rope.freq_base", 10000.0)), "max_position_embeddings": int(g("context_length", 8192)),
        "head_dim": int(g("attention.key_length", hidden // heads)),
    }
    toks = meta.get("tokenizer.ggml.tokens")
    cfg["vocab_size"] = int(g("vocab_size", len(toks) if toks is not None else 32000))
    if g("expert_count"):
        cfg["num_experts"] = int(g("expert_count"))
        cfg["num_experts_per_tok"] = int(g("expert_used_count", 2))
        cfg["moe_intermediate_size"] = int(g("expert_feed_forward_length", cfg["intermediate_size"]))
        if g("expert_shared_feed_forward_length"):
            cfg["shared_expert_intermediate_size"] = int(g("expert_shared_feed_forward_length"))
    if g("rope.scaling.type") in ("linear", "yarn"):
        cfg["rope_scaling"] = {"type": g("rope.scaling.type"), "factor": float(g("rope.scaling.factor", 1.0)),
                               "original_max_position_embeddings": int(g("rope.scaling.original_context_length", cfg["max_position_embeddings"]))}
    if "tokenizer.ggml.eos_token_id" in meta:
        cfg["eos_token_id"] = int(meta["tokenizer.ggml.eos_token_id"])
    if "tokenizer.ggml.bos_token_id" in meta:
        cfg["bos_token_id"] = int(meta["tokenizer.ggml.bos_token_id"])
    return cfg


def _unpermute_rope(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """llama.cpp stores llama-architecture Q/K rows in interleaved-pair order; restore the half-split (neox) order."""
    rows = w.shape[0]
    hd = rows // n_head
    return w.reshape(n_head, hd // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def canonical_tensors(f: GGUFFile, cfg, dtype=torch.float32):
    """name -> tensor under the canonical names the shard builder consumes."""
    arch = f.meta.get("general.architecture", "llama")
    permuted = arch in ("llama", "baichuan", "internlm2", "mistral")
    out = {}
    for name in f.tensors:
        if name in _TOP:
            out[_TOP[name]] = f.tensor(name, dtype)
            continue
        if not name.startswith("blk."):
            continue
        _, idx, rest = name.split(".", 2)
        p = f"model.layers.{idx}."
        if rest in _EXPERT:
            w = f.tensor(name, dtype)                      # [n_expert, out, in]
            for e in range(w.shape[0]):
                out[f"{p}mlp.experts.{e}.{_EXPERT[rest]}.weight"] = w[e]
        elif rest in _BLK:
            w = f.tensor(name, dtype)
            if permuted and rest in ("attn_q.weight", "attn_q.bias"):
                w = _unpermute_rope(w, cfg.num_heads)
            elif permuted and rest in ("attn_k.weight", "attn_k.bias"):
                w = _unpermute_rope(w, cfg.num_kv_heads)
            out[p + _BLK[rest]] = w
    return out


def tokenizer_json_from_meta(meta: dict) -> dict | None:
    """Byte-level BPE ``tokenizer.json`` dictionary from the GGUF vocabulary (model ``gpt2``); None for other kinds."""
    if meta.get("tokenizer.ggml.model") != "gpt2" or "tokenizer.ggml.tokens" not in meta:
        return None
    toks = meta["tokenizer.ggml.tokens"]
    types = meta.get("tokenizer.ggml.token_type")
    added = []
    if types is not None:
        for i, t in enumerate(types):
            if int(t) in (3, 4):                          # control / user-defined
                added.append({"id": i, "content": toks[i], "special": int(t) == 3})
    pre = meta.get("tokenizer.ggml.pre", "")
    return {"model": {"type": "BPE", "vocab": {t: i for i, t in enumerate(toks)}, "merges": list(meta.get("tokenizer.ggml.merges", []))},
            "added_tokens": added,
            # digit runs are capped at three ("{1,3}") by every pre-tokenizer llama.cpp names except the GPT-2 one
            "pre_tokenizer": {"type": "ByteLevel", "gguf_pre": pre, "digits": "" if pre in ("", "default", "gpt-2") else "{1,3}"}}


def load_model(path: str, device="cuda", dtype=None, ori: str | None = None, wdtype: str = "auto", tp=None):
    """Load a GGUF file into a ``DecoderModel`` (reference entry: create_llm_model_from_gguf, tools/src/pytools.cpp:404)."""
    import json

    from ..models.config import from_hf_dict
    from ..models.decoder import DecoderModel
    from .shard import finalize_model

    f = GGUFFile(path)
    if ori and (Path(ori) / "config.json").exists():
        raw = json.loads((Path(ori) / "config.json").read_text())
    else:
        raw = config_from_meta(f.meta)
    cfg = from_hf_dict(raw)
    if dtype is None:
        dtype = torch.float32 if str(device) == "cpu" else torch.bfloat16
    m = DecoderModel(cfg, device, dtype, tp)
    sd = canonical_tensors(f, cfg, torch.float32)
    if "lm_head.weight" not in sd:
        cfg.tie_embeddings = True
    finalize_model(m, lambda: {k: v for k, v in sd.items() if not k.startswith("model.layers.")},
                   lambda i: {k: v for k, v in sd.items() if k.startswith(f"model.layers.{i}.")},
                   wdtype="dense" if wdtype == "auto" else wdtype)
    m.gguf_meta = f.meta
    return m
