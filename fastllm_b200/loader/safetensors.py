"""Minimal safetensors reader / writer (no external dependency).

File = 8-byte little-endian header length, JSON header ``{name: {dtype, shape, data_offsets}}``, raw data.
Reading maps the file and returns zero-copy ``torch`` views; the reference's reader
(src/model.cpp:876-1420) does the same with optional mmap.  The extra dtype string ``"fastllm"`` marks a
tensor that holds an already-quantised weight in the exporter's byte format (src/model.cpp:4590); such
tensors are returned as raw uint8 blobs for ``loader.flm`` to decode.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from pathlib import Path

import numpy as np
import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
    "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafeTensorFile:
    """One mapped .safetensors file."""

    def __init__(self, path: str | Path):
        self.path = str(path)
        self._f = open(self.path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        self.header = json.loads(self._f.read(n).decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self.data_start = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._buf = np.frombuffer(self._mm, dtype=np.uint8)

    def keys(self):
        return self.header.keys()

    def info(self, name: str):
        return self.header[name]

    def get(self, name: str) -> torch.Tensor:
        e = self.header[name]
        b0, b1 = e["data_offsets"]
        raw = self._buf[self.data_start + b0:self.data_start + b1]
        dt = e["dtype"]
        if dt == "fastllm" or dt not in _DTYPES:
            return torch.from_numpy(raw.copy())
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # the mapping is read-only; callers never write through the view
            t = torch.from_numpy(raw)
        tdt = _DTYPES[dt]
        if b1 == b0:
            return torch.empty(e["shape"], dtype=tdt)
        return t.view(tdt).reshape(e["shape"])

    def span(self, first: str, second: str):
        """One tensor over two matrices that lie back to back in the file (same dtype and column count): ``[rows_a + rows_b, K]``
        without a copy, else None.  Writers that sort tensors by name put an expert's gate_proj and up_proj side by side."""
        a, b = self.header[first], self.header[second]
        if a["dtype"] != b["dtype"] or a["dtype"] not in _DTYPES or len(a["shape"]) != 2 or a["shape"][1:] != b["shape"][1:]:
            return None
        if a["data_offsets"][1] != b["data_offsets"][0]:
            return None
        raw = self._buf[self.data_start + a["data_offsets"][0]:self.data_start + b["data_offsets"][1]]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.from_numpy(raw)
        return t.view(_DTYPES[a["dtype"]]).reshape(a["shape"][0] + b["shape"][0], a["shape"][1])

    def close(self):
        try:
            self._buf = None
            self._mm.close()
            self._f.close()
        except Exception:
            pass


def save_file(tensors: dict, path: str | Path, metadata: dict | None = None, raw_dtypes: dict | None = None) -> None:
    """Write tensors (name -> torch.Tensor on CPU) to ``path``.  ``raw_dtypes[name]`` overrides the dtype string
    (used for ``"fastllm"`` blobs stored as uint8)."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = list(tensors.keys())
    for name in order:
        t = tensors[name]
        nbytes = t.numel() * t.element_size()
        dt = (raw_dtypes or {}).get(name) or _NAMES[t.dtype]
        header[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(hj) % 8) % 8
    hj += b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name in order:
            t = tensors[name].contiguous()
            if t.dtype in (torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2):
                arr = t.view(torch.uint8 if t.element_size() == 1 else torch.int16).numpy()
            else:
                arr = t.numpy()
            f.write(arr.tobytes())


def open_model_dir(path: str | Path):
    """Return (list of SafeTensorFile, name -> file index) for an HF folder (sharded or single file)."""
    p = Path(path)
    idx = p / "model.safetensors.index.json"
    files, where = [], {}
    if idx.exists():
        wm = json.loads(idx.read_text())["weight_map"]
        names = sorted(set(wm.values()))
        files = [SafeTensorFile(p / n) for n in names]
        pos = {n: i for i, n in enumerate(names)}
        where = {k: pos[v] for k, v in wm.items()}
    else:
        names = sorted(x.name for x in p.glob("*.safetensors"))
        if not names:
            raise FileNotFoundError(f"no .safetensors files in {p}")
        files = [SafeTensorFile(p / n) for n in names]
        for i, f in enumerate(files):
            for k in f.keys():
                where[k] = i
    return files, where
