"""Quantised Hugging Face export: the folder keeps its config / tokenizer files, weights are quantised once and
stored in safetensors with the dtype string ``"fastllm"`` whose payload is the reference's tensor blob
(ExportFastllmFormat / CreateFromFastllmFormat, src/fastllm.cpp:2783-2940; written by ExportLLMModelFromHF,
src/model.cpp:4189+).  Loading such a folder needs no re-quantisation.

Blob: ``int32 1, int32 DataType`` then
    FP8_E4M3(10):            int32 blockK, int32 blockM, int32 n_scales, n_scales x float, data
    INT8(3) / INT4(4):       int32 axis, k x (float min, float max), data
    INT4_NOZERO(8):          int32 axis, k x (float min, float scale), data
    INT4_GROUP(9):           int32 axis, int32 group, int32 groupCnt, k*group x (float min, float scale), data
"""
from __future__ import annotations

import json
import shutil
import struct
from pathlib import Path

import numpy as np
import torch

from ..ops import quant
from . import safetensors as st

INT8, INT4_GROUP, FP8_E4M3 = 3, 9, 10


def encode_blob(w: torch.Tensor, kind: str) -> torch.Tensor:
    k, group = quant.normalize_wdtype(kind)
    if k == "int8":
        wf = w.float()
        mn = wf.amin(1).clamp(max=0.0)
        mx = wf.amax(1).clamp(min=0.0)
        scale = ((mx - mn) / 255.0).clamp(min=1e-30)
        zero = torch.round(-mn / scale).clamp(0, 255)
        q = torch.round(wf / scale[:, None] + zero[:, None]).clamp(0, 255).to(torch.uint8)
        head = struct.pack("<iii", 1, INT8, 0)
        body = torch.stack([mn, mx], 1).numpy().astype("<f4").tobytes() + q.numpy().tobytes()
    elif k == "int4g":
        packed, scale, mn = quant.quantize_int4g(w, group)
        head = struct.pack("<iiiii", 1, INT4_GROUP, 0, scale.shape[1], group)
        body = torch.stack([mn, scale], 2).numpy().astype("<f4").tobytes() + packed.numpy().tobytes()
    elif k == "fp8":
        q, scale = quant.quantize_fp8_block(w, 128)
        head = struct.pack("<iiiii", 1, FP8_E4M3, 128, 128, scale.numel())
        body = scale.numpy().astype("<f4").tobytes() + q.view(torch.uint8).numpy().tobytes()
    else:
        raise ValueError(f"cannot export dtype {kind} as a fastllm blob")
    return torch.from_numpy(np.frombuffer(head + body, dtype=np.uint8).copy())


def decode_blob(raw: torch.Tensor, shape, dtype=torch.bfloat16) -> torch.Tensor:
    b = raw.numpy().tobytes()
    version, dt = struct.unpack_from("<ii", b, 0)
    if version != 1:
        raise ValueError(f"unsupported fastllm blob version {version}")
    n, k = shape
    pos = 8
    if dt == INT8:
        pos += 4
        mm = np.frombuffer(b, "<f4", 2 * n, pos).reshape(n, 2)
        pos += 8 * n
        q = np.frombuffer(b, np.uint8, n * k, pos).reshape(n, k).astype(np.float32)
        scale = np.maximum((mm[:, 1] - mm[:, 0]) / 255.0, 1e-30)
        zero = np.clip(np.round(-mm[:, 0] / scale), 0, 255)
        return torch.from_numpy((q - zero[:, None]) * scale[:, None]).to(dtype)
    if dt == INT4_GROUP:
        _axis, groups, gc = struct.unpack_from("<iii", b, pos)
        pos += 12
        ms = np.frombuffer(b, "<f4", 2 * n * groups, pos).reshape(n, groups, 2)
        pos += 8 * n * groups
        packed = torch.from_numpy(np.frombuffer(b, np.uint8, n * k // 2, pos).reshape(n, k // 2).copy())
        return quant.dequantize_int4g(packed, torch.from_numpy(ms[..., 1].copy()), torch.from_numpy(ms[..., 0].copy()), dtype, gc)
    if dt == FP8_E4M3:
        bk, bm, ns = struct.unpack_from("<iii", b, pos)
        pos += 12
        scale = torch.from_numpy(np.frombuffer(b, "<f4", ns, pos).copy()).reshape((n + bk - 1) // bk, (k + bm - 1) // bm)
        pos += 4 * ns
        q = torch.from_numpy(np.frombuffer(b, np.uint8, n * k, pos).reshape(n, k).copy()).view(torch.float8_e4m3fn)
        return quant.dequantize_fp8_block(q, scale, dtype, bk)
    raise ValueError(f"unsupported fastllm blob data type {dt}")


def _is_linear(name: str, t: torch.Tensor) -> bool:
    return t.dim() == 2 and name.endswith(".weight") and not any(x in name for x in ("embed", "norm", "lm_head", "mlp.gate.weight"))


def export_quantized_hf(src: str, dst: str, dtype: str = "int4g128", moe_dtype: str | None = None, shard_bytes: int = 4 << 30):
    srcp, dstp = Path(src), Path(dst)
    dstp.mkdir(parents=True, exist_ok=True)
    for f in srcp.iterdir():
        if f.is_file() and not f.name.endswith(".safetensors") and f.name != "model.safetensors.index.json":
            shutil.copy2(f, dstp / f.name)
    files, where = st.open_model_dir(srcp)
    weight_map, cur, raw_dt, size, shard = {}, {}, {}, 0, 0

    def flush():
        nonlocal cur, raw_dt, size, shard
        if not cur:
            return
        shard += 1
        fn = f"model-{shard:05d}.safetensors"
        st.save_file(cur, dstp / fn, metadata={"format": "pt"}, raw_dtypes=raw_dt)
        for k in cur:
            weight_map[k] = fn
        cur, raw_dt, size = {}, {}, 0

    kind_main, _ = quant.normalize_wdtype(dtype)
    for name in sorted(where):
        t = files[where[name]].get(name)
        kind = (moe_dtype or dtype) if ".experts." in name else dtype
        if _is_linear(name, t) and quant.normalize_wdtype(kind)[0] != "dense" and t.is_floating_point():
            blob = encode_blob(t, kind)
            # the header keeps the logical shape; the payload length is the blob length
            cur[name] = blob
            raw_dt[name] = "fastllm"
            cur[name]._fb_shape = list(t.shape)
        else:
            cur[name] = t.contiguous()
        size += cur[name].numel() * cur[name].element_size()
        if size >= shard_bytes:
            flush()
    flush()
    # logical shapes of the blobs live in a side file (the safetensors header carries the blob's byte length)
    shapes = {}
    for fobj in files:
        for k in fobj.keys():
            shapes[k] = fobj.info(k)["shape"]
        fobj.close()
    (dstp / "fastllm_shapes.json").write_text(json.dumps(shapes))
    (dstp / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"fastllm_dtype": dtype}, "weight_map": weight_map}))
