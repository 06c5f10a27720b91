"""Binding of the native whole-model CPU forward (``fbcpu_model_*`` in ``lib/libfb_cpu.so``).

A dense llama-family ``DecoderModel`` on the CPU in fp32 is mirrored into a native structure that points at the model's own
weight tensors (no copy).  One call then runs a complete scheduler step for decode-sized batches, like the reference's C++
layer loop (src/models/qwen3.cpp:3058-3210); longer prefill chunks keep using the operator path, whose fp32 GEMMs go to the
BLAS behind ``torch.matmul``.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p

import torch

from ..ops import cpu

MAX_NATIVE_TOKENS = 32
_WT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


class _Lin(Structure):
    _fields_ = [("w", c_void_p), ("wtype", c_int), ("scale", c_void_p), ("zero", c_void_p), ("group", c_int), ("bias", c_void_p),
                ("N", c_int), ("K", c_int), ("interleaved", c_int)]


class _Layer(Structure):
    _fields_ = [("ln1", c_void_p), ("ln2", c_void_p), ("q_norm", c_void_p), ("k_norm", c_void_p),
                ("qkv", _Lin), ("o", _Lin), ("gate_up", _Lin), ("down", _Lin)]


class _Cfg(Structure):
    _fields_ = [(n, c_int) for n in ("hidden", "layers", "Hq", "Hkv", "D", "inter", "vocab", "rot", "rope_mode", "page_len", "window")] + \
               [(n, c_float) for n in ("eps", "unit_offset", "embed_scale", "attn_scale", "logit_scale")]


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def eligible(model) -> bool:
    c = model.cfg
    if model.on_cuda or model.dtype != torch.float32 or model.tp.size != 1 or not cpu.available():
        return False
    if c.use_mla or c.num_experts or c.hidden_act not in ("silu", "swiglu") or c.norm_kind != "rms" or c.parallel_block or not c.mlp_gated or c.post_norms or model.general_attn or c.final_softcap:
        return False
    if c.has_linear_attn or c.attn_output_gate or c.attn_softcap or c.attn_sinks or c.layer_heads or c.layer_rope or c.head_gate:
        return False
    if any(lw.attn.window or lw.attn.sinks is not None for lw in model.layers):
        return False
    for lw in model.layers:
        for lin in (lw.attn.qkv, lw.attn.o, lw.mlp.gate_up, lw.mlp.down):
            if lin is None or lin.kind not in ("dense", "int8", "int4g"):
                return False
            if lin.kind == "dense" and lin.w.dtype not in _WT:
                return False
    return model.embed is not None and model.embed.dtype == torch.float32 and model.lm_head is not None


class NativeCpuModel:
    def __init__(self, model):
        L = cpu.lib()
        L.fbcpu_model_create.restype = c_void_p
        L.fbcpu_model_create.argtypes = [POINTER(_Cfg)]
        L.fbcpu_model_destroy.argtypes = [c_void_p]
        L.fbcpu_model_set_layer.argtypes = [c_void_p, c_int, POINTER(_Layer)]
        L.fbcpu_model_set_top.argtypes = [c_void_p, c_void_p, c_void_p, POINTER(_Lin), c_void_p, c_void_p]
        L.fbcpu_model_forward.restype = c_int
        L.fbcpu_model_forward.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                          c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        self.L = L
        self.model = model
        self.keep = []          # tensors the native structure points at (fp32 copies of biases / norm weights)
        c = model.cfg
        cos, sin = model.rope_tables()
        cfg = _Cfg(hidden=c.hidden_size, layers=len(model.layers), Hq=model.num_heads_local, Hkv=model.num_kv_heads_local,
                   D=c.head_dim, inter=model.layers[0].mlp.down.k, vocab=model.lm_head.n, rot=model.rot_dim, rope_mode=model.rope_mode,
                   page_len=128, window=0, eps=c.rms_eps, unit_offset=c.norm_unit_offset, embed_scale=c.embed_scale,
                   attn_scale=model.attn_scale, logit_scale=c.logit_scale)
        self.h = c_void_p(L.fbcpu_model_create(ctypes.byref(cfg)))
        for i, lw in enumerate(model.layers):
            lay = _Layer(ln1=_ptr(self._f32(lw.attn.ln)), ln2=_ptr(self._f32(lw.mlp.ln)), q_norm=_ptr(self._f32(lw.attn.q_norm)),
                         k_norm=_ptr(self._f32(lw.attn.k_norm)), qkv=self._lin(lw.attn.qkv), o=self._lin(lw.attn.o),
                         gate_up=self._lin(lw.mlp.gate_up), down=self._lin(lw.mlp.down))
            L.fbcpu_model_set_layer(self.h, i, ctypes.byref(lay))
        head = self._lin(model.lm_head)
        L.fbcpu_model_set_top(self.h, _ptr(model.embed), _ptr(self._f32(model.final_norm)), ctypes.byref(head),
                              _ptr(self._f32(cos)), _ptr(self._f32(sin)))
        self._pools = None

    def __del__(self):
        try:
            self.L.fbcpu_model_destroy(self.h)
        except Exception:
            pass

    def _f32(self, t):
        if t is None:
            return None
        t = t.float().contiguous()
        self.keep.append(t)
        return t

    def _lin(self, lw) -> _Lin:
        w = lw.w if lw.w.is_contiguous() else lw.w.contiguous()
        self.keep.append(w)
        wt = _WT[w.dtype] if lw.kind == "dense" else (3 if lw.kind == "int8" else 4)
        return _Lin(w=_ptr(w), wtype=wt, scale=_ptr(self._f32(lw.scale)), zero=_ptr(self._f32(lw.zero)), group=int(lw.group or 0),
                    bias=_ptr(self._f32(lw.bias)), N=lw.n, K=lw.k, interleaved=int(bool(lw.interleaved)))

    def forward(self, fb, kv_caches) -> torch.Tensor:
        n = len(kv_caches)
        if self._pools is None or self._pools[0] is not kv_caches:
            K = (c_void_p * n)(*[kv[0].data_ptr() for kv in kv_caches])
            V = (c_void_p * n)(*[kv[1].data_ptr() for kv in kv_caches])
            self._pools = (kv_caches, K, V)
        _, K, V = self._pools
        i32 = lambda t: t.to(torch.int32).contiguous()
        ids, pos, slots, pt, kl, cq = i32(fb.ids), i32(fb.positions), i32(fb.slots), i32(fb.page_table), i32(fb.kv_lens), i32(fb.cu_q)
        T = ids.numel()
        rows = fb.logit_rows.to(torch.int64).contiguous() if fb.logit_rows is not None else None
        R = rows.numel() if rows is not None else T
        logits = torch.empty((R, self.model.lm_head.n), dtype=torch.float32)
        rc = self.L.fbcpu_model_forward(self.h, _ptr(ids), _ptr(pos), _ptr(slots), T, _ptr(pt), pt.shape[1], _ptr(kl), _ptr(cq),
                                        kl.numel(), K, V, _ptr(rows), R, _ptr(logits))
        if rc != 0:
            raise RuntimeError(f"fbcpu_model_forward failed at stage {rc}")
        return logits
