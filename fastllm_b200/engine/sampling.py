"""Token sampling: greedy arg-max (CUDA kernel) and penalty / temperature / top-k / top-p sampling.

Order of operations follows the reference sampler (src/fastllm.cpp:3037-3138): repeat penalty on the
recent-token window, temperature, top-k, softmax, top-p cut, random draw.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..ops import basic as B

_P, _I = ctypes.c_void_p, ctypes.c_int
_lib.register_sigs({"fb_sample": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P]}, ["sampling"])


def sample_fused(logits: torch.Tensor, recent_ids, penalties, top_k, top_p, temperature, uniforms=None, want_prob: bool = False):
    """Penalty + temperature + top-k + top-p + draw in one kernel launch (CUDA, fp32 logits ``[R, V]``, modified in place).

    ``uniforms``: per-row variates in [0, 1) (drawn here from the default generator when None).  Returns int32 ids ``[R]``
    (and the chosen token's probability when ``want_prob``).
    """
    R, V = logits.shape
    dev = logits.device
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1
    width = max(1, max((len(set(x)) for x in recent_ids), default=1))
    rec = torch.full((R, width), -1, dtype=torch.int32)
    for r, ids in enumerate(recent_ids):
        u = sorted(set(i for i in ids if 0 <= i < V))
        if u:
            rec[r, :len(u)] = torch.tensor(u, dtype=torch.int32)
    host = torch.tensor([list(map(float, temperature)), list(map(float, top_p)), list(map(float, penalties)),
                         list(uniforms) if uniforms is not None else torch.rand(R).tolist()], dtype=torch.float32)
    f = host.to(dev, non_blocking=True)
    tk = torch.tensor(list(top_k), dtype=torch.int32).to(dev, non_blocking=True)
    rec = rec.to(dev, non_blocking=True)
    out = torch.empty(R, dtype=torch.int32, device=dev)
    prob = torch.empty(R, dtype=torch.float32, device=dev) if want_prob else None
    rc = _lib.kernels().fb_sample(B._ptr(logits), logits.stride(0), R, V, B._ptr(f[0]), B._ptr(tk), B._ptr(f[1]), B._ptr(f[3]), B._ptr(f[2]),
                                  B._ptr(rec), width, B._ptr(out), B._ptr(prob), B._stream())
    _lib.check(rc, "fb_sample")
    return (out, prob) if want_prob else out


def apply_repeat_penalty(logits: torch.Tensor, recent_ids: list[list[int]], penalties: list[float]) -> torch.Tensor:
    """logits ``[R, V]``; for each row divide positive / multiply negative logits of recently seen tokens."""
    for r, (ids, pen) in enumerate(zip(recent_ids, penalties)):
        if abs(pen - 1.0) < 1e-8 or not ids:
            continue
        idx = torch.tensor(sorted(set(ids)), device=logits.device, dtype=torch.long)
        idx = idx[idx < logits.shape[1]]
        v = logits[r, idx]
        logits[r, idx] = torch.where(v > 0, v / pen, v * pen)
    return logits


def sample(logits: torch.Tensor, top_k, top_p, temperature, generators=None) -> torch.Tensor:
    """Batched top-k / top-p sampling. ``top_k``/``top_p``/``temperature`` are per-row lists. Returns int64 [R]."""
    R, V = logits.shape
    dev = logits.device
    t = torch.tensor([max(x, 1e-6) for x in temperature], device=dev, dtype=torch.float32)[:, None]
    lg = logits.float() / t
    # top_k <= 0 means "top-k off": like the CUDA sampler, such a row draws from its 1024 best candidates
    eff = [int(k) if k > 0 else min(V, 1024) for k in top_k]
    kmax = int(min(V, max(max(eff), 1)))
    vals, idx = lg.topk(kmax, dim=-1)
    ks = torch.tensor(eff, device=dev)[:, None]
    ar = torch.arange(kmax, device=dev)[None, :]
    vals = vals.masked_fill(ar >= ks, float("-inf"))
    probs = torch.softmax(vals, dim=-1)
    cum = probs.cumsum(-1)
    tp = torch.tensor(top_p, device=dev, dtype=torch.float32)[:, None]
    keep = (cum - probs) < tp          # always keeps the first token
    probs = probs * keep
    probs = probs / probs.sum(-1, keepdim=True)
    if generators is None or all(g is None for g in generators):
        choice = torch.multinomial(probs, 1)
    else:
        choice = torch.stack([torch.multinomial(probs[r], 1, generator=generators[r]) for r in range(R)])
    return idx.gather(1, choice).squeeze(1)


def greedy(logits: torch.Tensor, id_offset: int = 0):
    return B.argmax(logits, id_offset)
