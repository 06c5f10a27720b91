"""Token sampling: greedy arg-max (CUDA kernel) and penalty / temperature / top-k / top-p sampling.

Order of operations follows the reference sampler (src/fastllm.cpp:3037-3138): repeat penalty on the
recent-token window, temperature, top-k, softmax, top-p cut, random draw.
"""
from __future__ import annotations

import torch

from ..ops import basic as B


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
    kmax = int(min(V, max(max(top_k), 1)))
    kmax = min(V, kmax if kmax > 0 else 50)
    vals, idx = lg.topk(kmax, dim=-1)
    ks = torch.tensor([k if k > 0 else kmax for k in top_k], device=dev)[:, None]
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
