"""Paged KV cache: device page pools per layer plus the host page manager (C++, with prefix trie).

Pool shape per layer follows the reference (``[maxPages, pageLen, numHeads, headDim]``,
src/fastllm.cpp:4885-4992); capacity is derived from free device memory times ``gpu_mem_ratio`` like the
reference's warm-up (src/models/basellm.cpp:3905+).  Pools are zero-filled: the attention kernels rely
on unused slots holding finite values.
"""
from __future__ import annotations

import ctypes
import math

import torch

from ..ops import _lib
from ..ops.attention import PAGE_LEN


class PageManager:
    """Thin ctypes wrapper over ``csrc/runtime/page_manager.cpp``."""

    def __init__(self, num_pages: int, page_len: int = PAGE_LEN):
        self.lib = _lib.runtime()
        L = self.lib
        L.fbpm_create.restype = ctypes.c_void_p
        L.fbpm_create.argtypes = [ctypes.c_int, ctypes.c_int]
        L.fbpm_destroy.argtypes = [ctypes.c_void_p]
        L.fbpm_num_available.argtypes = [ctypes.c_void_p]
        L.fbpm_num_free.argtypes = [ctypes.c_void_p]
        ip = ctypes.POINTER(ctypes.c_int)
        L.fbpm_alloc.argtypes = [ctypes.c_void_p, ctypes.c_int, ip]
        L.fbpm_release.argtypes = [ctypes.c_void_p, ip, ctypes.c_int]
        L.fbpm_query.argtypes = [ctypes.c_void_p, ip, ctypes.c_int, ip, ctypes.c_int]
        L.fbpm_record.argtypes = [ctypes.c_void_p, ip, ctypes.c_int, ip, ctypes.c_int]
        L.fbpm_clear_cache.argtypes = [ctypes.c_void_p]
        L.fbpm_stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_longlong)]
        self.num_pages, self.page_len = num_pages, page_len
        self.h = ctypes.c_void_p(L.fbpm_create(num_pages, page_len))

    def __del__(self):
        try:
            if self.h:
                self.lib.fbpm_destroy(self.h)
                self.h = None
        except Exception:
            pass

    @staticmethod
    def _arr(v):
        return (ctypes.c_int * len(v))(*v)

    def num_available(self) -> int:
        return self.lib.fbpm_num_available(self.h)

    def num_free(self) -> int:
        return self.lib.fbpm_num_free(self.h)

    def alloc(self, n: int) -> list[int] | None:
        if n <= 0:
            return []
        out = (ctypes.c_int * n)()
        got = self.lib.fbpm_alloc(self.h, n, out)
        return list(out) if got == n else None

    def release(self, pages) -> None:
        if pages:
            self.lib.fbpm_release(self.h, self._arr(pages), len(pages))

    def query(self, tokens) -> list[int]:
        """Pages holding the longest cached whole-page prefix of ``tokens`` (a reference is taken on each)."""
        n = len(tokens)
        maxp = max(1, n // self.page_len)
        out = (ctypes.c_int * maxp)()
        got = self.lib.fbpm_query(self.h, self._arr(tokens), n, out, maxp)
        return list(out[:got])

    def record(self, tokens, pages) -> None:
        if pages:
            self.lib.fbpm_record(self.h, self._arr(tokens), len(tokens), self._arr(pages), len(pages))

    def clear_cache(self) -> None:
        self.lib.fbpm_clear_cache(self.h)

    def stats(self) -> dict:
        out = (ctypes.c_longlong * 4)()
        self.lib.fbpm_stats(self.h, out)
        return dict(free=out[0], cached=out[1], lookups=out[2], hits=out[3])


class KVCache:
    """Device page pools of one rank + the shared page manager."""

    def __init__(self, model, num_pages: int, page_len: int = PAGE_LEN, state_slots: int = 0):
        self.num_pages = num_pages
        self.page_len = page_len
        ks, vs = model.kv_cache_shape(num_pages)
        dev, dt = model.device, (getattr(model, "kv_dtype", None) or model.dtype)
        self.pools = []
        self.state_slots = state_slots         # requests that can hold linear-attention state at once (+ one scratch slot)
        self.linear_layers = [i for i in range(model.cfg.num_layers) if model.cfg.layer_is_linear(i)]
        staged = getattr(model, "layer_devices", None)
        for i in range(model.cfg.num_layers):
            if staged is not None:
                dev = staged[i]            # layer-split placement: a layer's pages live on that layer's device
            if model.cfg.layer_is_linear(i):
                # no pages: a convolution window and a delta-rule state per request slot; the last slot is scratch for
                # padded decode rows
                cs, rs = model.linear_state_shapes(state_slots + 1)
                self.pools.append((torch.zeros(cs, device=dev, dtype=model.dtype), torch.zeros(rs, device=dev, dtype=torch.float32)))
                continue
            lks, lvs = ks, vs
            if hasattr(model, "kv_cache_shape_layer"):
                # layers with their own page shape; a layer that projects no keys / values reads an earlier layer's pools
                shp = model.kv_cache_shape_layer(i, num_pages)
                if shp is None:
                    self.pools.append(self.pools[model.kv_donor(i)])
                    continue
                lks, lvs = shp
            k = torch.zeros(lks, device=dev, dtype=dt)
            v = torch.zeros(lvs, device=dev, dtype=dt) if lvs is not None else None
            self.pools.append((k, v))
        if getattr(model, "mtp", None) is not None:
            # the draft head's decoder layer keeps its own pages under the same page ids (pool index num_layers)
            self.pools.append((torch.zeros(ks, device=model.device, dtype=dt),
                               torch.zeros(vs, device=model.device, dtype=dt) if vs is not None else None))
        self.manager = PageManager(num_pages, page_len)


    def reset_state(self, slot: int) -> None:
        """Zero the linear-attention state of one request slot (a request starts, or restarts after an eviction)."""
        for conv, rec in self.linear_pools():
            conv[slot].zero_()
            rec[slot].zero_()

    def snapshot_states(self, slots):
        """Copies of the linear-attention state (convolution window, recurrent state) of the given request slots, per layer."""
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.pools[self.linear_layers[0]][0].device) if self.linear_layers else None
        return [(conv.index_select(0, idx), rec.index_select(0, idx)) for conv, rec in self.linear_pools()], list(slots)

    def restore_states(self, snap, slots) -> None:
        """Put the snapshot rows of ``slots`` (a subset of the snapshot's slots) back."""
        saved, order = snap
        rows = [order.index(s) for s in slots]
        for (conv, rec), (c0, r0) in zip(self.linear_pools(), saved):
            for s, j in zip(slots, rows):
                conv[s].copy_(c0[j])
                rec[s].copy_(r0[j])

    def linear_pools(self):
        return [self.pools[i] for i in self.linear_layers]

    @staticmethod
    def plan_num_pages(model, gpu_mem_ratio: float = 0.9, max_tokens: int | None = None, reserve_bytes: int = 2 << 30) -> int:
        """Pages that fit the memory budget (after the linear-attention state pools, when the model has such layers)."""
        per_page = model.kv_bytes_per_page() + getattr(model, "_extra_page_bytes", 0)     # + a draft model's pools under the same page ids
        if model.device.type == "cuda":
            free, _total = torch.cuda.mem_get_info(model.device)
            budget = int(free * gpu_mem_ratio) - reserve_bytes - getattr(model, "_state_bytes_reserved", 0)
            n = max(16, budget // per_page)
        else:
            n = 512
        if max_tokens:
            n = min(n, math.ceil(max_tokens / PAGE_LEN) + 8)
        return int(n)
