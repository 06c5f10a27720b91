"""ctypes loader for the in-tree native libraries.

``kernels()`` returns the CUDA kernel library (``lib/libfb_kernels.so``); it raises if the library is
missing while a GPU is present, so that a GPU run can never silently fall back to the PyTorch path.
``runtime()`` returns the host runtime library (``lib/libfb_runtime.so``).
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_lock = threading.Lock()
_kernels = None
_runtime = None

P = c_void_p
I = c_int
F = c_float
LL = c_longlong

_KERNEL_SIGS = {
    "fb_gemm_16bit": [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P],
    "fb_gemm_16bit_wait": [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, P, P],
    "fb_gemm_qkv_post": [P, P, P, I, I, I, I, I, I, P, P, P, I, P, P, P, P, P, P, P, P, I, I, I, I, F, F, P],
    "fb_gemm_route": [P, P, I, I, I, I, I, I, P, P, P, I, I, I, F, P],
    "fb_gemm_16bit_batched": [P, P, P, I, I, I, I, I, I, I, I, I, I, P],
    "fb_mla_post": [P, I, P, I, P, I, P, P, P, P, P, P, I, I, I, I, I, I, LL, F, I, P],
    "fb_gemm_pick_split": [I, I, I, I],
    "fb_rmsnorm": [P, P, P, P, I, I, I, I, F, F, I, P],
    "fb_rmsnorm_quant": [P, P, P, P, I, I, I, I, F, F, I, I, P, I, P, P, I, P],
    "fb_qkv_post": [P, I, P, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, F, I, P],
    "fb_qkv_post_kv8": [P, I, P, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, F, I, P, P, P],
    "fb_silu_mul": [P, P, I, I, I, I, I, P],
    "fb_glu_act": [P, P, I, I, I, I, I, I, I, P],
    "fb_kv_append_fp8": [P, P, P, P, P, I, I, I, P],
    "fb_quant_q_e4m3x2": [P, P, P, LL, I, P],
    "fb_dequant_weight": [P, P, P, P, I, I, I, I, I, I, I, P],
    "fb_softmax_causal_rows": [P, I, P, I, I, I, I, I, F, I, P],
    "fb_embedding": [P, P, P, I, I, I, P],
    "fb_argmax": [P, P, P, I, I, I, I, I, P],
    "fb_route_topk": [P, P, P, P, I, I, I, I, I, I, I, F, P],
    "fb_attn_decode_plan": [P, I, P, P, I, P],
    "fb_attn_decode_plan_window": [P, I, P, P, I, I, P],
    "fb_attn_decode_opts": [P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, LL, I, I, I, F, I, I, P, I, P, I, P, P, I, I, F, P, P],
    "fb_attn_decode": [P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, LL, I, I, I, F, I, I, P, I, P, I, P, P, I, P],
    "fb_attn_prefill": [P, I, LL, P, P, P, I, P, I, P, P, P, I, I, I, LL, I, F, I, P],
}

_ERROR_READERS = ["gemm", "elementwise", "attn_decode", "attn_prefill"]


class KernelLibraryMissing(RuntimeError):
    pass


_launch_count = 0
_LAUNCHES_PER_CALL = {}


def launch_count() -> int:
    """Number of kernel launches issued through this library so far (launcher calls x kernels per call)."""
    return _launch_count


class KernelProfile:
    """Per-kernel device time table (the reference's per-op profile, src/executor.cpp:335-440, printed with
    FASTLLM_PRINT_PROFILE).  Every launcher call is bracketed by CUDA events on the current stream and an NVTX range;
    ``report()`` synchronises once and sums the events.  Not usable while a CUDA graph is being captured."""

    def __init__(self):
        self.events = []

    def timed(self, name, fn, args):
        import torch

        if torch.cuda.is_current_stream_capturing():
            return fn(*args)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.nvtx.range_push(name)
        a.record()
        rc = fn(*args)
        b.record()
        torch.cuda.nvtx.range_pop()
        self.events.append((name, a, b))
        return rc

    def report(self) -> dict:
        import torch

        torch.cuda.synchronize()
        tot: dict = {}
        for name, a, b in self.events:
            t = tot.setdefault(name, [0, 0.0])
            t[0] += 1
            t[1] += a.elapsed_time(b)
        self.events.clear()
        return {k: {"calls": v[0], "ms": v[1]} for k, v in sorted(tot.items(), key=lambda kv: -kv[1][1])}

    def format(self) -> str:
        rep = self.report()
        total = sum(v["ms"] for v in rep.values()) or 1.0
        lines = [f"{'kernel':32s} {'calls':>8s} {'ms':>10s} {'us/call':>10s} {'share':>7s}"]
        for k, v in rep.items():
            lines.append(f"{k:32s} {v['calls']:8d} {v['ms']:10.3f} {v['ms'] / v['calls'] * 1e3:10.1f} {v['ms'] / total * 100:6.1f}%")
        return "\n".join(lines)


_profile: KernelProfile | None = None


def start_profile() -> KernelProfile:
    """Turn on per-kernel timing (decode should run without CUDA graphs while profiling)."""
    global _profile
    _profile = KernelProfile()
    return _profile


def stop_profile() -> KernelProfile | None:
    global _profile
    p, _profile = _profile, None
    return p


class _KernelProxy:
    """Attribute access returns the ctypes function wrapped with a launch counter."""

    def __init__(self, lib):
        self._lib = lib
        self._cache = {}

    def __getattr__(self, name):
        c = self._cache.get(name)
        if c is not None:
            return c
        fn = getattr(self._lib, name)
        if not name.startswith("fb_") or name.endswith("_read_error") or name == "fb_gemm_pick_split":
            self._cache[name] = fn
            return fn
        n = _LAUNCHES_PER_CALL.get(name, 1)

        def counted(*args, _fn=fn, _n=n, _name=name):
            global _launch_count
            _launch_count += _n
            if _profile is None:
                return _fn(*args)
            return _profile.timed(_name, _fn, args)

        self._cache[name] = counted
        return counted

    def has(self, name) -> bool:
        return hasattr(self._lib, name)


def kernels():
    global _kernels
    if _kernels is not None:
        return _kernels
    with _lock:
        if _kernels is not None:
            return _kernels
        path = _LIB_DIR / "libfb_kernels.so"
        if not path.exists():
            raise KernelLibraryMissing(
                f"{path} not found: run `python -m fastllm_b200.build` (sm_100a kernels are required on GPU)")
        lib = ctypes.CDLL(str(path))
        for name, args in _KERNEL_SIGS.items():
            if hasattr(lib, name):
                fn = getattr(lib, name)
                fn.argtypes = args
                fn.restype = c_int
        for name in list(_ERROR_READERS):
            fn = getattr(lib, f"fb_{name}_read_error", None)
            if fn is not None:
                fn.argtypes = [ctypes.POINTER(c_int), c_int]
                fn.restype = c_int
        _kernels = _KernelProxy(lib)
        return _kernels


def register_sigs(sigs: dict, error_readers: list[str] | None = None) -> None:
    """Let other op modules add signatures for kernels that live in the same library."""
    _KERNEL_SIGS.update(sigs)
    if error_readers:
        for r in error_readers:
            if r not in _ERROR_READERS:
                _ERROR_READERS.append(r)
    if _kernels is not None:
        raw = _kernels._lib
        for name, args in sigs.items():
            if hasattr(raw, name):
                fn = getattr(raw, name)
                fn.argtypes = args
                fn.restype = c_int
        for name in error_readers or []:
            fn = getattr(raw, f"fb_{name}_read_error", None)
            if fn is not None:
                fn.argtypes = [ctypes.POINTER(c_int), c_int]
                fn.restype = c_int


class DeviceKernelError(RuntimeError):
    """A kernel recorded an error (bounded wait ran out, bad argument) in its device-side status word."""


def check_device_errors(reset: bool = True) -> None:
    """Read every translation unit's device error word; raise if any kernel reported a problem.

    Costs one small device-to-host copy per translation unit, so call it between steps, not per kernel.
    """
    lib = kernels()._lib
    buf = (c_int * 8)()
    for name in _ERROR_READERS:
        fn = getattr(lib, f"fb_{name}_read_error", None)
        if fn is None:
            continue
        rc = fn(buf, 1 if reset else 0)
        if rc != 0:
            raise DeviceKernelError(f"reading error word of '{name}' failed with cudaError {rc}")
        if buf[0] != 0:
            raise DeviceKernelError(
                f"kernel error in '{name}': code={buf[0]} kernel_id={buf[1]} site={buf[2]} block=({buf[3]},{buf[4]})")


def set_wait_limit_ns(ns: int) -> None:
    """Time after which a device-side wait (mbarrier, peer arrival counter) gives up and reports, for every kernel of the
    library on the current device.  Default 2 s; tests of the failure path use milliseconds."""
    lib = kernels()._lib
    for name in _ERROR_READERS:
        fn = getattr(lib, f"fb_{name}_set_wait_limit_ns", None)
        if fn is not None:
            fn.argtypes = [ctypes.c_ulonglong]
            fn.restype = c_int
            rc = fn(int(ns))
            if rc != 0:
                raise RuntimeError(f"setting the wait limit of '{name}' failed with cudaError {rc}")


def runtime():
    global _runtime
    if _runtime is not None:
        return _runtime
    with _lock:
        if _runtime is not None:
            return _runtime
        path = _LIB_DIR / "libfb_runtime.so"
        if not path.exists():
            from .. import build

            build.build_runtime()
        _runtime = ctypes.CDLL(str(path))
        return _runtime


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
