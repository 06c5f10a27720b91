"""Read-throughput probe for model files: ``python -m fastllm_b200.utils.ssd_read_bench [--threads N] [--seconds S]
[--block-mb M] [--direct] PATH...`` (a directory stands for its ``*.safetensors`` / ``*.flm`` files).

The reads run in native threads (``csrc/runtime/read_bench.cpp``).  Counterpart of the reference's
``tools/ssd_read_bench.cpp``.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

from ..ops import _lib


def expand(paths) -> list[str]:
    files = []
    for p in paths:
        if os.path.isdir(p):
            files += sorted(os.path.join(p, f) for f in os.listdir(p) if f.endswith((".safetensors", ".flm", ".gguf")))
        elif os.path.isfile(p):
            files.append(p)
    return files


def read_bench(paths, threads: int = 8, seconds: float = 5.0, block_mb: int = 8, direct: bool = False) -> dict:
    files = expand(paths)
    if not files:
        raise FileNotFoundError("no input files")
    L = _lib.runtime()
    L.fbio_read_bench.argtypes = [ctypes.POINTER(ctypes.c_char_p), ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_longlong,
                                  ctypes.c_int, ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_ulonglong),
                                  ctypes.POINTER(ctypes.c_double)]
    L.fbio_read_bench.restype = ctypes.c_int
    arr = (ctypes.c_char_p * len(files))(*[f.encode() for f in files])
    nbytes, nreads, elapsed = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0), ctypes.c_double(0.0)
    rc = L.fbio_read_bench(arr, len(files), int(threads), float(seconds), int(block_mb) << 20, 1 if direct else 0,
                           ctypes.byref(nbytes), ctypes.byref(nreads), ctypes.byref(elapsed))
    if rc != 0:
        raise OSError(f"read bench failed (code {rc}); O_DIRECT needs a file system that supports it")
    return {"files": len(files), "threads": threads, "block_mb": block_mb, "direct": bool(direct), "elapsed_s": elapsed.value,
            "bytes": nbytes.value, "reads": nreads.value, "gb_per_s": nbytes.value / 1e9 / max(elapsed.value, 1e-9)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("paths", nargs="+")
    ap.add_argument("--threads", type=int, default=8)
    ap.add_argument("--seconds", type=float, default=5.0)
    ap.add_argument("--block-mb", type=int, default=8)
    ap.add_argument("--direct", action="store_true", help="O_DIRECT: bypass the page cache")
    a = ap.parse_args(argv)
    print(json.dumps(read_bench(a.paths, a.threads, a.seconds, a.block_mb, a.direct)))


if __name__ == "__main__":
    main()
