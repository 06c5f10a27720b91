"""Build the native libraries in-tree.

The shared objects are produced under ``fastllm_b200/lib``:

* ``libfb_kernels.so`` -- every CUDA kernel, compiled for sm_100a only (``nvcc -gencode
  arch=compute_100a,code=sm_100a``).  Plain ``extern "C"`` launchers, no libtorch dependency; Python
  calls them through ctypes with raw device pointers and the current CUDA stream.
* ``libfb_runtime.so`` -- the host runtime in C++ (paged-KV page manager with prefix trie, tokenizer,
  chat-template engine, quantiser, CPU operator backend).

* ``libfb_cpu.so`` -- the CPU operator backend; ``libfastllm_b200.so`` -- the C ABI for native hosts, with the
  ``fastllm_chat`` / ``fastllm_benchmark`` / ``fastllm_apiserver`` programs under ``fastllm_b200/bin``.

Run ``python -m fastllm_b200.build`` (add ``--force`` to rebuild everything).  Objects are rebuilt only
when a source or header is newer than the object.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "_build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fopenmp", "-march=x86-64-v3", "-Wall", "-Wno-unused-function"]


def _newer(src: Path, deps: list[Path], out: Path) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in [src, *deps])


def _run(cmd: list[str], log: Path | None = None) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))


def build_kernels(force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    out = LIB / "libfb_kernels.so"
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _newer(src, headers, obj):
            jobs.append((["nvcc", *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], OBJ / (src.stem + ".ptxas.log")))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or not out.exists():
        _run(["nvcc", "-shared", "-o", str(out), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"])
    return out


def build_runtime(force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    rt = CSRC / "runtime"
    sources = sorted(rt.glob("*.cpp"))
    headers = sorted(rt.glob("*.h"))
    out = LIB / "libfb_runtime.so"
    if not sources:
        return out
    jobs = []
    for src in sources:
        obj = OBJ / ("rt_" + src.stem + ".o")
        if force or _newer(src, headers, obj):
            jobs.append((["g++", *CXX_FLAGS, "-I", str(rt), "-c", str(src), "-o", str(obj)], None))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    objs = [OBJ / ("rt_" + s.stem + ".o") for s in sources]
    if force or jobs or not out.exists():
        _run(["g++", "-shared", "-fopenmp", "-o", str(out), *map(str, objs), "-lpthread"])
    return out


CPU_MATH = ["-fno-math-errno", "-fno-trapping-math", "-fassociative-math", "-fno-signed-zeros"]
CPU_ISA = {
    "_avx2": ["-mavx2", "-mfma", "-mf16c"],
    "_avx512": ["-mavx512f", "-mavx512bw", "-mavx512vl", "-mavx512dq", "-mavx2", "-mfma", "-mf16c"],
}


def build_cpu(force: bool = False) -> Path:
    """Native CPU backend: the ISA-specific kernel file is compiled once per instruction set, the dispatcher once."""
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    cpu = CSRC / "cpu"
    headers = sorted(cpu.glob("*.h"))
    out = LIB / "libfb_cpu.so"
    base = ["g++", "-O3", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", *CPU_MATH, "-I", str(cpu)]
    jobs, objs = [], []
    for suffix, isa in CPU_ISA.items():
        obj = OBJ / f"cpu_kernels{suffix}.o"
        objs.append(obj)
        if force or _newer(cpu / "cpu_kernels.cpp", headers, obj):
            jobs.append(([*base, *isa, f"-DFB_ISA_SUFFIX={suffix}", "-c", str(cpu / "cpu_kernels.cpp"), "-o", str(obj)], None))
    for name in ("cpu_ops", "cpu_model", "numa_moe"):
        obj = OBJ / f"{name}.o"
        objs.append(obj)
        if force or _newer(cpu / f"{name}.cpp", headers, obj):
            jobs.append(([*base, "-march=x86-64-v3", "-c", str(cpu / f"{name}.cpp"), "-o", str(obj)], None))
    # VNNI / AVX-512 BF16 / AMX kernels: their own translation unit (only entered after a run-time capability check)
    obj = OBJ / "cpu_accel.o"
    objs.append(obj)
    if force or _newer(cpu / "cpu_accel.cpp", headers, obj):
        jobs.append(([*base, *CPU_ISA["_avx512"], "-mavx512vnni", "-mavx512bf16", "-mamx-tile", "-mamx-int8", "-mamx-bf16", "-c",
                      str(cpu / "cpu_accel.cpp"), "-o", str(obj)], None))
    if jobs:
        with ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    if force or jobs or not out.exists():
        _run(["g++", "-shared", "-o", str(out), *map(str, objs), "-lpthread", "-lm"])
    return out


def build_capi(force: bool = False) -> Path | None:
    """``libfastllm_b200.so`` (the C ABI for hosts that are not Python: it embeds the interpreter, ``csrc/capi``) and the
    native hosts over it under ``fastllm_b200/bin``: ``fastllm_chat``, ``fastllm_benchmark``, ``fastllm_apiserver``.
    Needs the interpreter's headers and shared library; returns ``None`` (nothing built) where they are missing."""
    import sysconfig

    inc = sysconfig.get_paths()["include"]
    if not (Path(inc) / "Python.h").exists():
        return None
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_config_var("VERSION")
    libdirs = [d for d in (sysconfig.get_config_var("LIBDIR"), sysconfig.get_config_var("LIBPL")) if d]
    LIB.mkdir(exist_ok=True)
    bindir = ROOT / "bin"
    bindir.mkdir(exist_ok=True)
    capi, apps = CSRC / "capi", CSRC / "apps"
    out = LIB / "libfastllm_b200.so"
    if force or _newer(capi / "fastllm_capi.cpp", [capi / "fastllm_b200.h"], out):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", inc, str(capi / "fastllm_capi.cpp"), "-o", str(out),
              *[f"-L{d}" for d in libdirs], f"-lpython{ver}", "-ldl", "-lpthread", *[f"-Wl,-rpath,{d}" for d in libdirs]])
    for name in ("chat", "benchmark", "apiserver"):
        exe = bindir / f"fastllm_{name}"
        if force or _newer(apps / f"{name}.cpp", [apps / "app_common.h", capi / "fastllm_b200.h", out], exe):
            _run(["g++", "-O2", "-std=c++17", "-Wall", str(apps / f"{name}.cpp"), "-o", str(exe), f"-L{LIB}", "-lfastllm_b200", "-lpthread",
                  "-Wl,-rpath,$ORIGIN/../lib"])
    return out


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_runtime(force)
    build_cpu(force)
    build_capi(force)


if __name__ == "__main__":
    build_all("--force" in sys.argv)
    print("built:", *(p.name for p in sorted(LIB.glob("*.so"))))
