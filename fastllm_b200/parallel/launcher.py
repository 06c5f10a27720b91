"""Tensor-/expert-parallel groups as one process per GPU, started from a single command.

``TPGroup.launch(spec, devices)`` is what ``llm.model(path, tp=N)``, ``ftllm server --tp N`` and
``--device multicuda:0,1,...`` use: the calling process becomes rank 0 (scheduler, HTTP, page manager), spawns one
worker process per further GPU, and every rank builds its shard of the model from the same *spec* (a JSON-able
description: an HF folder with dtype flags, or a random-init preset).  The workers then sit in
``control.WorkerLoop`` replaying rank 0's step plans.  ``TPGroup.attach(spec)`` does the same when the ranks were
started by an outer launcher (``torchrun`` sets RANK / WORLD_SIZE): rank 0 returns with a control plane, the other
ranks serve until rank 0 stops them and then return ``None``.

Reference behaviour matched: ``--tp N`` / ``--device multicuda:...`` serve a model over several GPUs from one
command line (tools/fastllm_pytools/util.py:244-307, 855-880); its workers are threads
(src/models/qwen3.cpp:2902-2915), ours are processes because every rank owns a CUDA context, its NCCL
communicator and its symmetric-memory arena.
"""
from __future__ import annotations

import atexit
import json
import os
import socket
import subprocess
import sys
import time

import torch

from .control import ControlPlane, StepRing, WorkerLoop

SPEC_ENV = "FB_TP_WORKER_SPEC"


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def build_rank_model(spec: dict, rank: int, world: int, device: str):
    """Build this rank's model + engine from the spec.  Returns ``(engine, extra)``; runs the same collective
    set-up calls (symmetric arena rendezvous, page-count agreement) on every rank, in the same order."""
    from ..engine import EngineConfig, LLMEngine
    from ..models.decoder import TPInfo
    from .tp import TPComm

    dev = torch.device(device)
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    tp = TPInfo(rank, world, TPComm(rank, world, dev, backend="nccl" if dev.type == "cuda" else "gloo") if world > 1 else None)
    kind = spec.get("kind", "hf")
    ecfg = EngineConfig(**spec.get("engine", {}))
    comm_mode = spec.get("comm", "auto")
    if kind == "preset":
        from ..models import preset, random_init
        from .ep import EPInfo

        cfg = preset(spec["model"])
        cfg.raw.update(spec.get("config_raw", {}))          # extra config.json keys for the synthetic architecture (tests)
        dt = getattr(torch, spec.get("dtype", "bfloat16"))
        if world > 1 and dev.type == "cuda" and comm_mode in ("auto", "fused"):
            from . import symm

            tp.comm.fused = symm.try_create(tp.comm, cfg, int(spec.get("max_m", ecfg.max_batch)), strict=(comm_mode == "fused"),
                                            max_big_m=symm.prefill_rows(ecfg))
        ep = EPInfo.from_tp(tp) if (world > 1 and cfg.is_moe and not spec.get("moe_tp")) else None
        model = random_init(cfg, dev, dt, tp=tp, ep=ep, seed=int(spec.get("seed", 0)), std=float(spec.get("std", 0.02)),
                            wdtype=spec.get("wdtype", "auto"), moe_wdtype=spec.get("moe_wdtype") or None)
        if spec.get("kv_cache_dtype"):
            model.set_kv_cache_dtype(spec["kv_cache_dtype"])
        eng = LLMEngine(model, ecfg, num_pages=spec.get("num_pages"), eos_token_ids=spec.get("eos_token_ids"))
        return eng, None
    if kind == "hf":
        from .. import llm

        llm._settings.update(spec.get("settings", {}))
        kw = dict(spec.get("kwargs", {}))
        m = llm.model(kw.pop("path"), device=str(dev), tp=tp, engine_config=ecfg if spec.get("engine") else None,
                      _defer_fused=True, **kw)
        if world > 1 and dev.type == "cuda" and comm_mode in ("auto", "fused"):
            from . import symm

            tp.comm.fused = symm.try_create(tp.comm, m.torch_model.cfg, min(256, m.engine.cfg.max_batch), strict=(comm_mode == "fused"),
                                            max_big_m=symm.prefill_rows(m.engine.cfg))
        return m.engine, m
    raise ValueError(f"unknown model spec kind '{kind}'")


class TPGroup:
    """Rank 0's handle on the group: the control plane, the worker processes, orderly shutdown."""

    def __init__(self, world: int, ring: StepRing | None, procs=None, owns_dist: bool = False):
        self.world = world
        self.ring = ring
        self.control = ControlPlane(ring, world) if ring is not None else None
        self.procs = procs or []
        self.owns_dist = owns_dist
        self.closed = False
        self.engine = None
        atexit.register(self.shutdown)

    # -- spawn mode -------------------------------------------------------------------------------------
    @staticmethod
    def launch(spec: dict, devices: list[str], extra_env: dict | None = None):
        """The caller becomes rank 0 of a new group over ``devices`` (``["cuda:0", "cuda:1"]`` or ``["cpu", "cpu"]``).
        Returns ``(group, engine, extra)``."""
        import torch.distributed as dist

        world = len(devices)
        if world < 2:
            raise ValueError("a parallel group needs at least two devices")
        if dist.is_available() and dist.is_initialized():
            raise RuntimeError("torch.distributed is already initialised in this process; use TPGroup.attach")
        ring = StepRing(create=True, n_consumers=world - 1)
        port = _free_port()
        base = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world))
        base.update(extra_env or {})
        wspec = dict(spec, ring=ring.path, devices=devices, parent_pid=os.getpid())
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        base["PYTHONPATH"] = root + os.pathsep + base.get("PYTHONPATH", "")
        procs = []
        for r in range(1, world):
            env = dict(base, RANK=str(r), LOCAL_RANK=str(r))
            env[SPEC_ENV] = json.dumps(wspec)
            procs.append(subprocess.Popen([sys.executable, "-m", "fastllm_b200.parallel.launcher"], env=env))
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK="0", LOCAL_RANK="0")
        group = TPGroup(world, ring, procs, owns_dist=True)
        try:
            _init_dist(0, world, devices[0])
            eng, extra = build_rank_model(spec, 0, world, devices[0])
        except BaseException:
            group.shutdown()
            raise
        eng.control = group.control
        eng.runner.control = group.control
        group.engine = eng
        return group, eng, extra

    # -- attach mode (ranks started by torchrun or a test harness) ----------------------------------------
    @staticmethod
    def attach(spec: dict, device: str | None = None):
        """Every rank of an already-launched job calls this.  Rank 0 gets ``(group, engine, extra)`` back at once;
        the other ranks serve step plans until rank 0 shuts the group down, then get ``(None, engine, extra)``."""
        import torch.distributed as dist

        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        local = int(os.environ.get("LOCAL_RANK", str(rank)))
        if device is None:
            device = f"cuda:{local}" if torch.cuda.is_available() else "cpu"
        owns = not (dist.is_available() and dist.is_initialized())
        if world > 1 and owns:
            _init_dist(rank, world, device)
        if world == 1:
            eng, extra = build_rank_model(spec, 0, 1, device)
            group = TPGroup(1, None)
            group.engine = eng
            return group, eng, extra
        box = [None]
        ring = None
        if rank == 0:
            ring = StepRing(create=True, n_consumers=world - 1)
            box[0] = ring.path
        dist.broadcast_object_list(box, src=0)
        if rank != 0:
            ring = StepRing(box[0])
        eng, extra = build_rank_model(spec, rank, world, device)
        if rank == 0:
            group = TPGroup(world, ring, owns_dist=owns)
            eng.control = group.control
            eng.runner.control = group.control
            group.engine = eng
            return group, eng, extra
        loop = WorkerLoop(eng.runner, ring, rank)
        eng.worker_loop = loop
        hook = spec.get("_worker_hook")
        if hook is not None:
            hook(loop, eng)
        loop.run()
        ring.release()
        teardown_rank(eng, owns)
        return None, eng, extra

    def poll(self) -> None:
        """Raise if a spawned worker process has exited."""
        for r, p in enumerate(self.procs, start=1):
            rc = p.poll()
            if rc is not None and not self.closed:
                raise RuntimeError(f"tensor-parallel worker rank {r} exited with code {rc}")

    def shutdown(self) -> None:
        if self.closed:
            return
        self.closed = True
        if self.control is not None:
            self.control.stop()
        for p in self.procs:
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                p.terminate()
                try:
                    p.wait(timeout=5)
                except subprocess.TimeoutExpired:
                    p.kill()
        if self.ring is not None:
            self.ring.release()
        if self.engine is not None:
            self.engine.stop()
            teardown_rank(self.engine, self.owns_dist and self.world > 1)
            self.engine = None
        elif self.world > 1:
            _finish_dist(self.owns_dist)


def _init_dist(rank: int, world: int, device: str) -> None:
    import torch.distributed as dist

    dev = torch.device(device)
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)


def _finish_dist(owns: bool) -> None:
    import torch.distributed as dist

    if owns and dist.is_available() and dist.is_initialized():
        try:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            dist.destroy_process_group()
        except Exception:
            pass


def teardown_rank(eng, owns_dist: bool) -> None:
    """Release one rank's GPU-side state in an order that lets the process exit normally: captured graphs first (they
    reference communicator buffers), then the symmetric arena, then the process group."""
    import gc

    cuda = eng.model.device.type == "cuda"
    if cuda:
        torch.cuda.synchronize()
    for s in eng.runner.slots.values():
        s.graph = None
    eng.runner.slots.clear()
    if eng.model.tp.comm is not None:
        eng.model.tp.comm.fused = None
    gc.collect()
    if cuda:
        torch.cuda.synchronize()
    _finish_dist(owns_dist)


def worker_main() -> int:
    """Entry point of a spawned worker rank (``python -m fastllm_b200.parallel.launcher``)."""
    spec = json.loads(os.environ[SPEC_ENV])
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    device = spec["devices"][rank]
    _init_dist(rank, world, device)
    eng, _extra = build_rank_model(spec, rank, world, device)
    ring = StepRing(spec["ring"])
    loop = WorkerLoop(eng.runner, ring, rank, parent_pid=spec.get("parent_pid"))
    reason = loop.run()
    ring.release()
    teardown_rank(eng, True)
    return 0 if reason in ("stop", "closed") else 3


if __name__ == "__main__":
    t0 = time.time()
    sys.exit(worker_main())
