"""Operator executor: an ordered list of devices, each able to run some operators; an operator runs on the first device of
the list that accepts it, after its tensor arguments have been moved there.

The kernels themselves are reached through ``ops.api`` (which picks the CUDA kernel, the native CPU backend or PyTorch by
where the tensors live); the executor is the placement layer above it: device order (``SetFirstDevice``), forced placement
(``RunOnDevice``), migration of operands (``ToDevice``) and a per-operator timing table.

Reference: ``Executor`` (include/executor.h, src/executor.cpp:211-339): devices in priority order, ``CanRun`` probing,
operand migration before ``Run``, ``AddProfiler`` / ``PrintProfiler``.
"""
from __future__ import annotations

import time

import torch

from . import api


class Device:
    """One placement target: a torch device plus the set of operators it may run (``None``: all of ``ops.api``)."""

    def __init__(self, device_type: str, index: int = 0, ops: set | None = None):
        self.device_type = device_type
        self.index = index
        self.ops = ops
        self.torch_device = torch.device("cuda", index) if device_type == "cuda" else torch.device("cpu")

    def available(self) -> bool:
        return self.device_type != "cuda" or (torch.cuda.is_available() and self.index < torch.cuda.device_count())

    def can_run(self, op: str, args, kwargs) -> bool:
        if not self.available() or not hasattr(api, op):
            return False
        if self.ops is not None and op not in self.ops:
            return False
        probe = getattr(api, "CanRun" + op, None)
        if probe is not None:
            try:
                return bool(probe(*args[:2]))
            except Exception:
                return True
        return True


def ToDevice(value, device):
    """Tensors (also inside lists / tuples / dicts) moved to ``device``; everything else is passed through."""
    if isinstance(value, torch.Tensor):
        return value if value.device == torch.device(device) else value.to(device)
    if isinstance(value, (list, tuple)):
        return type(value)(ToDevice(v, device) for v in value)
    if isinstance(value, dict):
        return {k: ToDevice(v, device) for k, v in value.items()}
    return value


class Executor:
    def __init__(self, devices: list[Device] | None = None):
        if devices is None:
            devices = ([Device("cuda", 0)] if torch.cuda.is_available() else []) + [Device("cpu")]
        self.devices = list(devices)
        self.profiler: dict[str, list] = {}          # op -> [calls, seconds]

    # ---- device list ----
    def ClearDevices(self):
        self.devices = []

    def AddDevice(self, device: Device):
        self.devices.append(device)

    def SetFirstDevice(self, device: str):
        """``"cuda"``, ``"cuda:1"`` or ``"cpu"`` moves that device to the front of the order (added when not present)."""
        kind, _, idx = device.partition(":")
        idx = int(idx) if idx else 0
        for i, d in enumerate(self.devices):
            if d.device_type == kind and (kind != "cuda" or d.index == idx):
                self.devices.insert(0, self.devices.pop(i))
                return
        self.devices.insert(0, Device(kind, idx))

    def GetFirstDeviceType(self) -> str:
        return self.devices[0].device_type if self.devices else ""

    def GetDeviceIds(self, device_type: str) -> list[int]:
        return [d.index for d in self.devices if d.device_type == device_type]

    def HasDevice(self, device_type: str) -> bool:
        return any(d.device_type == device_type and d.available() for d in self.devices)

    def CanRunOnFirstDevice(self, op: str, *args, **kwargs) -> bool:
        return bool(self.devices) and self.devices[0].can_run(op, args, kwargs)

    # ---- running ----
    def _run_on(self, dev: Device, op: str, args, kwargs):
        a, k = ToDevice(args, dev.torch_device), ToDevice(kwargs, dev.torch_device)
        t0 = time.perf_counter()
        out = getattr(api, op)(*a, **k)
        if dev.device_type == "cuda" and self._timed:
            torch.cuda.synchronize(dev.torch_device)
        self.AddProfiler(op, time.perf_counter() - t0)
        return out

    _timed = False          # True: synchronise after CUDA operators so the table holds device-inclusive times

    def Run(self, op: str, *args, **kwargs):
        """Run ``op`` on the first device in the order that accepts it; operands are migrated there."""
        for d in self.devices:
            if d.can_run(op, args, kwargs):
                return self._run_on(d, op, args, kwargs)
        raise RuntimeError(f"no device can run operator '{op}'")

    def RunOnDevice(self, device_type: str, op: str, *args, **kwargs):
        for d in self.devices:
            if d.device_type == device_type and d.can_run(op, args, kwargs):
                return self._run_on(d, op, args, kwargs)
        raise RuntimeError(f"no '{device_type}' device can run operator '{op}'")

    # ---- profile ----
    def ClearProfiler(self):
        self.profiler.clear()

    def AddProfiler(self, op: str, spend: float):
        row = self.profiler.setdefault(op, [0, 0.0])
        row[0] += 1
        row[1] += spend

    def PrintProfiler(self) -> str:
        total = sum(v[1] for v in self.profiler.values()) or 1e-12
        lines = [f"{op:32s} calls {n:6d}  {s * 1e3:10.3f} ms  {100.0 * s / total:5.1f} %"
                 for op, (n, s) in sorted(self.profiler.items(), key=lambda kv: -kv[1][1])]
        text = "\n".join(lines)
        print(text)
        return text


_current: Executor | None = None


def GetExecutor() -> Executor:
    global _current
    if _current is None:
        _current = Executor()
    return _current


def SetCurrentThreadExecutor(executor: Executor | None):
    global _current
    _current = executor
