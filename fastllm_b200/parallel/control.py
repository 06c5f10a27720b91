"""Multi-rank control plane: the scheduler rank publishes one small step plan per forward pass, the other
tensor-parallel ranks replay it.

Only rank 0 owns the HTTP server, the request queues, the page manager and the scheduler.  Every time its
``ModelRunner`` is about to run a prefill or decode pass it first publishes the pass's plan -- exactly the
integers it is about to copy to its own GPU (token ids, positions, cache slots, lengths, page table) -- on a
shared-memory ring (``csrc/runtime/step_ring.cpp``).  Ranks 1..N-1 run ``WorkerLoop``: consume a plan, run
the same ``ModelRunner`` call, wait for the next one.  The collectives inside the forward pass (fused NVLink
kernels or NCCL) therefore line up without the workers knowing anything about requests.

The reference does the same fan-out inside one process: the scheduler thread hands each step to one host
thread per GPU (src/models/qwen3.cpp:2902-2915, ``PersistentWorkerGroup``; op-level:
src/devices/multicuda/multicudadevice.cpp:97-224).  One process per GPU needs the plan to cross a process
boundary; a ring in /dev/shm costs a memcpy and two cache-line hand-overs per step.

The channel is host-only and has no GPU dependency, so the whole protocol (including abort, eviction and
worker shutdown) is exercised with CPU ranks in the tests.
"""
from __future__ import annotations

import ctypes
import json
import mmap
import os
import tempfile

import numpy as np

from ..ops import _lib

KIND_STOP, KIND_DECODE, KIND_PREFILL, KIND_GATHER, KIND_RESET, KIND_CALL, KIND_PREFILL_KEEP, KIND_MTP, KIND_MM_PUT, KIND_MM_DROP = 0, 1, 2, 3, 4, 5, 6, 7, 8, 9
CONT = 0x100                    # this message continues in the next one (payload larger than a slot)
OK, TIMEOUT, CLOSED, TOO_BIG, BAD, OVERRUN = range(6)


class RingClosed(Exception):
    pass


def _rt():
    L = _lib.runtime()
    if not getattr(L, "_fbring_sigs", False):
        P, U32, U64, I64, I = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int64, ctypes.c_int
        L.fbring_bytes.restype = U64
        L.fbring_bytes.argtypes = [U32, U32]
        L.fbring_init.argtypes = [P, U32, U32, U32]
        L.fbring_check.argtypes = [P]
        L.fbring_close.argtypes = [P]
        L.fbring_close.restype = None
        L.fbring_is_closed.argtypes = [P]
        L.fbring_head.argtypes = [P]
        L.fbring_head.restype = U64
        L.fbring_cursor.argtypes = [P, I]
        L.fbring_cursor.restype = U64
        L.fbring_publish.argtypes = [P, I, P, U32, I64]
        L.fbring_consume.argtypes = [P, I, ctypes.POINTER(I), P, U32, ctypes.POINTER(U32), I64, I64]
        L._fbring_sigs = True
    return L


class StepRing:
    """One publisher, ``n_consumers`` consumers, over a file mapping every rank of the node can open."""

    def __init__(self, path: str | None = None, create: bool = False, n_consumers: int = 1, n_slots: int = 8,
                 slot_bytes: int = 1 << 20):
        self.L = _rt()
        self.owner = create
        if create:
            if path is None:
                d = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
                fd, path = tempfile.mkstemp(prefix="fb_step_ring_", dir=d)
            else:
                fd = os.open(path, os.O_RDWR | os.O_CREAT | os.O_TRUNC, 0o600)
            nbytes = int(self.L.fbring_bytes(n_slots, slot_bytes))
            os.ftruncate(fd, nbytes)
        else:
            fd = os.open(path, os.O_RDWR)
            nbytes = os.fstat(fd).st_size
        self.path = path
        self.mm = mmap.mmap(fd, nbytes)
        os.close(fd)
        self._buf = (ctypes.c_char * nbytes).from_buffer(self.mm)
        self.base = ctypes.c_void_p(ctypes.addressof(self._buf))
        if create:
            rc = self.L.fbring_init(self.base, n_slots, slot_bytes, n_consumers)
            if rc != OK:
                raise ValueError(f"step ring geometry rejected ({rc})")
        elif self.L.fbring_check(self.base) != OK:
            raise RuntimeError(f"{path} is not an initialised step ring")
        self.slot_bytes = slot_bytes if create else int(np.frombuffer(self.mm, dtype=np.uint32, count=4)[2])
        self._out = np.empty(self.slot_bytes, dtype=np.uint8)
        self._kind = ctypes.c_int(0)
        self._n = ctypes.c_uint32(0)

    # -- publisher ------------------------------------------------------------------------------------
    def publish(self, kind: int, payload=None, timeout_s: float = 30.0) -> None:
        if payload is None:
            data = np.empty(0, dtype=np.uint8)
        elif isinstance(payload, (bytes, bytearray)):
            data = np.frombuffer(payload, dtype=np.uint8)
        else:
            data = np.ascontiguousarray(payload).view(np.uint8).reshape(-1)
        off, total = 0, data.size
        while True:
            n = min(self.slot_bytes, total - off)
            last = off + n >= total
            part = data[off:off + n]
            rc = self.L.fbring_publish(self.base, kind | (0 if last else CONT), part.ctypes.data_as(ctypes.c_void_p) if n else None,
                                       n, int(timeout_s * 1e6))
            if rc == CLOSED:
                raise RingClosed()
            if rc == TIMEOUT:
                raise TimeoutError("the worker ranks stopped consuming step plans (a worker process died or is stuck)")
            if rc != OK:
                raise RuntimeError(f"step ring publish failed ({rc})")
            off += n
            if last:
                return

    def close(self) -> None:
        if self.mm is not None:
            self.L.fbring_close(self.base)

    # -- consumer -------------------------------------------------------------------------------------
    def consume(self, consumer: int, timeout_s: float = 1.0, spin_us: int = 200):
        """Next message as ``(kind, uint8 array)``, or None when nothing arrived within the timeout."""
        parts = []
        while True:
            rc = self.L.fbring_consume(self.base, consumer, ctypes.byref(self._kind), self._out.ctypes.data_as(ctypes.c_void_p),
                                       self.slot_bytes, ctypes.byref(self._n), int(timeout_s * 1e6), spin_us)
            if rc == TIMEOUT:
                if parts:
                    continue            # in the middle of a split message: keep waiting for the rest
                return None
            if rc == CLOSED:
                raise RingClosed()
            if rc != OK:
                raise RuntimeError(f"step ring consume failed ({rc})")
            kind, n = self._kind.value, self._n.value
            chunk = self._out[:n].copy()
            if kind & CONT:
                parts.append(chunk)
                continue
            if parts:
                parts.append(chunk)
                chunk = np.concatenate(parts)
            return kind & ~CONT, chunk

    def lag(self) -> int:
        """Messages published and not yet consumed by the slowest consumer."""
        head = int(self.L.fbring_head(self.base))
        n = int(np.frombuffer(self.mm, dtype=np.uint32, count=4)[3])
        return head - min((int(self.L.fbring_cursor(self.base, c)) for c in range(n)), default=head)

    def release(self) -> None:
        """Unmap; the creator also removes the file."""
        if self.mm is None:
            return
        self._buf = None
        self.base = None
        try:
            self.mm.close()
        except BufferError:
            pass
        self.mm = None
        if self.owner:
            try:
                os.unlink(self.path)
            except OSError:
                pass


# ---------------------------------------------------------------------------------------------------------
# plan encoding (int32 arrays; the decode plan is the runner's own metadata buffer, prefixed by three words)
# ---------------------------------------------------------------------------------------------------------
def encode_decode_plan(n: int, bsz: int, want_logits: bool, meta: np.ndarray) -> np.ndarray:
    out = np.empty(3 + meta.size, dtype=np.int32)
    out[0], out[1], out[2] = n, bsz, int(want_logits)
    out[3:] = meta
    return out


def decode_decode_plan(buf: np.ndarray):
    a = buf.view(np.int32)
    return int(a[0]), int(a[1]), bool(a[2]), a[3:]


def encode_prefill_plan(chunks) -> np.ndarray:
    """chunks: list of (token_ids, start_pos, pages, want_logits[, state_slot])."""
    head = [len(chunks)]
    body: list[int] = []
    for ch in chunks:
        toks, start, pages, want = ch[:4]
        ss = ch[4] if len(ch) > 4 and ch[4] is not None else -1
        mm = ch[5] if len(ch) > 5 else None
        head += [len(toks), int(start), len(pages), (1 if want is True else int(want or 0)), int(ss),
                 int(getattr(mm, "ctx_id", -1)) if mm is not None else -1]
        body += list(toks)
        body += list(pages)
    return np.asarray(head + body, dtype=np.int32)


def decode_prefill_plan(buf: np.ndarray, mm_table: dict | None = None):
    """``mm_table``: the multimodal contexts this rank has received, by id (chunks of prompts with images refer to them)."""
    a = buf.view(np.int32)
    nc = int(a[0])
    off = 1 + 6 * nc
    chunks = []
    for c in range(nc):
        nt, start, npg, want, ss, mm = (int(x) for x in a[1 + 6 * c:7 + 6 * c])
        toks = a[off:off + nt].tolist()
        off += nt
        pages = a[off:off + npg].tolist()
        off += npg
        chunks.append((toks, start, pages, (True if want == 1 else (want if want > 1 else False)), ss,
                       (mm_table or {}).get(mm) if mm >= 0 else None))
    return chunks


def encode_mm(mm) -> np.ndarray:
    """A prompt's multimodal context as one message: [id, n, H, prompt length, delta, 0 | 1 (fp32 | bf16 rows)], the image
    tokens' prompt positions, the 3-D rotary positions, then the embedding rows."""
    import torch

    emb = mm.embeds.detach().cpu()
    bf = emb.dtype == torch.bfloat16
    rows = (emb.view(torch.int16) if bf else emb.float()).contiguous().numpy().view(np.uint8).reshape(-1)
    n, H = emb.shape
    head = np.asarray([mm.ctx_id, n, H, mm.pos3.shape[1], mm.delta, 1 if bf else 0], dtype=np.int32)
    return np.concatenate([head.view(np.uint8), np.asarray(mm.embed_positions, dtype=np.int32).view(np.uint8),
                           mm.pos3.to(torch.int32).contiguous().numpy().view(np.uint8).reshape(-1), rows])


def decode_mm(buf: np.ndarray, device):
    import torch

    from ..engine.engine import MultimodalContext

    cid, n, H, L, delta, bf = (int(x) for x in buf[:24].view(np.int32))
    off = 24
    at = buf[off:off + 4 * n].view(np.int32).tolist()
    off += 4 * n
    pos3 = torch.from_numpy(buf[off:off + 12 * L].view(np.int32).reshape(3, L).copy()).long()
    off += 12 * L
    raw = buf[off:].copy()
    emb = torch.from_numpy(raw.view(np.int16).reshape(n, H)).view(torch.bfloat16) if bf else torch.from_numpy(raw.view(np.float32).reshape(n, H))
    mm = MultimodalContext(emb.to(device), at, pos3, delta)
    mm.ctx_id = cid
    return mm


class ControlPlane:
    """Rank 0's side: what the runner / engine call to keep the worker ranks in step."""

    def __init__(self, ring: StepRing, world: int):
        self.ring = ring
        self.world = world
        self.published = 0

    def decode(self, n, bsz, want_logits, meta_np):
        self.ring.publish(KIND_DECODE, encode_decode_plan(n, bsz, want_logits, meta_np))
        self.published += 1

    def prefill(self, chunks, keep_hidden: bool = False):
        self.ring.publish(KIND_PREFILL_KEEP if keep_hidden else KIND_PREFILL, encode_prefill_plan(chunks))
        self.published += 1

    def mtp(self, chunks, sel, src: int):
        """A pass of the draft head: the plan of its chunks, then which rows of the stored hidden rows feed it (``src`` 0: the
        decoder's last pass, 1: the head's own last pass)."""
        plan = encode_prefill_plan(chunks)
        tail = np.asarray([int(src), len(sel)] + [int(i) for i in sel], dtype=np.int32)
        self.ring.publish(KIND_MTP, np.concatenate([np.asarray([plan.size], dtype=np.int32), plan, tail]))
        self.published += 1

    def mm_put(self, mm):
        """Hand a prompt's image embeddings and rotary positions to the worker ranks (its chunks then name the context)."""
        self.ring.publish(KIND_MM_PUT, encode_mm(mm))

    def mm_drop(self, ctx_id: int):
        self.ring.publish(KIND_MM_DROP, int(ctx_id).to_bytes(4, "little", signed=True))

    def gather_logits(self, k: int = 0):
        """``k`` > 0: the ranks exchange their ``k`` best (logit, token id) candidates per row instead of whole logit rows."""
        self.ring.publish(KIND_GATHER, int(k).to_bytes(4, "little") if k > 0 else b"")

    def reset(self):
        self.ring.publish(KIND_RESET)

    def call(self, name: str, **kwargs):
        """Run a named handler on every worker (``WorkerLoop.handlers``), e.g. benchmark timing marks."""
        self.ring.publish(KIND_CALL, json.dumps({"name": name, "args": kwargs}).encode())

    def stop(self):
        try:
            self.ring.publish(KIND_STOP, timeout_s=5.0)
        except (RingClosed, TimeoutError, RuntimeError):
            pass
        self.ring.close()


class WorkerLoop:
    """Ranks 1..N-1: replay the published plans on this rank's ``ModelRunner`` until told to stop."""

    def __init__(self, runner, ring: StepRing, rank: int, parent_pid: int | None = None):
        self.runner = runner
        self.ring = ring
        self.consumer = rank - 1
        self.parent_pid = parent_pid
        self.last_logits = None
        self.steps = 0
        self.errors = 0
        self.handlers = {}          # name -> callable(**args), for KIND_CALL
        self.mm_table = {}          # multimodal contexts received from rank 0, by id
        self.timing = None          # a list: CUDA event pairs around every decode step are appended (device-time benchmarks)
        self.idle_spin_us = 200
        self.busy_spin_us = 20000   # between decode steps the next plan is microseconds away: keep spinning

    def _parent_alive(self) -> bool:
        if self.parent_pid is None:
            return True
        try:
            os.kill(self.parent_pid, 0)
            return True
        except ProcessLookupError:
            return False
        except PermissionError:
            return True

    def run(self) -> str:
        """Returns the reason the loop ended: "stop", "closed" or "orphaned"."""
        import torch

        from ..ops._lib import DeviceKernelError

        model = self.runner.model
        if model.device.type == "cuda":
            torch.cuda.set_device(model.device)
        busy = False
        while True:
            try:
                msg = self.ring.consume(self.consumer, timeout_s=1.0, spin_us=self.busy_spin_us if busy else self.idle_spin_us)
            except RingClosed:
                return "closed"
            if msg is None:
                busy = False
                if not self._parent_alive():
                    return "orphaned"
                continue
            kind, buf = msg
            busy = kind in (KIND_DECODE, KIND_PREFILL, KIND_GATHER)
            try:
                if kind == KIND_STOP:
                    return "stop"
                if kind == KIND_DECODE:
                    n, bsz, want, meta = decode_decode_plan(buf)
                    ev = None
                    if self.timing is not None:
                        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                        ev[0].record()
                    _ids, logits = self.runner.decode_from_plan(n, bsz, want, meta)
                    if ev is not None:
                        ev[1].record()
                        self.timing.append(ev)
                    self.last_logits = logits
                    self.steps += 1
                elif kind in (KIND_PREFILL, KIND_PREFILL_KEEP):
                    self.last_logits = self.runner.prefill(decode_prefill_plan(buf, self.mm_table), keep_hidden=kind == KIND_PREFILL_KEEP)
                    self.steps += 1
                elif kind == KIND_MM_PUT:
                    mm = decode_mm(np.frombuffer(bytes(buf), dtype=np.uint8), model.device)
                    self.mm_table[mm.ctx_id] = mm
                elif kind == KIND_MM_DROP:
                    self.mm_table.pop(int.from_bytes(bytes(buf[:4]), "little", signed=True), None)
                elif kind == KIND_MTP:
                    a = buf.view(np.int32)
                    n = int(a[0])
                    tail = a[1 + n:]
                    self.last_logits = self.runner.mtp_pass(decode_prefill_plan(a[1:1 + n], self.mm_table), tail[2:2 + int(tail[1])].tolist(), int(tail[0]))
                    self.steps += 1
                elif kind == KIND_GATHER:
                    k = int.from_bytes(bytes(buf[:4]), "little") if len(buf) >= 4 else 0
                    if k > 0:
                        model.tp.comm.gather_candidates(self.last_logits, model.vocab_shard, k)
                    else:
                        model.tp.comm.gather_logits(self.last_logits, model.vocab_shard, model.cfg.vocab_size)
                elif kind == KIND_RESET:
                    self.runner.reset_after_device_error()
                elif kind == KIND_CALL:
                    req = json.loads(bytes(buf).decode())
                    fn = self.handlers.get(req["name"])
                    if fn is not None:
                        fn(**req.get("args", {}))
            except DeviceKernelError as e:
                # a bounded wait gave up (e.g. a peer that never arrived); rank 0 sees the same failure on its own
                # GPU, ends the requests in flight and publishes a reset, which arrives as the next message
                self.errors += 1
                print(f"[fastllm_b200 worker {self.consumer + 1}] device error: {e}", flush=True)
