"""Symmetric peer-memory arena and the fused tensor-parallel kernels that run on it.

``torch.distributed._symmetric_memory`` does the plumbing only: it allocates one arena per rank, exchanges
the handles and returns every peer's pointer plus the NVSwitch multicast mapping.  All data movement is
done by our own kernels (``csrc/comm.cu``) with P2P or ``multimem`` loads/stores; no NCCL call is made
on the decode path.  (Reference counterpart: peer-access setup + custom all-reduce buffers,
src/devices/multicuda/fastllm-custom-allreduce.cu:2234-2481.)

Arena layout (same offsets on every rank):
    [0, 1 KiB)          counters / expected value / ticket
    part   fp32 [tp, max_m, max_n] slot s = partial rows pushed by rank s (reduce-scatter by push)
    h      16-bit [max_m, hidden]  residual stream (replicated, written by the row owners)
    x      16-bit [max_m, hidden]  RMSNorm(h) for the next column-parallel GEMM
    amax   [tp, max_m, 2] u32      greedy candidates of the vocab shards
    big    (only when ``max_big_m`` > 256) second header (per-row-block ready / expect / done words, job ticket) and
           src 16-bit [max_big_m, hidden]: this rank's partial sums of a prefill-sized batch, read by every rank through
           the multicast mapping; h and x are then sized for ``max_big_m`` rows
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import basic as B
from ..ops.basic import _ptr, _stream, dtype_code

P, I, F, ULL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_ulonglong
_lib.register_sigs({
    "fb_gemm_ar_norm": [P, P, P, I, I, I, I, I, P, P, P, I, I, ULL, ULL, ULL, P, I, F, F, I, I, P],
    "fb_ar_norm": [P, I, I, I, P, P, P, I, I, ULL, ULL, ULL, P, I, F, F, I, P],
    "fb_argmax_merge": [P, P, P, I, P, P, P, I, I, ULL, P],
    "fb_moe_combine_ar_norm": [P, P, P, P, I, I, I, P, P, P, I, I, ULL, ULL, ULL, P, I, F, F, I, P],
    "fb_comm_wait": [P, P],
    "fb_gemm_fp8_ar_norm": [P, I, P, I, P, P, P, I, I, I, P, P, P, I, I, ULL, ULL, ULL, P, I, F, F, I, P],
    "fb_gemm_i8_ar_norm": [P, I, P, P, I, P, P, P, P, I, I, I, I, P, P, P, I, I, ULL, ULL, ULL, P, I, F, F, I, P],
    "fb_gemm_ar_norm_big": [P, P, P, I, I, I, I, I, P, P, P, I, I, ULL, ULL, ULL, ULL, P, I, F, F, I, P],
    "fb_ar_norm_big": [P, I, I, I, P, P, P, I, I, ULL, ULL, ULL, ULL, P, I, F, F, I, P],
}, ["comm", "comm_prefill"])
OFF_CNT2, OFF_EXPECT = 128, 256      # arena header words the deferred all-gather wait reads (csrc/comm.cu)

HEADER = 1024
BIG_HEADER = (3 * 512 + 1) * 4      # ready / expect / done words of 512 row blocks + the job ticket (csrc/comm_prefill.cu)
SMALL_M = 256                       # rows the latency-regime kernels take; above it the bandwidth-regime kernels run


def _align(n, a=4096):
    return (n + a - 1) // a * a


class FusedComm:
    name = "fused-p2p"

    def __init__(self, comm, hidden: int, max_m: int, max_n: int, dtype=torch.bfloat16, use_multicast: bool = True,
                 max_big_m: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        self.comm = comm
        self.rank, self.tp, self.device = comm.rank, comm.size, comm.device
        self.hidden, self.max_m, self.max_n, self.dtype = hidden, max_m, max(max_n, hidden), dtype
        self.max_big_m = max_big_m if (max_big_m > SMALL_M and hidden <= 8192 and max_big_m <= 65536) else 0
        rows = max(max_m, self.max_big_m)          # h / x hold whichever batch is larger
        self.off_part = _align(HEADER)
        self.off_h = _align(self.off_part + self.tp * max_m * self.max_n * 4)
        self.off_x = _align(self.off_h + rows * hidden * 2)
        self.off_amax = _align(self.off_x + rows * hidden * 2)
        self.off_bighdr = _align(self.off_amax + self.tp * max_m * 8)
        self.off_src = _align(self.off_bighdr + BIG_HEADER)
        self.nbytes = _align(self.off_src + self.max_big_m * hidden * 2, 1 << 21)
        self.arena = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.arena, dist.group.WORLD)
        self.arena.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        ptrs = list(self.handle.buffer_ptrs)
        self.peers = (ctypes.c_void_p * 8)(*([ctypes.c_void_p(p) for p in ptrs] + [ctypes.c_void_p(0)] * (8 - len(ptrs))))
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if not use_multicast or os.environ.get("FB_DISABLE_MULTICAST", "0") == "1":
            mc = 0
        self.mc = mc
        # The prefill-sized kernels move whole activations.  A multicast reduction load makes NVSwitch fetch the row from
        # every rank, the requester included, so with two ranks it puts 3x the bytes of plain peer loads on the links
        # (measured, 8192 x 4096 rows: reduce phase 159 us against 96 us); from four ranks on the in-switch sum moves fewer
        # bytes than tp - 1 peer loads.  FB_BIG_MULTICAST=0 / 1 overrides.
        big = os.environ.get("FB_BIG_MULTICAST", "auto")
        self.big_mc = mc if (big == "1" or (big == "auto" and self.tp >= 4)) else 0
        self.name = "fused-nvls-multimem" if mc else "fused-p2p"
        self.local = ptrs[self.rank]
        assert self.local == self.arena.data_ptr()
        self.h_buf = self.arena[self.off_h:self.off_h + rows * hidden * 2].view(dtype).view(rows, hidden)
        self.x_buf = self.arena[self.off_x:self.off_x + rows * hidden * 2].view(dtype).view(rows, hidden)
        self.trace = False          # True: kernels stamp their phases (read back with read_trace)
        self.poison = os.environ.get("FB_ARENA_POISON", "0") == "1"

    # ---------------------------------------------------------------------------------------------
    def usable(self, M: int, N: int) -> bool:
        return 0 < M <= max(min(self.max_m, SMALL_M), self.max_big_m) and N == self.hidden and N % 8 == 0

    def _big(self, M: int) -> bool:
        """Prefill-sized batch: the bandwidth-regime kernels (row blocks of 128 owned round-robin) take it."""
        return M > min(self.max_m, SMALL_M)

    def load_h(self, h: torch.Tensor) -> torch.Tensor:
        """Place the (replicated) residual stream rows into the arena; returns the arena view."""
        B.flush_pending_wait()
        M = h.shape[0]
        if self.poison:
            # debug aid: everything a forward pass may read from the arena without having written it first becomes NaN
            # (0xFF bytes are NaN in bf16 / fp16 / fp32), so a stale partial slot or a row that was never broadcast shows up
            # in the logits instead of passing as plausible old data.  All ranks do this at the same point of the step.
            torch.cuda.synchronize()
            dist.barrier()
            self.arena[self.off_part:self.off_amax].fill_(0xFF)
            if self.max_big_m:
                self.arena[self.off_src:self.off_src + self.max_big_m * self.hidden * 2].fill_(0xFF)
            torch.cuda.synchronize()
            dist.barrier()
        v = self.h_buf[:M]
        v.copy_(h)
        return v

    def _flags(self, has_residual: bool, defer: bool) -> int:
        return (1 if has_residual else 0) | (2 if self.trace else 0) | (4 if defer else 0)

    def _after_launch(self, defer: bool) -> None:
        if defer:
            B.set_pending_wait(self.local + OFF_CNT2, self.local + OFF_EXPECT, self.wait_all_gather)

    def wait_all_gather(self) -> None:
        """Stand-alone wait for a deferred all-gather (used when the next consumer is not a kernel that waits itself)."""
        _lib.check(_lib.kernels().fb_comm_wait(ctypes.c_void_p(self.local), _stream()), "fb_comm_wait")

    def gemm_ar_norm(self, w, x: torch.Tensor, ln_w, eps: float, unit_offset: float = 0.0, has_residual: bool = True,
                     defer: bool = False):
        """h[:M] (+)= sum over ranks of x @ w.T ; x_out = RMSNorm(h) * ln_w.  One launch.  Returns (h, x_out) views; of
        ``h`` only this rank's own rows are current (the residual stream stays with the row owner).

        ``defer``: the kernel ends after broadcasting its rows, without waiting for the peers' rows; the next ``linear``
        on this stream waits inside its GEMM, after its weight prefetch (``ops.basic.set_pending_wait``)."""
        M, K = x.shape
        N = w.n
        if w.kind != "dense" and self.usable(M, N) and not self._big(M):
            return self._gemm_ar_norm_quant(w, x, ln_w, eps, unit_offset, has_residual, defer)
        if w.kind != "dense" or not self.usable(M, N) or (w.bias is not None and self.rank != 0 and False):
            return None
        wt = w.w if w.w.dtype == x.dtype else w.w.to(x.dtype)
        bias = w.bias if self.rank == 0 else None
        if self._big(M):
            if K % 64 != 0 or x.stride(1) != 1 or os.environ.get("FB_FUSED_PREFILL_GEMM", "1") == "0":
                return None
            rc = _lib.kernels().fb_gemm_ar_norm_big(_ptr(x), _ptr(wt), _ptr(bias), M, N, K, x.stride(0), wt.stride(0),
                                                    ctypes.c_void_p(self.local), ctypes.c_void_p(self.big_mc), self.peers, self.rank, self.tp,
                                                    self.off_bighdr, self.off_src, self.off_h, self.off_x, _ptr(ln_w),
                                                    self._flags(has_residual, False), float(eps), float(unit_offset), dtype_code(x.dtype), _stream())
            _lib.check(rc, "fb_gemm_ar_norm_big")
            return self.h_buf[:M], self.x_buf[:M]
        rc = _lib.kernels().fb_gemm_ar_norm(_ptr(x), _ptr(wt), _ptr(bias), M, N, K, x.stride(0), wt.stride(0),
                                            ctypes.c_void_p(self.local), ctypes.c_void_p(self.mc), self.peers, self.rank, self.tp,
                                            self.off_part, self.off_h, self.off_x, _ptr(ln_w),
                                            self._flags(has_residual, defer), float(eps), float(unit_offset), dtype_code(x.dtype), 0, _stream())
        if rc != 0:
            if rc == 701:      # cudaErrorLaunchOutOfResources: grid cannot be co-resident -> caller uses the unfused path
                return None
            _lib.check(rc, "fb_gemm_ar_norm")
        self._after_launch(defer)
        return self.h_buf[:M], self.x_buf[:M]

    def _gemm_ar_norm_quant(self, w, x, ln_w, eps, unit_offset, has_residual, defer):
        """Quantised row-parallel weights on the 8-bit-activation tensor-core kernels (fp8 W8A8, int8 / int4-group with int8
        activations), fused with the same collective tail.  None: the shape is outside those kernels (caller: GEMM, then
        ``ar_norm``)."""
        from ..ops import quant_gemm as QG

        M, K = x.shape
        N = w.n
        if x.dtype not in (torch.float16, torch.bfloat16) or K % 128 != 0 or x.stride(-1) != 1 or x.stride(0) % 4 != 0 or w.adapters:
            return None
        if os.environ.get("FB_FUSED_QUANT_AR", "1") == "0":
            return None
        pre = getattr(x, "fb_quant", None)
        bias = w.bias if self.rank == 0 else None
        if bias is not None and bias.dtype != x.dtype:
            bias = bias.to(x.dtype)
        lib = _lib.kernels()
        arena = (ctypes.c_void_p(self.local), ctypes.c_void_p(self.mc), self.peers, self.rank, self.tp, self.off_part, self.off_h, self.off_x,
                 _ptr(ln_w), self._flags(has_residual, defer), float(eps), float(unit_offset), dtype_code(x.dtype), _stream())
        if w.kind == "fp8" and QG.FP8_NATIVE and M <= 128:
            if pre is not None and pre[0] == 2 and pre[1].shape == (M, K):
                _, xq, sa, _xs, ld_a = pre
            else:
                xq, sa, ld_a = QG.quant_act_fp8(x)
            rc = lib.fb_gemm_fp8_ar_norm(_ptr(xq), K, _ptr(sa), ld_a, _ptr(w.w), _ptr(QG._kernel_tensors(w)[0]), _ptr(bias), M, N, K, *arena)
        elif QG.uses_int_a8(w) and M <= QG.INT_A8_MAX_M[w.kind]:
            wq, sc, zr, kind = QG._a8_tensors(w)
            if pre is not None and pre[0] == 1 and pre[1].shape == (M, K):
                _, xq, sa, xs, ld_a = pre
            else:
                xq, sa, xs, ld_a = QG.quant_act_i8(x)
            rc = lib.fb_gemm_i8_ar_norm(_ptr(xq), K, _ptr(sa), _ptr(xs), ld_a, _ptr(wq), _ptr(sc), _ptr(zr), _ptr(bias), M, N, K, kind, *arena)
        else:
            return None
        if os.environ.get("FB_DEBUG_FUSED") == "1" and self.rank == 0:
            print(f"[fused quant] kind={w.kind} M={M} N={N} K={K} pre={'yes' if pre is not None else 'no'} rc={rc}", flush=True)
        if rc == 701:          # the grid cannot be co-resident: unfused path
            return None
        _lib.check(rc, "fb_gemm_quant_ar_norm")
        self._after_launch(defer)
        return self.h_buf[:M], self.x_buf[:M]

    def ar_norm(self, partial: torch.Tensor, ln_w, eps: float, unit_offset: float = 0.0, has_residual: bool = True,
                defer: bool = False):
        """Same as gemm_ar_norm for a partial sum computed elsewhere (any float dtype, ``[M, hidden]``)."""
        M, N = partial.shape
        if not self.usable(M, N):
            return None
        if partial.dtype not in (torch.float32, self.dtype) or not partial.is_contiguous():
            partial = partial.to(self.dtype).contiguous()
        if self._big(M):
            rc = _lib.kernels().fb_ar_norm_big(_ptr(partial), 1 if partial.dtype == torch.float32 else 0, M, N, ctypes.c_void_p(self.local),
                                               ctypes.c_void_p(self.big_mc), self.peers, self.rank, self.tp, self.off_bighdr, self.off_src,
                                               self.off_h, self.off_x, _ptr(ln_w), self._flags(has_residual, False), float(eps),
                                               float(unit_offset), dtype_code(self.dtype), _stream())
            _lib.check(rc, "fb_ar_norm_big")
            return self.h_buf[:M], self.x_buf[:M]
        rc = _lib.kernels().fb_ar_norm(_ptr(partial), 1 if partial.dtype == torch.float32 else 0, M, N, ctypes.c_void_p(self.local), ctypes.c_void_p(self.mc), self.peers, self.rank, self.tp,
                                       self.off_part, self.off_h, self.off_x, _ptr(ln_w),
                                       self._flags(has_residual, defer), float(eps),
                                       float(unit_offset), dtype_code(self.dtype), _stream())
        _lib.check(rc, "fb_ar_norm")
        self._after_launch(defer)
        return self.h_buf[:M], self.x_buf[:M]

    def moe_combine_ar_norm(self, ys, pos, w, add, ln_w, eps: float, unit_offset: float = 0.0, has_residual: bool = True,
                            defer: bool = False):
        """Expert-parallel combine: weighted sum of this rank's expert outputs (+ ``add``) formed inside the kernel that
        pushes it to the row owners, reduces over ranks, adds the residual, normalises and broadcasts.  One launch."""
        M, topk = pos.shape
        N = self.hidden
        if not (0 < M <= min(self.max_m, SMALL_M)) or ys.shape[1] != N:
            return None
        rc = _lib.kernels().fb_moe_combine_ar_norm(_ptr(ys), _ptr(pos), _ptr(w), _ptr(add), topk, M, N, ctypes.c_void_p(self.local),
                                                   ctypes.c_void_p(self.mc), self.peers, self.rank, self.tp, self.off_part, self.off_h,
                                                   self.off_x, _ptr(ln_w), self._flags(has_residual, defer),
                                                   float(eps), float(unit_offset), dtype_code(self.dtype), _stream())
        _lib.check(rc, "fb_moe_combine_ar_norm")
        self._after_launch(defer)
        return self.h_buf[:M], self.x_buf[:M]

    # -- TPComm hooks --------------------------------------------------------------------------------
    def all_reduce(self, t, residual=None):
        return None        # generic tensors go through NCCL; the decoder calls the fused entry points directly

    def row_linear(self, w, x, residual):
        return None

    def merge_argmax(self, ids: torch.Tensor, vals: torch.Tensor):
        n = ids.shape[0]
        if n > self.max_m:
            return None
        B.flush_pending_wait()
        out = torch.empty_like(ids)
        rc = _lib.kernels().fb_argmax_merge(_ptr(vals), _ptr(ids), _ptr(out), n, ctypes.c_void_p(self.local),
                                            ctypes.c_void_p(self.mc), self.peers, self.rank, self.tp, self.off_amax, _stream())
        _lib.check(rc, "fb_argmax_merge")
        return out

    def read_trace(self):
        """Phase time stamps (ns, device global timer) of CTA 0 in the last traced launch:
        [start, sync1 arrive begin, sync1 arrive end, sync1 wait end, sync2 arrive begin, sync2 arrive end, sync2 wait end]."""
        torch.cuda.synchronize()
        return self.arena[768:768 + 56].view(torch.int64).cpu().tolist()

    def reset(self):
        """Re-initialise the counters after a reported peer timeout (all ranks must call this together)."""
        torch.cuda.synchronize()
        dist.barrier()
        self.arena[:HEADER].zero_()
        self.arena[self.off_bighdr:self.off_bighdr + BIG_HEADER].zero_()
        torch.cuda.synchronize()
        dist.barrier()


def prefill_rows(engine_cfg) -> int:
    """Largest token batch one forward pass of this engine can carry: a prefill chunk plus the decode rows mixed into it
    (0 turns the bandwidth-regime kernels off: FB_FUSED_PREFILL=0)."""
    if os.environ.get("FB_FUSED_PREFILL", "1") == "0":
        return 0
    return min(65536, int(engine_cfg.chunked_prefill_size) + int(engine_cfg.max_batch))


def try_create(comm, cfg, max_m: int, strict: bool = False, dtype=torch.bfloat16, max_big_m: int = 0):
    """Create the fused communicator; on failure return None (NCCL path) unless ``strict``.  ``max_big_m`` > 256 also
    reserves the buffers of the prefill-sized (bandwidth-regime) kernels for that many token rows."""
    try:
        max_m = max(16, min(256, max_m))
        return FusedComm(comm, cfg.hidden_size, max_m, cfg.hidden_size, dtype, max_big_m=max_big_m)
    except Exception as e:  # symmetric memory unavailable (no P2P, old driver, ...)
        if strict:
            raise
        if comm.rank == 0:
            print(f"[fastllm_b200] fused NVLink path unavailable ({e!r}); using NCCL collectives", flush=True)
        return None
