"""Expert parallelism.

Experts are placed in contiguous blocks over the ranks of the tensor-parallel group (reference placement:
``devices[expert % ownerCount]``, src/devices/multicuda/multicudadevice.cpp:6226-6236; contiguous blocks here so
that a rank's experts form one stacked weight matrix for the grouped GEMM).

Attention runs tensor-parallel, so after its fused all-reduce every rank already holds every token's hidden state:
the *dispatch* half of the all-to-all is a no-op (the reference broadcasts the full hidden state for the same
reason, multicudadevice.cpp:5607-6009).  The *combine* half is where data crosses NVLink: each rank's weighted sum
over its local experts is pushed row-wise to the row owner (P2P stores from inside the kernel), reduced in rank
order, joined with the residual, RMS-normalised and multicast back -- ``csrc/comm.cu`` (``fb_moe_combine_ar_norm``),
one launch, no NCCL.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class EPInfo:
    rank: int = 0
    size: int = 1
    combines: bool = False      # moe_forward never returns the cross-rank sum itself; the decoder reduces it

    @staticmethod
    def from_tp(tp) -> "EPInfo | None":
        return EPInfo(tp.rank, tp.size) if tp is not None and tp.size > 1 else None
