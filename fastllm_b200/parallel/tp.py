"""Tensor-parallel communication for one-process-per-GPU execution.

``TPComm`` offers the collectives the decoder needs -- all-reduce (+residual) after the row-parallel
GEMMs, the vocab-sharded greedy merge and logits gather -- with two back ends:

* ``nccl``: ``torch.distributed`` collectives.  This is the plumbing / baseline path and the CPU (gloo)
  test path.  It matches what the reference does: local GEMM, rank 0 adds the residual, then one
  all-reduce per row-parallel linear (src/models/qwen3.cpp:825-859).
* ``fused``: hand-written kernels over NVLink peer memory (``parallel/symm.py`` + ``csrc/comm.cu``):
  one-shot all-reduce + residual + RMSNorm in a single launch, no NCCL call on the decode path.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


class TPComm:
    def __init__(self, rank: int, size: int, device, group=None, backend: str = "nccl"):
        self.rank, self.size, self.device = rank, size, torch.device(device)
        self.group = group
        self.backend = backend
        self.fused = None        # parallel.symm.FusedComm when the peer-memory path is active
        self.launches = 0

    # -- collectives ---------------------------------------------------------------------------------
    def all_reduce(self, t: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if self.fused is not None and t.is_cuda:
            out = self.fused.all_reduce(t, residual)
            if out is not None:
                return out
        dist.all_reduce(t, group=self.group)
        if residual is not None:
            t = t + residual
        return t

    def row_linear(self, w, x, residual):
        """Partial GEMM on this rank's input shard; rank 0 folds the residual into its partial sum."""
        if self.fused is not None and x.is_cuda:
            out = self.fused.row_linear(w, x, residual)
            if out is not None:
                return out
        part = w(x, residual=residual if self.rank == 0 else None)
        dist.all_reduce(part, group=self.group)
        return part

    def merge_argmax(self, ids: torch.Tensor, vals: torch.Tensor) -> torch.Tensor:
        """Combine per-rank (arg-max id, max value) of vocab shards into the global arg-max (int32 [B]).
        Ties resolve to the lowest rank, i.e. the lowest token id (reference: sharded greedy merge,
        src/devices/cuda/fastllm-cuda.cu:13878)."""
        if self.fused is not None and ids.is_cuda:
            out = self.fused.merge_argmax(ids, vals)
            if out is not None:
                return out
        packed = torch.stack([vals.float(), ids.float()], dim=0).contiguous()          # [2, B]
        flat = torch.empty((self.size * 2, ids.shape[0]), device=ids.device, dtype=torch.float32)
        dist.all_gather_into_tensor(flat, packed, group=self.group)
        allp = flat.view(self.size, 2, ids.shape[0])
        best = allp[:, 0, :].argmax(dim=0, keepdim=True)                                  # first max = lowest rank
        return allp[:, 1, :].gather(0, best).squeeze(0).to(torch.int32)

    def gather_logits(self, logits: torch.Tensor, shard, vocab: int) -> torch.Tensor:
        """All-gather vocab-sharded logits ``[R, V_local]`` into ``[R, vocab]``."""
        R, VL = logits.shape
        flat = torch.empty((self.size * R, VL), device=logits.device, dtype=logits.dtype)
        dist.all_gather_into_tensor(flat, logits.contiguous(), group=self.group)
        allp = flat.view(self.size, R, VL)
        return allp.permute(1, 0, 2).reshape(R, self.size * VL)[:, :vocab].contiguous()

    def gather_candidates(self, logits: torch.Tensor, shard, k: int):
        """Sampling without moving the whole vocabulary: every rank sends the ``k`` largest logits of its vocab shard with
        their token ids.  Returns (values fp32 ``[R, tp * k]``, global ids int64 ``[R, tp * k]``); the global top-``k`` of
        every row is among them.  One all-gather of ``R * 2k`` floats per rank instead of ``R * V / tp``."""
        R, VL = logits.shape
        lo, hi = shard
        lg = logits.float()
        if hi - lo < VL:                      # rows of the padded shard beyond the vocabulary never win
            lg = lg.clone()
            lg[:, hi - lo:] = float("-inf")
        k = max(1, min(int(k), VL))
        v, i = torch.topk(lg, k, dim=-1)
        pack = torch.cat([v, (i + lo).float()], dim=-1).contiguous()           # ids < 2^24: exact in fp32
        flat = torch.empty((self.size * R, 2 * k), device=logits.device, dtype=torch.float32)
        dist.all_gather_into_tensor(flat, pack, group=self.group)
        allp = flat.view(self.size, R, 2 * k).permute(1, 0, 2)
        return allp[:, :, :k].reshape(R, self.size * k).contiguous(), allp[:, :, k:].reshape(R, self.size * k).long().contiguous()

    def barrier(self):
        dist.barrier(group=self.group)


def init_distributed(backend: str | None = None):
    """Initialise torch.distributed from the torchrun environment. Returns (rank, world, local_rank)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, rank=rank, world_size=world, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world)
    return rank, world, local
