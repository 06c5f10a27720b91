"""Model runner: turns scheduler decisions into device batches, owns the decode CUDA graphs.

Decode steps are captured once per batch-size bucket into a CUDA graph (whole layer stack + greedy
sampler) and replayed with new metadata, as the reference pre-captures per-batch-size decode graphs
after warm-up (src/models/qwen3.cpp:1632, 1723-2210).  Step metadata (token ids, positions, cache slots,
sequence lengths, page table) travels in ONE pinned host buffer -> ONE H2D copy per step.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..models.decoder import DecoderModel, ForwardBatch
from ..ops import _lib
from ..ops import attention as A
from ..ops import basic as B
from .kv_cache import KVCache


@dataclass
class EngineConfig:
    max_batch: int = 256
    max_context: int = 8192
    tp_candidate_sampling: bool = True     # vocab-sharded sampling exchanges per-rank top-k candidates instead of whole logit rows
    chunked_prefill_size: int = 8192
    gpu_mem_ratio: float = 0.9
    max_tokens: int | None = None
    prefill_page_limit: float = 0.8      # admit new prefills only while used pages stay below this fraction
    use_cuda_graph: bool = True
    graph_batch_sizes: list = field(default_factory=lambda: [1, 2, 4, 8, 16, 32, 64, 128, 256, 512])
    prefix_cache: bool = True
    page_len: int = A.PAGE_LEN
    check_device_errors_every: int = 64
    mixed_prefill_decode: bool = True    # a prefill step also advances the requests that are already decoding (one token each)
    speculative: str = ""                # "" | "ngram": drafts by looking the recent n-gram up in the request's own text | "mtp": drafts
                                         # from the checkpoint's multi-token-prediction head (falls back to "ngram" without one)
                                         # | "draft": from a separate smaller model given to the engine (``draft_model``)
    speculative_tokens: int = 4          # draft tokens verified per step
    speculative_ngram: int = 3           # longest suffix that is searched for (shorter ones are tried next)


class _DecodeSlot:
    """Static buffers (and the captured graph) of one decode batch-size bucket."""

    def __init__(self, runner: "ModelRunner", bsz: int):
        dev = runner.device
        P = runner.max_pages
        self.bsz = bsz
        n = 5 * bsz + bsz * P
        pin = dev.type == "cuda"
        self.meta_host = torch.zeros(n, dtype=torch.int32, pin_memory=pin)
        self.meta_np = self.meta_host.numpy()
        self.meta_dev = torch.zeros(n, dtype=torch.int32, device=dev)
        md = self.meta_dev
        self.ids, self.positions, self.slots, self.kv_lens, self.state_slots = (md[i * bsz:(i + 1) * bsz] for i in range(5))
        self.page_table = md[5 * bsz:].view(bsz, P)
        self.cu_q = torch.arange(bsz + 1, dtype=torch.int32, device=dev)
        self.out_ids = torch.zeros(bsz, dtype=torch.int32, device=dev)
        self.out_host = torch.zeros(bsz, dtype=torch.int32, pin_memory=pin)
        self.logits = None
        self.graph = None
        m = runner.model
        G = max(1, max([m.num_heads_local] + [lw.attn.heads or 0 for lw in m.layers]) // m.num_kv_heads_local)
        self.ws = None
        if dev.type == "cuda" and not m.cfg.use_mla:
            windows = {int(lw.attn.window) for lw in m.layers if lw.attn.window}
            # one sliding-window length per model is planned alongside the full list (layers alternate local / global)
            self.ws = A.DecodeWorkspace(bsz, m.num_kv_heads_local, G, P, dev, m.cfg.head_dim, window=windows.pop() if len(windows) == 1 else 0)

    def batch(self) -> ForwardBatch:
        return ForwardBatch(ids=self.ids, positions=self.positions, slots=self.slots, page_table=self.page_table,
                            kv_lens=self.kv_lens, cu_q=self.cu_q, logit_rows=None, is_decode=True,
                            cu_q_host=list(range(self.bsz + 1)), decode_ws=self.ws, state_slots=self.state_slots)


class ModelRunner:
    def __init__(self, model: DecoderModel, cfg: EngineConfig, num_pages: int | None = None):
        self.model = model
        self.cfg = cfg
        self.device = model.device
        self.max_pages = (cfg.max_context + cfg.page_len - 1) // cfg.page_len
        if num_pages is None:
            model._state_bytes_reserved = model.linear_state_bytes_per_slot() * (cfg.max_batch + 1)
            num_pages = KVCache.plan_num_pages(model, cfg.gpu_mem_ratio, cfg.max_tokens)
            num_pages = self._agree_on_pages(num_pages)
        self.state_slots = cfg.max_batch if model.cfg.has_linear_attn else 0
        self.kv = KVCache(model, num_pages, cfg.page_len, self.state_slots)
        self.control = None      # parallel.control.ControlPlane on the scheduler rank of a multi-process group
        self.slots: dict[int, _DecodeSlot] = {}
        self.graph_ok = cfg.use_cuda_graph and self.device.type == "cuda" and self._graph_safe()
        self.steps = 0
        self.kernel_launches = 0
        self.launches_per_decode_step = 0
        model.rope_tables()

    def _agree_on_pages(self, num_pages: int) -> int:
        """Page ids are chosen by the scheduler rank and used by every rank: all pools get the smallest planned size."""
        import torch.distributed as dist

        if self.model.tp.size > 1 and dist.is_available() and dist.is_initialized():
            dev = self.device if dist.get_backend() == "nccl" else torch.device("cpu")
            t = torch.tensor([num_pages], dtype=torch.int64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            num_pages = int(t.item())
        return num_pages

    def reset_after_device_error(self) -> None:
        """After a kernel reported a failed bounded wait: start a new epoch of the collective arena (every rank calls
        this together) and clear arrival counters a kernel that gave up may have left mid-count."""
        comm = getattr(self.model.tp, "comm", None)
        fused = getattr(comm, "fused", None) if comm is not None else None
        if fused is not None:
            fused.reset()
        for s in self.slots.values():
            if s.ws is not None:
                s.ws.counters.zero_()

    def _graph_safe(self) -> bool:
        c = self.model.cfg
        if getattr(self.model, "layer_devices", None) is not None:
            return False        # one graph cannot span the devices of a layer-split placement
        if c.use_mla and not (c.kv_lora_rank == 512 and c.qk_rope_head_dim == 64 and self.model.dtype in (torch.float16, torch.bfloat16)):
            return False        # latent shapes outside the MLA decode kernel run the PyTorch evaluation
        kvd = getattr(self.model, "kv_dtype", None)
        kv8 = kvd == torch.float8_e4m3fn and self.model.kv8_decode_ok
        if (self.model.general_attn and not kv8) or (kvd not in (None, self.model.dtype) and not kv8):
            return False        # these paths evaluate attention with host-synchronising PyTorch ops
        if len({int(lw.attn.window) for lw in self.model.layers if lw.attn.window}) > 1 or (c.rope_local_theta and any(lw.attn.window for lw in self.model.layers)):
            return False        # several window lengths / a second RoPE base for local layers: PyTorch evaluation
        if not c.use_mla and c.head_dim != 128:
            return False        # the tensor-core attention kernels cover head_dim 128; other widths run the PyTorch evaluation
        if c.has_linear_attn and not (c.lin_kind == "gdn" and c.lin_k_dim == 128 and c.lin_v_dim == 128
                                      and self.model.dtype in (torch.float16, torch.bfloat16)):
            return False        # delta-rule state shapes outside the recurrent kernel run the PyTorch evaluation
        if c.is_moe:
            # the per-expert fallback loop synchronises with the host; graphs need every MoE layer on the grouped kernels
            return all(lw.mlp.experts is None or (lw.mlp.experts.stacked is not None and not lw.mlp.experts.host)
                       for lw in self.model.layers)
        return True

    # ---------------------------------------------------------------------------------------------
    def prefill(self, chunks, keep_hidden: bool = False, mtp_hidden=None):
        """chunks: list of (token_ids, start_pos, pages, want_logits). Returns fp32 logits ``[R, V_local]``
        for the chunks that asked for them (last token of the chunk), in order.

        ``keep_hidden``: the final-normed rows of the whole packed batch stay in ``model.last_hidden`` (the draft head reads
        them).  ``mtp_hidden``: run the draft head instead of the decoder -- the chunks then hold, per position, the token that
        FOLLOWS it, ``mtp_hidden`` the matching hidden rows; returns (logits, the head's final-normed rows)."""
        if self.control is not None and mtp_hidden is None:
            self.control.prefill(chunks, keep_hidden)
        dev = self.device
        ids, pos, slots, cu, kv_lens, rows = [], [], [], [0], [], []
        P = self.max_pages
        pt = np.zeros((len(chunks), P), dtype=np.int32)
        pl = self.cfg.page_len
        sslots = []
        mm_rows, mm_vals, pos3 = [], [], []          # image-token rows of the packed batch, their embeddings, 3-D positions
        ex_rows = []                                 # rows that take a model's visual-expert weights
        any_mm = any(len(ch) > 5 and ch[5] is not None for ch in chunks)
        for b, ch in enumerate(chunks):
            toks, start, pages, want = ch[:4]
            if any_mm:
                mm = ch[5] if len(ch) > 5 else None
                if mm is not None:
                    offs, rws = mm.rows(start, len(toks))
                    if offs:
                        mm_rows.extend(cu[-1] + o for o in offs)
                        mm_vals.append(mm.embeds[rws])
                    pos3.append(mm.positions(start, len(toks)))
                    ex_rows.extend(cu[-1] + o for o in mm.expert_rows(start, len(toks)))
                else:
                    pos3.append(torch.arange(start, start + len(toks))[None].expand(3, -1))
            ss = ch[4] if len(ch) > 4 and ch[4] is not None and ch[4] >= 0 else self.state_slots     # default: the scratch slot
            sslots.append(ss)
            if self.state_slots and start == 0 and mtp_hidden is None:
                self.kv.reset_state(ss)              # a request starts (or restarts after an eviction) from empty state
            n = len(toks)
            ids.extend(toks)
            pos.extend(range(start, start + n))
            pg = np.asarray(pages, dtype=np.int64)
            p_idx = np.arange(start, start + n)
            slots.extend((pg[p_idx // pl] * pl + p_idx % pl).tolist())
            cu.append(cu[-1] + n)
            kv_lens.append(start + n)
            pt[b, :len(pages)] = pages
            if want:
                # True: the chunk's last row; an integer n > 1: its last n rows (speculative verification reads them all)
                nrows = 1 if want is True else max(1, min(int(want), n))
                rows.extend(range(cu[-1] - nrows, cu[-1]))
        T = len(ids)
        meta = torch.tensor(ids + pos + slots, dtype=torch.int32)
        if dev.type == "cuda":
            meta = meta.pin_memory().to(dev, non_blocking=True)
        fb = ForwardBatch(ids=meta[:T], positions=meta[T:2 * T], slots=meta[2 * T:3 * T],
                          page_table=torch.from_numpy(pt).to(dev), kv_lens=torch.tensor(kv_lens, dtype=torch.int32).to(dev),
                          cu_q=torch.tensor(cu, dtype=torch.int32).to(dev),
                          logit_rows=torch.tensor(rows, dtype=torch.long).to(dev) if rows else torch.zeros(0, dtype=torch.long, device=dev),
                          is_decode=False, cu_q_host=cu,
                          state_slots=torch.tensor(sslots, dtype=torch.int32).to(dev) if self.state_slots else None,
                          state_slots_host=sslots if self.state_slots else None)
        if not rows:
            # still run the stack to fill the cache; ask for one row to keep shapes valid
            fb.logit_rows = torch.zeros(1, dtype=torch.long, device=dev)
        if any_mm:
            fb.rope_pos3 = torch.cat(pos3, dim=1)
            if mm_rows and mtp_hidden is None:
                fb.embed_rows = torch.tensor(mm_rows, dtype=torch.long, device=dev)
                fb.embed_vals = torch.cat(mm_vals, dim=0).to(dev)
            if ex_rows:
                fb.expert_rows = torch.tensor(ex_rows, dtype=torch.long, device=dev)
        fb.kv_max_host = max(kv_lens) if kv_lens else 0
        if mtp_hidden is not None:
            logits, x = self.model.mtp_forward(fb, mtp_hidden, self.kv.pools)
            return (logits if rows else None), x
        fb.keep_hidden = keep_hidden
        logits = self.model.forward(fb, self.kv.pools)
        self.steps += 1
        return logits if rows else None

    def mtp_pass(self, chunks, sel, src: int):
        """One pass of the draft head over ``chunks`` (per position, the token that follows it); its hidden input rows are rows
        ``sel`` of the decoder's last kept pass (``src`` 0) or of the head's own last pass (``src`` 1: chained drafts).  Worker
        ranks replay the same call from the published plan.  Returns the logits of the rows that asked for them."""
        if self.control is not None:
            self.control.mtp(chunks, sel, src)
        base = self.model.last_hidden if src == 0 else self._mtp_x
        idx = torch.tensor(list(sel), dtype=torch.long, device=base.device)
        logits, x = self.prefill(chunks, mtp_hidden=base.index_select(0, idx))
        self._mtp_x = x
        return logits

    # ---------------------------------------------------------------------------------------------
    def _bucket(self, n: int) -> int:
        for b in self.cfg.graph_batch_sizes:
            if b >= n:
                return b
        return n

    def _get_slot(self, bsz: int) -> _DecodeSlot:
        s = self.slots.get(bsz)
        if s is None:
            s = _DecodeSlot(self, bsz)
            self.slots[bsz] = s
        return s

    def _decode_forward(self, s: _DecodeSlot):
        fb = s.batch()
        fb.kv_max_host = getattr(s, "kv_max_host", 0)
        if s.ws is not None:
            s.ws.plan(s.kv_lens)
            fb.decode_planned = True
        logits = self.model.forward(fb, self.kv.pools)
        s.logits = logits
        self._greedy(logits, s.out_ids)

    def _greedy(self, logits, out_ids):
        m = self.model
        if m.tp.size == 1:
            B.argmax(logits, out=out_ids)
        else:
            lo, hi = m.vocab_shard
            lg = logits
            if hi - lo < lg.shape[1]:
                lg = lg[:, :hi - lo]
            ids, vals = B.argmax(lg, id_offset=lo, want_values=True)
            out_ids.copy_(m.tp.comm.merge_argmax(ids, vals))

    def decode(self, ids, positions, pages_per_req, want_logits=False, state_slots=None, rope_offsets=None):
        """One token per request. Returns (token ids int32 host tensor [n], logits or None).  ``rope_offsets``: per request,
        what is added to the token's index to get its rotary position (prompts with images)."""
        n = len(ids)
        pl = self.cfg.page_len
        bsz = self._bucket(n) if self.graph_ok else n
        s = self._get_slot(bsz)
        mp = s.meta_np
        mp[:4 * bsz] = 0
        mp[2 * bsz:3 * bsz] = -1                      # padded rows never write the cache
        mp[4 * bsz:5 * bsz] = self.state_slots        # ... and keep their linear-attention state in the scratch slot
        mp[0:n] = ids
        mp[bsz:bsz + n] = positions
        if state_slots is not None:
            mp[4 * bsz:4 * bsz + n] = state_slots
        pt = mp[5 * bsz:].reshape(bsz, self.max_pages)
        for b in range(n):
            pg = pages_per_req[b]
            p = positions[b]
            mp[2 * bsz + b] = pg[p // pl] * pl + p % pl
            mp[3 * bsz + b] = p + 1
            pt[b, :len(pg)] = pg
        if rope_offsets is not None:
            mp[bsz:bsz + n] += np.asarray(rope_offsets, dtype=mp.dtype)
        s.kv_max_host = (max(positions) + 1) if n else 0
        if self.control is not None:
            self.control.decode(n, bsz, want_logits, mp)
        return self._run_decode(s, n, want_logits)

    def decode_from_plan(self, n: int, bsz: int, want_logits: bool, meta):
        """A worker rank's decode step: the metadata buffer arrives ready-made from the scheduler rank."""
        s = self._get_slot(bsz)
        s.meta_np[:] = meta
        s.kv_max_host = int(s.meta_np[3 * bsz:3 * bsz + n].max()) if n else 0
        return self._run_decode(s, n, want_logits)

    def _run_decode(self, s: _DecodeSlot, n: int, want_logits: bool):
        s.meta_dev.copy_(s.meta_host, non_blocking=True)
        # sparse-attention models: once a context outgrows the indexer's selection size the step selects keys per request
        # (host-synchronising tensor ops), outside the captured graph
        topk = self.model.cfg.index_topk if getattr(self.model, "has_indexer", False) else 0
        if self.graph_ok and not (topk and getattr(s, "kv_max_host", 0) > topk):
            if s.graph is None:
                self._capture(s)
            s.graph.replay()
        else:
            c0 = _lib.launch_count()
            self._decode_forward(s)
            self.launches_per_decode_step = _lib.launch_count() - c0
        s.out_host.copy_(s.out_ids, non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        self.steps += 1
        if self.device.type == "cuda" and self.steps % self.cfg.check_device_errors_every == 0:
            _lib.check_device_errors()
        logits = s.logits[:n] if want_logits else None
        return s.out_host[:n], logits

    def _capture(self, s: _DecodeSlot):
        # warm-up run outside capture (lazy inits, tensor-map cache, cudaFuncSetAttribute), then capture.
        # Writing K/V twice to the same cache slot is harmless, advancing a recurrent state twice is not: the warm-up run
        # works on the scratch state slot, the requests' own slots are put back before the first replay.
        saved_slots = None
        if self.state_slots:
            saved_slots = s.state_slots.clone()
            s.state_slots.fill_(self.state_slots)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._decode_forward(s)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        c0 = _lib.launch_count()
        with torch.cuda.graph(g):
            self._decode_forward(s)
        self.launches_per_decode_step = _lib.launch_count() - c0
        s.graph = g
        if saved_slots is not None:
            s.state_slots.copy_(saved_slots)
        torch.cuda.synchronize()
