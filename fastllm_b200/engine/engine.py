"""Continuous-batching engine: admission, prefix reuse, chunked prefill, decode, eviction, result queues.

Behaviour follows the reference's new main loop (src/models/basellm.cpp:1262-2663):
* waiting requests are admitted while used pages stay under ``prefill_page_limit`` (80 %) of the pool,
  longest-first among the pending ones;
* prompts are looked up in the page trie and only the uncached tail is prefilled, in chunks of
  ``chunked_prefill_size`` tokens;
* when a decode step cannot get a page, the longest decoding request is evicted and later recomputed;
* results are pushed to per-handle queues; ``launch`` / ``fetch`` / ``abort`` mirror
  LaunchResponseTokens / FetchResponseTokens / AbortResponse (basellm.cpp:2665+).
"""
from __future__ import annotations

import queue
import threading
import time
import traceback

import torch

from ..models.decoder import DecoderModel
from ..ops import _lib
from . import sampling
from .request import GenerationConfig, Request, RequestState
from .runner import EngineConfig, ModelRunner


class MultimodalContext:
    """What a prompt with images carries beside its token ids: the image tokens' embeddings (rows of the language model's
    width, in prompt order), the prompt positions they replace, the (time, row, column) rotary positions of every prompt
    token and the offset between a later token's rotary position and its index in the sequence."""

    def __init__(self, embeds, embed_positions, pos3, delta: int, expert_positions=None):
        self.embeds = embeds                                  # [n, H]
        self.embed_positions = list(embed_positions)          # n prompt indices, ascending
        self.pos3 = pos3                                      # int64 [3, prompt_len]
        self.delta = int(delta)
        self._row_of = {p: i for i, p in enumerate(self.embed_positions)}
        # prompt indices whose rows run through a model's second set of layer weights (CogVLM's visual expert)
        self.expert_positions = frozenset(expert_positions or ())

    def expert_rows(self, start: int, n: int):
        """Offsets inside the chunk ``[start, start + n)`` of the rows that take the model's visual-expert weights."""
        return [p - start for p in range(start, start + n) if p in self.expert_positions] if self.expert_positions else []

    def rows(self, start: int, n: int):
        """(offsets inside the chunk ``[start, start + n)``, embedding rows) of the image tokens in that chunk."""
        offs, rows = [], []
        for p in range(start, start + n):
            i = self._row_of.get(p)
            if i is not None:
                offs.append(p - start)
                rows.append(i)
        return offs, rows

    def positions(self, start: int, n: int):
        """int64 ``[3, n]`` rotary positions of the chunk: from the prompt's table, then ``index + delta`` on all axes."""
        import torch

        L = self.pos3.shape[1]
        a = self.pos3[:, start:min(L, start + n)]
        if start + n > L:
            tail = torch.arange(max(start, L), start + n) + self.delta
            a = torch.cat([a, tail[None].expand(3, -1)], dim=1)
        return a


class LLMEngine:
    def __init__(self, model: DecoderModel, cfg: EngineConfig | None = None, num_pages: int | None = None,
                 eos_token_ids=None, control=None, draft_model: DecoderModel | None = None):
        """``draft_model``: a smaller model with the same vocabulary that proposes tokens for ``speculative="draft"``.  Its KV
        pools have as many pages as the target's and are indexed by the same page ids, so a request's page list serves both."""
        self.cfg = cfg or EngineConfig()
        self.model = model
        if draft_model is not None:
            model._extra_page_bytes = draft_model.kv_bytes_per_page()       # the page plan leaves room for the draft's pools
        self.runner = ModelRunner(model, self.cfg, num_pages)
        self.draft: ModelRunner | None = None
        if draft_model is not None:
            import dataclasses

            if control is not None or model.tp.size > 1:
                raise NotImplementedError("a separate draft model runs on one rank")
            if self.runner.state_slots or any(lw.lin is not None for lw in draft_model.layers):
                raise NotImplementedError("draft-model speculation needs attention-only target and draft models")
            if draft_model.cfg.vocab_size != model.cfg.vocab_size:
                raise ValueError("the draft model's vocabulary differs from the target's")
            self.draft = ModelRunner(draft_model, dataclasses.replace(self.cfg, use_cuda_graph=False, speculative=""), self.runner.kv.num_pages)
        self.control = control          # parallel.control.ControlPlane: this rank schedules, the other ranks replay its plans
        self.runner.control = control
        # models with linear-attention layers keep per-request recurrent state in slots; whole-page prefix reuse would need
        # state snapshots at the page boundaries, so it is off for them
        self.state_free = list(range(self.runner.state_slots))
        if self.runner.state_slots:
            self.cfg.prefix_cache = False
        self.pm = self.runner.kv.manager
        self.page_len = self.cfg.page_len
        self.eos = set(eos_token_ids if eos_token_ids is not None else model.cfg.eos_token_ids)
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self.requests: dict[int, Request] = {}
        self.lock = threading.Lock()
        self.cv = threading.Condition(self.lock)
        self._thread: threading.Thread | None = None
        self._stop = False
        self.step_count = 0
        self.decode_steps = 0
        self.device_errors = 0
        self.last_device_error = ""
        self.decode_tokens = 0
        self.spec_proposed = 0          # speculative decoding: draft tokens verified / accepted so far
        self.spec_accepted = 0
        self.error: Exception | None = None     # the last exception a scheduler step raised (kept for diagnosis)
        self.dead = False                       # the background loop gave up after repeated failures

    # ----------------------------------------------------------------------------------- public API
    def launch(self, prompt_ids, gen: GenerationConfig | None = None, handle: int | None = None, mm=None) -> int:
        """``mm``: a ``MultimodalContext`` for prompts whose placeholder tokens stand for image embeddings."""
        self._raise_if_dead()
        req = Request(prompt_ids, gen or GenerationConfig(), handle)
        limit = self.cfg.max_context
        if mm is not None:
            if len(req.prompt_ids) >= limit:
                raise ValueError("the prompt with its image tokens does not fit max_context")
            req.mm = mm
            mm.ctx_id = req.handle
            mm.sent = False
        if len(req.prompt_ids) >= limit:
            req.prompt_ids = req.prompt_ids[-(limit - 1):]
        if not req.prompt_ids:
            req.prompt_ids = [0]
        with self.cv:
            self.requests[req.handle] = req
            self.waiting.append(req)
            self.cv.notify_all()
        return req.handle

    def abort(self, handle: int) -> None:
        with self.cv:
            r = self.requests.get(handle)
            if r is not None:
                r.abort_flag = True
                self.cv.notify_all()

    def can_fetch(self, handle: int) -> bool:
        r = self.requests.get(handle)
        return r is None or not r.results.empty()

    def fetch(self, handle: int, timeout: float | None = None):
        """Next generated token id, or -1 when the request has finished (reference: fetch_response_llm_model)."""
        r = self.requests.get(handle)
        if r is None:
            return -1
        if timeout is None and self._thread is not None:
            # never block for ever on a loop that has died: poll, and raise once the thread is gone
            while True:
                try:
                    tok = r.results.get(timeout=0.5)
                    break
                except queue.Empty:
                    self._raise_if_dead()
                    if not self._thread.is_alive() and not self._stop:
                        self.dead = True
                        self._raise_if_dead()
        else:
            tok = r.results.get(timeout=timeout)
        if tok < 0:
            with self.lock:
                self.requests.pop(handle, None)
        return tok

    def _raise_if_dead(self):
        if self.dead:
            raise RuntimeError(f"the engine loop stopped after repeated failures: {self.error!r}")

    def stats(self, handle: int) -> dict:
        r = self.requests.get(handle)
        return r.stats.as_dict() if r else {}

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # --------------------------------------------------------------------------------- background loop
    def start(self):
        if self._thread is None:
            self._stop = False
            self._thread = threading.Thread(target=self._loop, name="fastllm-b200-engine", daemon=True)
            self._thread.start()

    def stop(self):
        with self.cv:
            self._stop = True
            self.cv.notify_all()
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None

    def shutdown(self):
        """Stop the background loop and release the worker ranks of a multi-process group."""
        self.stop()
        if self.control is not None:
            self.control.stop()
            self.control = None
            self.runner.control = None

    def _loop(self):
        if self.model.device.type == "cuda" and self.model.device.index is not None:     # "cuda" alone: the current device
            torch.cuda.set_device(self.model.device)
        while True:
            with self.cv:
                while not self._stop and not self.has_work():
                    self.cv.wait(timeout=0.01)
                if self._stop:
                    return
            try:
                self.step()
                self._consecutive_failures = 0
            except Exception as e:
                # A failed step ends the requests that were part of it with reason "error" and the loop goes on
                # serving; only a failure that keeps repeating stops the thread, and then launch / fetch raise.
                self.error = e
                self._consecutive_failures = getattr(self, "_consecutive_failures", 0) + 1
                traceback.print_exc()
                with self.cv:
                    victims = list(self.running) or list(self.waiting)   # nothing running: admission itself failed
                    for r in victims:
                        if not r.finished():
                            self._finish(r, "error")
                    self.running.clear()
                    self.waiting = [r for r in self.waiting if not r.finished()]
                if self._consecutive_failures >= 8:
                    self.dead = True
                    return

    # ------------------------------------------------------------------------------------- scheduling
    def _used_fraction(self) -> float:
        return 1.0 - self.pm.num_available() / max(1, self.pm.num_pages)

    def _pages_needed(self, n_tokens: int) -> int:
        return (n_tokens + self.page_len - 1) // self.page_len

    def _admit(self):
        """Move waiting requests to running while pages and batch slots allow."""
        with self.lock:
            pending = [r for r in self.waiting if not r.abort_flag]
            aborted = [r for r in self.waiting if r.abort_flag]
            self.waiting = []
        for r in aborted:
            self._finish(r, "abort")
        pending.sort(key=lambda r: -len(r.prefill_ids))
        keep = []
        for r in pending:
            if len(self.running) >= self.cfg.max_batch or (self.runner.state_slots and not self.state_free):
                keep.append(r)
                continue
            toks = r.prefill_ids
            # image placeholder tokens look the same for every image: such prompts neither read nor feed the prefix cache
            cached = self.pm.query(toks) if (self.cfg.prefix_cache and r.mm is None) else []
            need = self._pages_needed(len(toks) + 1) - len(cached)
            avail = self.pm.num_available()
            limit_ok = (self.pm.num_pages - (avail - need)) <= self.cfg.prefill_page_limit * self.pm.num_pages or not self.running
            pages = self.pm.alloc(need) if (need <= avail and limit_ok) else None
            if pages is None:
                self.pm.release(cached)
                keep.append(r)
                continue
            r.pages = cached + pages
            if self.runner.state_slots:
                r.state_slot = self.state_free.pop()
            r.num_computed = len(cached) * self.page_len
            r.num_cached_prefix = r.num_computed
            r.stats.cached_tokens = r.num_computed
            if r.mm is not None and self.control is not None and not r.mm.sent:
                # (published from the scheduling thread, like every other plan) the worker ranks get the image tokens'
                # embeddings and rotary positions before the request's first chunk
                self.control.mm_put(r.mm)
                r.mm.sent = True
            r.state = RequestState.PREFILL
            self.running.append(r)
        if keep:
            with self.lock:
                self.waiting = keep + self.waiting

    def _finish(self, r: Request, reason: str):
        if r.finished():
            return
        r.state = RequestState.ABORTED if reason == "abort" else RequestState.FINISHED
        r.finish_reason = reason
        r.stats.finished = time.time()
        if r.pages:
            if self.cfg.prefix_cache and reason != "error" and r.mm is None:
                n_full = r.num_computed // self.page_len
                self.pm.record(r.all_ids[:n_full * self.page_len], r.pages[:n_full])
            self.pm.release(r.pages)
            r.pages = []
        self._release_state(r)
        if r.mm is not None and self.control is not None and getattr(r.mm, "sent", False):
            self.control.mm_drop(r.mm.ctx_id)
        r.results.put(-1)

    def _release_state(self, r: Request) -> None:
        if getattr(r, "state_slot", None) is not None and r.state_slot >= 0:
            self.state_free.append(r.state_slot)
            r.state_slot = -1

    def _evict_for_pages(self, need: int) -> bool:
        """Free pages by evicting the longest decoding request (it is re-queued for recomputation)."""
        cands = [r for r in self.running if r.state == RequestState.DECODE]
        if len(cands) <= 1:
            return False
        victim = max(cands, key=lambda r: r.total_len)
        self.running.remove(victim)
        self.pm.release(victim.pages)
        victim.pages = []
        self._release_state(victim)
        victim.num_computed = 0
        victim.recompute_tokens = victim.all_ids[:-1] if victim.output_ids else victim.prompt_ids
        victim.state = RequestState.WAITING
        with self.lock:
            self.waiting.insert(0, victim)
        return True

    # ------------------------------------------------------------------------------------------ step
    def step(self) -> int:
        """Run one scheduler iteration (a prefill step if any request needs one, else a decode step).
        Returns the number of tokens produced."""
        self._admit()
        for r in [r for r in self.running if r.abort_flag]:
            self.running.remove(r)
            self._finish(r, "abort")
        if not self.running:
            return 0
        self.step_count += 1
        try:
            pre = [r for r in self.running if r.state == RequestState.PREFILL]
            if pre:
                return self._prefill_step(pre)
            return self._decode_step([r for r in self.running if r.state == RequestState.DECODE])
        except _lib.DeviceKernelError as e:
            self._recover(e)
            return 0

    def _recover(self, err) -> None:
        """A kernel reported a failed bounded wait / bad argument through its status word (e.g. a tensor-parallel peer
        that never arrived).  The requests in flight cannot be trusted any more: they end with reason "error"; the
        collective arena starts a new epoch; requests still waiting are served normally afterwards.  The reference keeps
        a per-thread CUDA error flag for the same purpose (src/devices/cuda/fastllm-cuda.cu:91-108) and a generation
        counter for its communicators (src/devices/multicuda/fastllm-multicuda.cu:2150-2222)."""
        self.device_errors += 1
        self.last_device_error = str(err)
        for r in list(self.running):
            self.running.remove(r)
            self._finish(r, "error")
        if self.control is not None:
            self.control.reset()
        self.runner.reset_after_device_error()

    def _prefill_step(self, reqs) -> int:
        budget = self.cfg.chunked_prefill_size
        chunks, owners = [], []
        # Requests that are already decoding ride along as one-token chunks, so a long prompt's prefill never stalls them for
        # more than one chunk (the reference batches prefill and decode rows in one forward, src/models/basellm.cpp:1786-2545).
        decoding = []
        if self.cfg.mixed_prefill_decode:
            decoding = self._ensure_decode_pages([r for r in self.running if r.state == RequestState.DECODE])
            reqs = [r for r in reqs if r in self.running and r.state == RequestState.PREFILL]
            for r in decoding:
                chunks.append(([r.all_ids[-1]], r.total_len - 1, r.pages, True, r.state_slot, r.mm))
            budget = max(self.page_len, budget - len(decoding))
        for r in reqs:
            if budget <= 0:
                break
            toks = r.prefill_ids
            n = min(len(toks) - r.num_computed, budget)
            if n <= 0:
                continue
            done = r.num_computed + n == len(toks)
            chunks.append((toks[r.num_computed:r.num_computed + n], r.num_computed, r.pages, done, r.state_slot, r.mm))
            owners.append((r, n, done))
            budget -= n
        if not chunks:
            return 0
        mtp = self._mtp_on()
        logits = self.runner.prefill(chunks, keep_hidden=mtp)
        mtp_items, off = [], 0
        if mtp or self._draft_on():    # (request, first position, rows, first row in the packed batch) of every chunk
            for r in decoding:
                mtp_items.append((r, r.total_len - 1, 1, off))
                off += 1
            for r, n, _ in owners:
                mtp_items.append((r, r.num_computed, n, off))
                off += n
        produced = 0
        finals = [r for r, _, d in owners if d]
        for r, n, _ in owners:
            r.num_computed += n
        for r in decoding:
            r.num_computed = r.total_len
        if decoding or finals:
            toks = self._sample(decoding + finals, logits)
            for r, t in zip(decoding, toks):
                produced += self._emit(r, int(t))
            if decoding:
                self.decode_tokens += len(decoding)
            for r, t in zip(finals, toks[len(decoding):]):
                if r.recompute_tokens is not None and r.output_ids:
                    # recomputation after eviction: the next token was already produced before the eviction
                    r.recompute_tokens = None
                    r.state = RequestState.DECODE
                    continue
                r.recompute_tokens = None
                r.state = RequestState.DECODE
                if not r.stats.first_token:
                    r.stats.first_token = time.time()
                produced += self._emit(r, int(t))
        if mtp:
            self._mtp_advance(mtp_items)
        elif self._draft_on():
            self._draft_advance(mtp_items, True)
        return produced

    # -------------------------------------------------------------------------------- speculative decoding
    def _mtp_on(self) -> bool:
        return bool(self.cfg.speculative == "mtp" and getattr(self.model, "mtp", None) is not None)

    def _draft_on(self) -> bool:
        return bool(self.cfg.speculative == "draft" and self.draft is not None)

    def _draft_advance(self, items, from_prefill: bool) -> None:
        """Keep the draft model's KV in step with the target and propose the next tokens.  For every request of ``items`` the
        draft model reads the true tokens it has not seen yet (a prefill chunk the target has just computed; after a decode
        step the accepted tokens and the newest one) into its own pools under the request's page ids; a decoding request's
        last row gives the first draft, and ``speculative_tokens - 1`` further one-token passes chain on the draft's own
        output.  Rows written for drafts are overwritten with the true tokens' rows by the next call."""
        chunks, heads, seen = [], [], set()
        for r, start, _n, _off in items:
            if id(r) in seen:
                continue
            seen.add(id(r))
            r.mtp_drafts = []
            if r.finished():
                continue
            if from_prefill:
                # the chunk the target has just computed starts at ``start``: rows before it sit in pages that a request with
                # the same prefix filled for both models (prefix reuse), rows after it are stale (restart after an eviction)
                r.draft_computed = start
            ids = r.all_ids
            decoding = r.state == RequestState.DECODE
            upto = len(ids) if decoding else r.num_computed
            dc = min(r.draft_computed, upto - 1 if decoding else upto)
            if upto <= dc:
                continue
            need = self._pages_needed(upto) - len(r.pages)
            if need > 0 and not self._grow_pages(r, need):
                continue
            chunks.append((ids[dc:upto], dc, r.pages, bool(decoding), None, None))
            r.draft_computed = upto
            if decoding:
                heads.append(r)
        if not chunks:
            return
        logits = self.draft.prefill(chunks)
        if not heads:
            return
        live = []
        for r, t in zip(heads, sampling.greedy(logits).tolist()):
            r.mtp_drafts = [int(t)]
            live.append(r)
        for j in range(1, self.cfg.speculative_tokens):
            chunks, nxt = [], []
            for r in live:
                pos = len(r.all_ids) - 1 + j                   # position of the draft token that is fed now
                need = self._pages_needed(pos + 1) - len(r.pages)
                if pos + 2 >= self.cfg.max_context or (need > 0 and not self._grow_pages(r, need)):
                    continue
                chunks.append(([r.mtp_drafts[-1]], pos, r.pages, True, None, None))
                nxt.append(r)
            if not chunks:
                break
            logits = self.draft.prefill(chunks)
            for r, t in zip(nxt, sampling.greedy(logits).tolist()):
                r.mtp_drafts.append(int(t))
            live = nxt

    def _mtp_advance(self, items) -> None:
        """Run the draft head over the rows the decoder has just produced: for every position whose following token is known
        it appends that position to the head's own KV pages; the row of a decoding request's newest token pair yields the
        first draft, further drafts chain the head on its own output (their pages are written again once the true rows
        arrive).  ``items``: (request, first position, rows, first row in ``model.last_hidden``)."""
        chunks, sel, heads = [], [], []
        for r, start, n, off in items:
            r.mtp_drafts = []
            if r.finished():
                continue
            ids = r.all_ids
            avail = min(n, len(ids) - 1 - start)
            if avail <= 0:
                continue
            tail = r.state == RequestState.DECODE and start + avail == len(ids) - 1
            chunks.append((ids[start + 1:start + 1 + avail], start, r.pages, bool(tail), r.state_slot, r.mm))
            sel.extend(range(off, off + avail))
            if tail:
                heads.append((r, start + avail - 1, len(sel) - 1))
        if not chunks:
            return
        logits = self.runner.mtp_pass(chunks, sel, 0)
        if not heads:
            return
        live = []
        for (r, pos, row), t in zip(heads, self._greedy_rows(logits)):
            r.mtp_drafts = [int(t)]
            live.append((r, pos, row))
        for _ in range(1, self.cfg.speculative_tokens):
            chunks, rows, nxt = [], [], []
            for r, pos, row in live:
                pos += 1
                need = self._pages_needed(pos + 1) - len(r.pages)
                if pos + 2 >= self.cfg.max_context or (need > 0 and not self._grow_pages(r, need)):
                    continue
                chunks.append(([r.mtp_drafts[-1]], pos, r.pages, True, r.state_slot, r.mm))
                rows.append(row)
                nxt.append((r, pos))
            if not chunks:
                break
            logits = self.runner.mtp_pass(chunks, rows, 1)           # the head's own rows of the pass before
            live = []
            for i, ((r, pos), t) in enumerate(zip(nxt, self._greedy_rows(logits))):
                r.mtp_drafts.append(int(t))
                live.append((r, pos, i))

    def _greedy_rows(self, logits) -> list:
        """Arg-max token of every row; with a sharded vocabulary the ranks exchange their best candidate per row."""
        if self.model.tp.size > 1:
            if self.control is not None:
                self.control.gather_logits(1)
            vals, ids = self.model.tp.comm.gather_candidates(logits, self.model.vocab_shard, 1)
            return ids.gather(1, vals.argmax(dim=-1, keepdim=True)).view(-1).tolist()
        return sampling.greedy(logits).tolist()

    def _grow_pages(self, r, need: int) -> bool:
        pg = self.pm.alloc(need)
        if pg is None:
            return False
        r.pages.extend(pg)
        return True

    # (prompt-lookup drafts)
    @staticmethod
    def _ngram_draft(ids: list[int], n_max: int, k: int) -> list[int]:
        """Draft tokens by prompt lookup: find the latest earlier occurrence of the text's last n tokens (n = n_max .. 1) and
        propose what followed it."""
        L = len(ids)
        for n in range(min(n_max, L - 1), 0, -1):
            tail = ids[L - n:]
            for st in range(L - n - 1, -1, -1):
                if ids[st:st + n] == tail:
                    out = ids[st + n:st + n + k]
                    if out:
                        return out
        return []

    def _speculative_step(self, reqs) -> int | None:
        """One decode step that verifies draft tokens: every request feeds its last token plus up to ``speculative_tokens``
        drafts through one forward pass; the longest prefix of drafts that equals the model's own greedy choices is
        accepted, plus the model's next token after it -- so a step yields between 1 and k + 1 tokens per request and the
        output is exactly the greedy output.  The reference's speculative paths (Qwen3.5 MTP heads, the DeepSeek-V4 draft
        model: tools/fastllm_pytools/util.py:518-532, acceptance kernel src/devices/cuda/fastllm-cuda.cu:13266) verify the
        same way; here the drafts come from the request's own text.  Returns None when nothing could be drafted."""
        k = self.cfg.speculative_tokens
        mtp = self._mtp_on()
        dm = self._draft_on()
        drafts = []
        for r in reqs:
            room = min(k, self.cfg.max_context - r.total_len - 1, (r.gen.max_new_tokens - len(r.output_ids) - 1) if r.gen.max_new_tokens > 0 else k)
            if mtp or dm:
                drafts.append(list(r.mtp_drafts[:max(0, room)]))
            else:
                drafts.append(self._ngram_draft(r.all_ids, self.cfg.speculative_ngram, room) if room > 0 else [])
        if not any(drafts) and not mtp and not dm:   # (a draft head / model follows every step: it always takes this path)
            return None
        chunks, owners = [], []
        for r, d in zip(reqs, drafts):
            need = self._pages_needed(r.total_len + len(d)) - len(r.pages)
            if need > 0:
                pg = self.pm.alloc(need)
                if pg is None:
                    d = []                              # no room for drafts: plain single-token step for this request
                else:
                    r.pages.extend(pg)
            chunks.append(([r.all_ids[-1]] + d, r.total_len - 1, r.pages, len(d) + 1, r.state_slot, r.mm))
            owners.append((r, d))
        # models with recurrent (linear-attention) state: the verification pass advances the state over every draft; where a
        # draft is rejected the state is put back and rebuilt from the accepted tokens alone
        snap = self.runner.kv.snapshot_states([r.state_slot for r, _ in owners]) if self.runner.state_slots else None
        logits = self.runner.prefill(chunks, keep_hidden=mtp)
        mtp_items, redo = [], []
        if self.model.tp.size > 1:                  # greedy verification: one candidate per rank and row is enough
            if self.control is not None:
                self.control.gather_logits(1)
            vals, ids = self.model.tp.comm.gather_candidates(logits, self.model.vocab_shard, 1)
            choice = ids.gather(1, vals.argmax(dim=-1, keepdim=True)).view(-1).tolist()
        else:
            choice = sampling.greedy(logits).tolist()
        produced, row = 0, 0
        for r, d in owners:
            mine = choice[row:row + len(d) + 1]
            n_ok = 0
            while n_ok < len(d) and d[n_ok] == mine[n_ok]:
                n_ok += 1
            mtp_items.append((r, r.total_len - 1, n_ok + 1, row))
            if snap is not None and n_ok < len(d):
                redo.append(([r.all_ids[-1]] + d[:n_ok], r.total_len - 1, r.pages, False, r.state_slot, r.mm))
            row += len(d) + 1
            self.spec_proposed += len(d)
            self.spec_accepted += n_ok
            for t in mine[:n_ok + 1]:
                if r.finished():
                    break
                produced += self._emit(r, int(t))
            if not r.finished():
                r.num_computed = r.total_len - 1        # the last emitted token's K/V is written by the next step
        if redo:
            self.runner.kv.restore_states(snap, [c[4] for c in redo])
            self.runner.prefill(redo)
        if mtp:
            self._mtp_advance(mtp_items)
        elif dm:
            self._draft_advance(mtp_items, False)
        self.decode_steps += 1
        self.decode_tokens += produced
        return produced

    def _decode_step(self, reqs) -> int:
        if not reqs:
            return 0
        reqs = self._ensure_decode_pages(reqs)
        if not reqs:
            return 0
        if self.cfg.speculative == "mtp" and not self._mtp_on():
            self.cfg.speculative = "ngram"          # no draft head with this model: prompt-lookup drafts instead
        if self.cfg.speculative == "draft" and self.draft is None:
            self.cfg.speculative = "ngram"          # no draft model was given
        if self.cfg.speculative in ("ngram", "mtp", "draft") and all(r.gen.is_simple_greedy() for r in reqs):
            n = self._speculative_step(reqs)
            if n is not None:
                return n
        ids = [r.all_ids[-1] for r in reqs]
        positions = [r.total_len - 1 for r in reqs]
        all_greedy = all(r.gen.is_simple_greedy() for r in reqs)
        out_ids, logits = self.runner.decode(ids, positions, [r.pages for r in reqs], want_logits=not all_greedy,
                                             state_slots=[r.state_slot for r in reqs] if self.runner.state_slots else None,
                                             rope_offsets=[r.mm.delta if r.mm is not None else 0 for r in reqs]
                                             if any(r.mm is not None for r in reqs) else None)
        for r in reqs:
            r.num_computed = r.total_len
        if all_greedy:
            toks = out_ids.tolist()
        else:
            toks = self._sample(reqs, logits)
        produced = 0
        for r, t in zip(reqs, toks):
            produced += self._emit(r, int(t))
        self.decode_steps += 1
        self.decode_tokens += produced
        return produced

    def _ensure_decode_pages(self, reqs):
        """Make sure every decoding request has a page for the token it is about to write; evicts the longest decoding
        request when the pool is empty.  Returns the requests that can run this step."""
        for r in list(reqs):
            if r not in self.running or r.state != RequestState.DECODE:
                continue                     # evicted (or ended) earlier in this loop on behalf of another request
            pos = r.total_len - 1            # position of the token fed in this step
            need = self._pages_needed(pos + 1) - len(r.pages)
            while need > 0:
                pg = self.pm.alloc(need)
                if pg is not None:
                    r.pages.extend(pg)
                    break
                if not self._evict_for_pages(need):
                    if r in self.running:
                        self.running.remove(r)
                    self._finish(r, "length")
                    break
                if r not in self.running:    # the victim was the request that is asking
                    break
        return [r for r in reqs if r in self.running and r.state == RequestState.DECODE]

    def _candidate_width(self, reqs) -> int:
        """How many of each rank's best logits decide this step's tokens: the largest top-k in the batch (1 for greedy rows,
        the sampler's cap where top-k is off) plus the recent tokens a repetition penalty may push out of that set.
        0: the step needs whole logit rows (log-probabilities, returned logits, logits processors)."""
        need = 1
        for r in reqs:
            g = r.gen
            if g.output_logits or g.logprobs or g.logits_processor is not None:
                return 0
            greedy = g.is_simple_greedy() or not g.do_sample
            k = 1 if greedy else (g.top_k if g.top_k > 0 else 1024)
            if abs(g.repeat_penalty - 1.0) > 1e-8:
                k += len(set(r.all_ids[-g.last_n:]))
            need = max(need, k)
        return 1 << (need - 1).bit_length()              # few distinct shapes

    def _sample_candidates(self, reqs, vals, ids):
        """Sampling over the gathered per-rank candidates (``vals`` / ``ids`` ``[R, C]``): penalties by token id, then the same
        top-k / top-p / temperature draw as on whole rows; the drawn column is mapped back to its token id."""
        lg = vals.float().clone()
        for row, r in enumerate(reqs):
            g = r.gen
            if abs(g.repeat_penalty - 1.0) > 1e-8:
                recent = torch.as_tensor(sorted(set(r.all_ids[-g.last_n:])), dtype=torch.long, device=lg.device)
                if recent.numel():
                    hit = torch.isin(ids[row], recent)
                    v = lg[row]
                    lg[row] = torch.where(hit, torch.where(v > 0, v / g.repeat_penalty, v * g.repeat_penalty), v)
        greedy_rows = [r.gen.is_simple_greedy() or not r.gen.do_sample for r in reqs]
        if all(greedy_rows):
            cols = lg.argmax(dim=-1)
        else:
            tk = [1 if gr else r.gen.top_k for r, gr in zip(reqs, greedy_rows)]
            none = [[] for _ in reqs]
            if lg.is_cuda:
                cols = sampling.sample_fused(lg, none, [1.0] * len(reqs), tk, [r.gen.top_p for r in reqs],
                                             [r.gen.temperature for r in reqs]).long()
            else:
                cols = sampling.sample(lg, tk, [r.gen.top_p for r in reqs], [r.gen.temperature for r in reqs]).long()
        return ids.gather(1, cols.view(-1, 1)).view(-1).tolist()

    def _sample(self, reqs, logits):
        m = self.model
        if m.tp.size > 1:
            k = self._candidate_width(reqs) if self.cfg.tp_candidate_sampling else 0
            if 0 < k < m.lm_head.n // 2:
                # vocab-sharded head: the ranks exchange their k best (logit, id) pairs per row, not whole logit rows
                if self.control is not None:
                    self.control.gather_logits(k)
                vals, ids = m.tp.comm.gather_candidates(logits, m.vocab_shard, k)
                return self._sample_candidates(reqs, vals, ids)
            if self.control is not None:
                self.control.gather_logits()
            logits = m.tp.comm.gather_logits(logits, m.vocab_shard, m.cfg.vocab_size)
        if all(r.gen.is_simple_greedy() for r in reqs):
            return sampling.greedy(logits).tolist()
        lg = logits.float().clone()
        for row, r in enumerate(reqs):
            proc = r.gen.logits_processor
            allowed = proc(r.output_ids) if proc is not None else None
            if allowed is not None:
                keep = torch.as_tensor(list(allowed), dtype=torch.long, device=lg.device)
                masked = torch.full_like(lg[row], float("-inf"))
                masked[keep] = lg[row, keep]
                lg[row] = masked
        greedy_rows = [r.gen.is_simple_greedy() or not r.gen.do_sample for r in reqs]
        tk = [1 if g else r.gen.top_k for r, g in zip(reqs, greedy_rows)]
        recent = [r.all_ids[-r.gen.last_n:] for r in reqs]
        if lg.is_cuda:
            toks = sampling.sample_fused(lg, recent, [r.gen.repeat_penalty for r in reqs], tk, [r.gen.top_p for r in reqs],
                                         [r.gen.temperature for r in reqs])
        else:
            sampling.apply_repeat_penalty(lg, recent, [r.gen.repeat_penalty for r in reqs])
            toks = sampling.sample(lg, tk, [r.gen.top_p for r in reqs], [r.gen.temperature for r in reqs])
        out = toks.tolist()
        for r, row in zip(reqs, range(len(reqs))):
            if r.gen.output_logits:
                r.last_logits = logits[row].float().cpu()
            if r.gen.logprobs:
                # log-probabilities of the model distribution (before penalties and truncation), as the OpenAI API defines them
                lp = torch.log_softmax(logits[row].float(), dim=-1)
                tv, ti = lp.topk(min(int(r.gen.logprobs), lp.numel()))
                r.logprob_entries.append((float(lp[out[row]]), list(zip(ti.tolist(), tv.tolist()))))
        return out

    def _emit(self, r: Request, tok: int) -> int:
        r.output_ids.append(tok)
        r.stats.output_tokens = len(r.output_ids)
        g = r.gen
        stop = False
        reason = None
        is_eos = (tok in self.eos and not g.ignore_eos) or tok in g.stop_token_ids
        if is_eos and len(r.output_ids) > g.min_new_tokens:
            stop, reason = True, "stop"
        elif g.max_new_tokens > 0 and len(r.output_ids) >= g.max_new_tokens:
            stop, reason = True, "length"
        elif r.total_len >= self.cfg.max_context:
            stop, reason = True, "length"
        if not (is_eos and stop):
            r.results.put(tok)
        if stop:
            if r in self.running:
                self.running.remove(r)
            self._finish(r, reason)
        return 1

    # -------------------------------------------------------------------------------- convenience
    def generate(self, prompts, gen: GenerationConfig | None = None):
        """Blocking helper: run the given prompts (lists of token ids) to completion, return output ids."""
        handles = [self.launch(p, gen) for p in prompts]
        reqs = [self.requests[h] for h in handles]
        while any(not r.finished() for r in reqs):
            self.step()
        return [r.output_ids for r in reqs]
