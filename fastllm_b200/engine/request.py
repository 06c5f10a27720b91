"""Request-level data: generation parameters, request state, per-request statistics.

``GenerationConfig`` carries the fields of the reference's struct of the same name
(include/fastllm.h:152-195) under the names its Python API uses (tools/fastllm_pytools/llm.py:789).
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from enum import Enum


@dataclass
class GenerationConfig:
    max_new_tokens: int = 256            # reference: output_token_limit (<= 0: until the context limit)
    min_new_tokens: int = 0
    do_sample: bool = False
    top_k: int = 1
    top_p: float = 1.0
    temperature: float = 1.0
    repeat_penalty: float = 1.0
    last_n: int = 64                     # window of recent tokens the repeat penalty looks at
    stop_token_ids: list = field(default_factory=list)
    ignore_eos: bool = False
    output_logits: bool = False
    seed: int | None = None
    logprobs: int = 0
    # ``logits_processor(output_ids) -> allowed token ids or None``: tokens outside the returned set are masked before sampling
    # (tool-call name constraints).  A request that carries one is sampled on the host-visible path, never in the decode graph.
    logits_processor: object | None = None

    def is_simple_greedy(self) -> bool:
        """Arg-max decoding with no penalty: eligible for the in-graph greedy sampler
        (reference: GenerationConfig::IsSimpleGreedy)."""
        if self.output_logits or self.logprobs or self.logits_processor is not None:
            return False
        if abs(self.repeat_penalty - 1.0) > 1e-8:
            return False
        if not self.do_sample or self.top_k <= 1:
            return True
        return self.temperature <= 1e-6


class RequestState(Enum):
    WAITING = 0
    PREFILL = 1
    DECODE = 2
    FINISHED = 3
    ABORTED = 4


@dataclass
class RequestStats:
    arrival: float = 0.0
    first_token: float = 0.0
    finished: float = 0.0
    prompt_tokens: int = 0
    cached_tokens: int = 0
    output_tokens: int = 0

    def as_dict(self):
        ttft = (self.first_token - self.arrival) if self.first_token else 0.0
        dur = (self.finished or time.time()) - (self.first_token or self.arrival)
        tpot = dur / max(1, self.output_tokens - 1) if self.output_tokens > 1 else 0.0
        return dict(prompt_tokens=self.prompt_tokens, cached_tokens=self.cached_tokens, output_tokens=self.output_tokens,
                    ttft_s=ttft, tpot_s=tpot)


class Request:
    _next = 0
    _lock = threading.Lock()

    def __init__(self, prompt_ids, gen: GenerationConfig, handle: int | None = None):
        if handle is None:
            with Request._lock:
                handle = Request._next
                Request._next += 1
        self.handle = handle
        self.prompt_ids = list(prompt_ids)
        self.gen = gen
        self.output_ids: list[int] = []
        self.state = RequestState.WAITING
        self.pages: list[int] = []
        self.num_computed = 0          # tokens whose K/V are in the cache
        self.num_cached_prefix = 0     # of those, how many came from the prefix cache
        self.results: "queue.Queue" = queue.Queue()
        self.abort_flag = False
        self.finish_reason: str | None = None
        self.stats = RequestStats(arrival=time.time(), prompt_tokens=len(self.prompt_ids))
        self.last_logits = None
        self.logprob_entries: list = []   # per output token: (token logprob, [(token id, logprob), ...]) when gen.logprobs > 0
        self.recompute_tokens: list[int] | None = None   # set when evicted: prompt + outputs to prefill again
        self.state_slot = -1           # linear-attention state slot while the request is running (-1: none)
        self.mtp_drafts: list[int] = []   # draft tokens for the next step, from the model's multi-token-prediction head or a draft model
        self.draft_computed = 0           # positions whose true tokens a separate draft model has read into its own KV pools
        self.mm = None                 # multimodal context (engine.MultimodalContext): image embeddings and 3-D rotary positions

    @property
    def all_ids(self):
        return self.prompt_ids + self.output_ids

    @property
    def prefill_ids(self):
        """Tokens that must be in the cache before decoding can (re)start."""
        return self.recompute_tokens if self.recompute_tokens is not None else self.prompt_ids

    @property
    def total_len(self):
        return len(self.prompt_ids) + len(self.output_ids)

    def finished(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.ABORTED)
