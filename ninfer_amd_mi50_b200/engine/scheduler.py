"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

The reference has none: ``Engine::run`` serves one sequence (prefill in chunks of
``prefill_chunk``, then one token at a time, src/runtime/engine.cpp:140-198) and the C API
leaves batching to its caller (``ninfer_decode_batch``, src/api/ninfer_c_api.cpp:219-246;
tools/demo_ninfer_capi.py:42-73).  This scheduler builds, every step, one batch that holds a
decode token for each running request that has finished its prompt, and fills the rest of
the budget with prompt portions.

What happens when pages run out is decided here: the most recently admitted running
request is preempted - its pages and slot are given back, it returns to the front of the
waiting queue and is later recomputed from its prompt plus what it has generated; a
request that cannot fit even alone finishes with reason "out_of_cache".  Decisions depend
only on the order of arrival and the options, never on time.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Set

from ..cache.manager import CacheManager, OutOfSlots
from ..sampling.params import SamplingParams
from .batch import StepEntry


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Set[int] = field(default_factory=set)
    generated: List[int] = field(default_factory=list)
    status: str = "waiting"              # waiting | running | finished
    finish_reason: Optional[str] = None  # length | stop | context | out_of_cache
    preemptions: int = 0
    computed: int = 0                    # tokens of (prompt + generated) that are in the cache

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def remaining(self) -> int:
        """Known tokens not yet run; the step that runs the last of them samples the next."""
        return len(self.prompt) + len(self.generated) - self.computed


@dataclass
class Scheduled:
    request: Request
    tokens: List[int]
    sample: bool          # this portion reaches the end of what is known: sample after it


@dataclass
class SchedulerStats:
    steps: int = 0
    prompt_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    out_of_cache: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_batched_tokens: int, prefill_chunk: int,
                 max_context: int):
        self.cache = cache
        self.max_batched_tokens = int(max_batched_tokens)
        self.prefill_chunk = int(prefill_chunk)
        self.max_context = int(max_context)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []       # in admission order, oldest first
        self.finished: List[Request] = []
        self.stats = SchedulerStats()

    # ---- intake -------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError(f"request {req.id!r}: empty prompt")
        if len(req.prompt) + 1 > self.max_context:
            raise ValueError(f"request {req.id!r}: a prompt of {len(req.prompt)} tokens leaves no "
                             f"room to generate within max_context={self.max_context}")
        req.status, req.computed = "waiting", 0
        self.waiting.append(req)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- one step's batch ------------------------------------------------------------
    def schedule(self) -> List[Scheduled]:
        """Decide this step's batch and hold its pages.  May preempt or finish requests."""
        while True:
            batch = self._schedule_once()
            if batch or self.idle:
                if batch:
                    self.stats.steps += 1
                return batch
            # nothing fits although work is left: `_schedule_once` has preempted or finished
            # something, so the next round sees a different state

    def _schedule_once(self) -> List[Scheduled]:
        budget = self.max_batched_tokens
        batch: List[Scheduled] = []
        self._preempted_now = False
        # 1. single tokens (decoding requests) first, oldest first
        for req in list(self.running):
            if budget > 0 and req.status == "running" and req.remaining == 1:
                budget -= self._place(req, 1, batch)
        # 2. portions of running requests that still have a prompt (or a recomputation) to run
        for req in list(self.running):
            if budget > 0 and req.status == "running" and req.remaining > 1:
                budget -= self._place(req, min(req.remaining, self.prefill_chunk, budget), batch)
        # 3. admit from the head of the queue, in order, while there is budget, a slot and room;
        #    not in a round that had to preempt: the pool is short, admitting would thrash
        while self.waiting and budget > 0 and not self._preempted_now:
            req = self.waiting[0]
            n = min(req.remaining, self.prefill_chunk, budget)
            try:
                self.cache.open(req.id)
            except OutOfSlots:
                break
            if not self._room_to_admit(req, n):
                self.cache.close(req.id)
                if not self.running and not batch:
                    # the pool is empty and its first portion still does not fit: it never will
                    self.waiting.popleft()
                    self._finish(req, "out_of_cache")
                    continue
                break
            self.waiting.popleft()
            req.status = "running"
            self.running.append(req)
            self.cache.reserve(req.id, n)
            batch.append(Scheduled(req, req.tokens[:n], n == req.remaining))
            budget -= n
        return batch

    def schedule_ahead(self, batch: Sequence[Scheduled]) -> Optional[List[Scheduled]]:
        """The batch that follows `batch` if none of its requests stops on the token it is about
        to receive - decided before that token is known, so that the next step can be launched
        while the host still waits for this one.  Only when nothing else could be in that
        batch: every running request decodes in `batch`, nobody waits, no request's sampling
        looks at earlier tokens (repetition penalty).  Requests that will finish by length or
        context with the coming token are left out; a request that stops on a stop token after
        all has run one token for nothing, which `update` is told to ignore.  Holds the pages
        of the returned batch; returns None (holding nothing) if running ahead is not possible.
        The entries' token ids are placeholders: the real ones are still on the device."""
        if self.waiting or not batch or len(batch) != len(self.running):
            return None
        nxt: List[Scheduled] = []
        for s in batch:
            req = s.request
            if not s.sample or len(s.tokens) != 1 or req.status != "running" or req.remaining != 1:
                return None
            if req.params.repetition_penalty != 1.0:
                return None
            after = len(req.generated) + 1                       # generated tokens once this step's is in
            if after >= req.params.max_new_tokens or len(req.prompt) + after >= self.max_context:
                continue                                         # finishes with the coming token
            nxt.append(Scheduled(req, [0], True))
        if not nxt:
            return None
        # this step's token sits at position `computed`, the next one at `computed + 1`
        if not all(self.cache.can_reserve(s.request.id, s.request.computed + 2) for s in nxt):
            return None
        done: List[Scheduled] = []
        try:
            for s in nxt:
                self.cache.reserve(s.request.id, s.request.computed + 2)
                done.append(s)
        except Exception:
            for s in done:
                self.cache.truncate(s.request.id)
            return None
        self.stats.steps += 1
        return nxt

    def _place(self, req: Request, n: int, batch: List[Scheduled]) -> int:
        """Hold pages for `n` more tokens of a running request and put it into the batch.
        If the pool is short, the most recently admitted request gives way - which may be
        `req` itself.  Returns the tokens placed (0 if `req` gave way)."""
        target = req.computed + n
        while not self.cache.can_reserve(req.id, target):
            victim = self.running[-1]
            if victim is req:
                if len(self.running) == 1:
                    self._finish(req, "out_of_cache")   # alone with the whole pool and still short
                else:
                    self._preempt(req, batch)
                return 0
            self._preempt(victim, batch)
        self.cache.reserve(req.id, target)
        known = req.tokens
        batch.append(Scheduled(req, known[req.computed:target], target == len(known)))
        return n

    def _preempt(self, req: Request, batch: List[Scheduled]) -> None:
        """Give back everything `req` holds; it restarts later from prompt + generated."""
        batch[:] = [s for s in batch if s.request is not req]
        self.cache.close(req.id)
        self.running.remove(req)
        req.status, req.computed = "waiting", 0
        req.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(req)
        self._preempted_now = True

    def _room_to_admit(self, req: Request, n: int) -> bool:
        """Pages for the first portion, and one page of headroom in every group for each
        request already running, so that an admission is not undone a step later."""
        if n > self.max_context:
            return False
        need = self.cache.pages_needed(req.id, n)
        free = self.cache.pages_free()
        return all(nd + len(self.running) <= fr or (not self.running and nd <= fr)
                   for nd, fr in zip(need, free))

    def _finish(self, req: Request, reason: str) -> None:
        if self.cache.is_open(req.id):
            self.cache.close(req.id)
        if req in self.running:
            self.running.remove(req)
        req.status, req.finish_reason = "finished", reason
        self.finished.append(req)
        self.stats.finished += 1
        if reason == "out_of_cache":
            self.stats.out_of_cache += 1

    @staticmethod
    def entries(batch: Sequence[Scheduled]) -> List[StepEntry]:
        """The batch as step entries: logits are wanted at the last row of portions that sample."""
        return [StepEntry(s.request.id, s.tokens, [len(s.tokens) - 1] if s.sample else [])
                for s in batch]

    # ---- after the step ----------------------------------------------------------------
    def update(self, batch: Sequence[Scheduled], sampled: Sequence[int]) -> List[Request]:
        """Record the step's results.  `sampled` holds one token for every entry with
        `sample` set, in batch order.  Returns the requests that finished."""
        done: List[Request] = []
        it = iter(sampled)
        for s in batch:
            req = s.request
            if req.status != "running":
                # a step that ran ahead of the news that this request had stopped: its row was
                # computed for nothing and its token is dropped
                if s.sample:
                    next(it)
                continue
            if len(s.tokens) == 1 and req.generated and req.computed >= len(req.prompt):
                self.stats.decode_tokens += 1
            else:
                self.stats.prompt_tokens += len(s.tokens)
            req.computed += len(s.tokens)
            if not s.sample:
                continue
            tok = int(next(it))
            req.generated.append(tok)
            reason = None
            if tok in req.stop_ids:
                reason = "stop"
            elif len(req.generated) >= req.params.max_new_tokens:
                reason = "length"
            elif len(req.prompt) + len(req.generated) >= self.max_context:
                reason = "context"
            if reason:
                self._finish(req, reason)
                done.append(req)
        return done
