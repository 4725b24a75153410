"""The engine: model runner + scheduler + sampler behind one object.

Reference: ``Engine`` (src/runtime/engine.h:32-64, engine.cpp:84-205) owns tokenizer, model and
a one-sequence generate loop.  This one serves many requests at a time from token ids.
"""

from __future__ import annotations

import itertools
from typing import Any, Dict, Hashable, Iterable, List, Optional, Sequence, Union

import torch

from ..config.engine_options import EngineOptions
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, check_params
from .loading import load_runner
from .scheduler import Request, Scheduler


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[Dict[str, Any]] = None,
                 random_seed: Optional[int] = None, options: Optional[EngineOptions] = None):
        self.options = options or EngineOptions()
        self.runner = load_runner(model_dir, config=config, random_seed=random_seed, options=self.options)
        self.cache = self.runner.cache
        self.vocab_size = self.runner.model.vocab_size
        self.scheduler = Scheduler(self.cache, max_batched_tokens=self.options.max_batched_tokens,
                                   prefill_chunk=self.options.prefill_chunk,
                                   max_context=self.options.max_context)
        self.sampler = Sampler(self.vocab_size, self.runner.device)
        self._ids = itertools.count()
        self._fresh_seed = itertools.count(0x5EED)
        self.requests: Dict[Hashable, Request] = {}
        self.d2h_bytes = 0
        self._ahead = None      # (batch, drawn tokens on the device) of a step launched ahead of its turn
        self.ahead_steps = 0    # steps launched that way
        self._copy_stream = None
        self._landing = [None, None]     # pinned buffers the drawn tokens land in, used in turn
        self._landing_turn = 0
        self._steps_since_check = 0

    # ---- requests ---------------------------------------------------------------------
    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
               stop_ids: Iterable[int] = (), request_id: Optional[Hashable] = None) -> Hashable:
        params = params or SamplingParams()
        check_params(params, self.vocab_size)
        for t in prompt:
            if not 0 <= int(t) < self.vocab_size:
                raise ValueError(f"token id {t} outside [0, {self.vocab_size})")
        if params.seed == 0 and not params.greedy:
            # the reference draws a random seed when none is given (engine.cpp:131); here it is
            # a counter, so that a run is repeatable
            params = SamplingParams(**{**params.__dict__, "seed": next(self._fresh_seed)})
        rid = request_id if request_id is not None else f"req-{next(self._ids)}"
        if rid in self.requests and self.requests[rid].status != "finished":
            raise ValueError(f"request id {rid!r} is in use")
        req = Request(rid, [int(t) for t in prompt], params, set(int(s) for s in stop_ids))
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    # ---- stepping ---------------------------------------------------------------------
    def step(self) -> List[Request]:
        """One scheduler step: build the batch, run it, sample, record.  Returns the requests
        that finished in this step.

        With `run_ahead`, a pure decode step launches its successor before the host reads the
        tokens it drew (they are handed on inside the device), so the device does not idle
        while the host schedules; that successor is picked up by the next call."""
        done: List[Request] = []
        if self._ahead is not None and not any(s.request.status == "running" for s in self._ahead[0]):
            self._ahead = None          # every request of that step has stopped meanwhile: nothing to record
        if self._ahead is not None:
            batch, picked = self._ahead
            self._ahead = None
        else:
            before = len(self.scheduler.finished)
            batch = self.scheduler.schedule()
            done = list(self.scheduler.finished[before:])      # finished without running (out of cache)
            if not batch:
                return done
            logits = self.runner.step(self.scheduler.entries(batch))
            picked = self._sample(batch, logits, ahead=False)
        tokens: List[int] = []
        if picked is not None:
            landing = self._start_readback(picked)
            if self.options.run_ahead:
                self._ahead = self._launch_ahead(batch, picked)
            tokens = self._finish_readback(landing)
            self.d2h_bytes += picked.numel() * 4
        self._check_kernels(batch)
        return done + self.scheduler.update(batch, tokens)

    def _check_kernels(self, batch) -> None:
        """Read the kernels' status flags (a bounded wait that ran out, an index outside its
        operands) and raise instead of handing on what such a step produced.  The read
        synchronises the device, so steps with prompt portions (the tensor-core kernels run there
        and the host has just waited for the step anyway) are checked at once, pure decode steps
        every `status_every` steps."""
        if self.runner.device.type != "cuda":
            return
        self._steps_since_check += 1
        prompt_rows = any(len(s.tokens) > 1 for s in batch)
        if prompt_rows or self._steps_since_check >= max(1, self.options.status_every):
            self._steps_since_check = 0
            from .. import kernels
            kernels.check_status("engine step")

    # The drawn tokens come to the host on a stream of their own, into pinned memory: a copy
    # on the compute stream would queue behind the step that has just been launched ahead, and
    # the host would wait for that step too.
    def _start_readback(self, picked: torch.Tensor):
        if not picked.is_cuda:
            return picked, None
        n = picked.numel()
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=picked.device)
        slot = self._landing[self._landing_turn % 2]
        if slot is None or slot.numel() < n:
            slot = torch.empty((max(n, 64),), dtype=torch.int32).pin_memory()
            self._landing[self._landing_turn % 2] = slot
        self._landing_turn += 1
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(picked.device))
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(ready)
            slot[:n].copy_(picked, non_blocking=True)
            landed = torch.cuda.Event()
            landed.record(self._copy_stream)
        picked.record_stream(self._copy_stream)
        return slot[:n], landed

    @staticmethod
    def _finish_readback(landing) -> List[int]:
        host, landed = landing
        if landed is not None:
            landed.synchronize()
        return host.tolist()

    def _sample(self, batch, logits: torch.Tensor, ahead: bool) -> Optional[torch.Tensor]:
        sampling = [s for s in batch if s.sample]
        if not sampling:
            return None
        # a step that runs ahead draws the token after the one still on its way to the host
        extra = 1 if ahead else 0
        return self.sampler.sample(
            logits, [s.request.params for s in sampling],
            recent=[s.request.tokens for s in sampling],
            counters=[len(s.request.generated) + extra for s in sampling])

    def _launch_ahead(self, batch, picked: torch.Tensor):
        """Launch the step after `batch` on the tokens in `picked` (still on the device), if the
        scheduler can say what that step is without knowing them.  Returns (batch, its drawn
        tokens on the device) or None."""
        if not self.runner.can_take_device_tokens(len(batch)):
            return None
        nxt = self.scheduler.schedule_ahead(batch)
        if nxt is None:
            return None
        tokens = picked
        if len(nxt) != len(batch):
            keep = [i for i, s in enumerate(batch) if any(n.request is s.request for n in nxt)]
            tokens = picked.index_select(0, torch.tensor(keep, dtype=torch.long, device=picked.device))
        try:
            logits = self.runner.step(self.scheduler.entries(nxt), device_tokens=tokens)
        except Exception:
            for s in nxt:
                self.cache.truncate(s.request.id)
            raise
        self.ahead_steps += 1
        return nxt, self._sample(nxt, logits, ahead=True)

    def run_until_idle(self, max_steps: Optional[int] = None) -> int:
        steps = 0
        while not self.scheduler.idle and (max_steps is None or steps < max_steps):
            self.step()
            steps += 1
        return steps

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 stop_ids: Iterable[int] = ()) -> List[List[int]]:
        """Generate for every prompt (token ids in, token ids out), batched by the scheduler."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.submit(p, sp, stop_ids) for p, sp in zip(prompts, params)]
        self.run_until_idle()
        return [list(self.requests[i].generated) for i in ids]

    def stream(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
               stop_ids: Iterable[int] = ()):
        """Generate for one prompt and yield each token id as soon as its step has been read
        back (the reference's CLI prints text as it comes, src/apps/ninfer.cpp:121-138).  Other
        requests that are live meanwhile keep running in the same steps."""
        rid = self.submit(prompt, params, stop_ids)
        req = self.requests[rid]
        sent = 0
        while True:
            while sent < len(req.generated):
                yield req.generated[sent]
                sent += 1
            if req.status == "finished" or self.scheduler.idle:
                return
            self.step()

    def io_bytes(self):
        """(host-to-device, device-to-host) bytes moved by the steps so far: the packed step
        inputs in, the sampled token ids out."""
        return self.runner.h2d_bytes, self.d2h_bytes

    def stats(self) -> Dict[str, Any]:
        st = self.scheduler.stats
        return {"steps": st.steps, "prompt_tokens": st.prompt_tokens, "decode_tokens": st.decode_tokens,
                "preemptions": st.preemptions, "finished": st.finished, "out_of_cache": st.out_of_cache,
                "pages_free": self.cache.pages_free(), "live_requests": len(self.cache.requests),
                "ahead_steps": self.ahead_steps}
