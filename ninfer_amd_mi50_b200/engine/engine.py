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
        that finished in this step."""
        before = len(self.scheduler.finished)
        batch = self.scheduler.schedule()
        done = self.scheduler.finished[before:]      # finished without running (out of cache)
        if not batch:
            return list(done)
        logits = self.runner.step(self.scheduler.entries(batch))
        sampling = [s for s in batch if s.sample]
        tokens: List[int] = []
        if sampling:
            picked = self.sampler.sample(
                logits, [s.request.params for s in sampling],
                recent=[s.request.tokens for s in sampling],
                counters=[len(s.request.generated) for s in sampling])
            tokens = picked.cpu().tolist()
            self.d2h_bytes += picked.numel() * 4
        return list(done) + self.scheduler.update(batch, tokens)

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

    def io_bytes(self):
        """(host-to-device, device-to-host) bytes moved by the steps so far: the packed step
        inputs in, the sampled token ids out."""
        return self.runner.h2d_bytes, self.d2h_bytes

    def stats(self) -> Dict[str, Any]:
        st = self.scheduler.stats
        return {"steps": st.steps, "prompt_tokens": st.prompt_tokens, "decode_tokens": st.decode_tokens,
                "preemptions": st.preemptions, "finished": st.finished, "out_of_cache": st.out_of_cache,
                "pages_free": self.cache.pages_free(), "live_requests": len(self.cache.requests)}
