"""The step function: run a batch of (request, its next tokens) from the cache.

Reference: ``Model::forward_batch(tokens, positions, seq_ids)`` (src/models/model.h:74-77,
src/models/model.hip:994-1032) returns the logits of each group's last row and leaves
length bookkeeping to its callers (src/api/ninfer_c_api.cpp:190, 210, 239).  This step
takes whole entries, keeps the lengths in the cache manager, accepts portions of prompts
beside single decoded tokens cut anywhere, and returns logits at exactly the rows asked
for.  It runs only the tokens it is given; everything earlier comes from the cache.
"""

from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..cache.page_pool import OutOfPages
from ..parts.model import DecoderModel
from .batch import BatchError, StepEntry, pack_step, validate_entries


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, dtype: torch.dtype, device,
                 use_graph: bool = False):
        self.model, self.cache, self.dtype = model, cache, dtype
        self.device = torch.device(device)
        self.graphs = None
        if use_graph and self.device.type == "cuda" and model.graph_safe:
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(self, cache.max_requests)
        self.steps_run = 0
        self.h2d_bytes = 0
        self.tokens_run = 0

    # ---- requests -------------------------------------------------------------------
    def open(self, req: Hashable) -> int:
        return self.cache.open(req)

    def close(self, req: Hashable) -> None:
        self.cache.close(req)

    # ---- the step -------------------------------------------------------------------
    def reserve(self, entries: Sequence[StepEntry]) -> None:
        """Hold pages for every entry's new tokens, or for none of them."""
        done: List[StepEntry] = []
        try:
            for e in entries:
                self.cache.reserve(e.req, self.cache.length(e.req) + len(e.tokens))
                done.append(e)
        except OutOfPages:
            for e in done:
                self.cache.truncate(e.req)
            raise

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """float32 logits [R, vocab] on the device, R = total wanted rows, in entry order.

        `device_tokens`: for a decode-only step replayed from a graph, the entries' token ids
        as an int32 tensor on the device, to be used instead of the (placeholder) ids in the
        entries; `can_take_device_tokens` says whether a step qualifies."""
        entries = list(entries)
        if not entries:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        validate_entries(entries, self.cache, self.model.vocab_size)
        self.reserve(entries)
        try:
            if self.graphs is not None and self.graphs.eligible(entries):
                logits, moved = self._step_from_graph(entries, device_tokens)
            elif device_tokens is not None:
                raise ValueError("token ids on the device can only feed a step that is replayed from a graph")
            else:
                ctx = pack_step(entries, self.cache, self.dtype, self.device)
                logits, moved = self.run(ctx), ctx.scratch.get("h2d_bytes", 0)
        except Exception:
            for e in entries:
                self.cache.truncate(e.req)
            raise
        for e in entries:
            self.cache.commit(e.req, self.cache.length(e.req) + len(e.tokens))
        self.steps_run += 1
        self.h2d_bytes += moved
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits

    def can_take_device_tokens(self, n_entries: int) -> bool:
        """Whether a step of `n_entries` single tokens would be replayed from a graph."""
        return self.graphs is not None and 0 < n_entries <= self.graphs.max_rows

    def _step_from_graph(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None):
        """A decode-only step: replay the captured graph for this many rows."""
        g = self.graphs.get(entries)
        logits = g.run(entries, device_tokens)
        n = len(entries)
        if all(len(e.want) == 1 for e in entries):
            return logits[:n], g.h2d_bytes
        rows = [i for i, e in enumerate(entries) for _ in e.want]
        if not rows:
            return logits[:0], g.h2d_bytes
        return logits.index_select(0, torch.tensor(rows, device=self.device)), g.h2d_bytes

    def run(self, ctx) -> torch.Tensor:
        cache = self.cache
        return self.model.forward(
            ctx,
            lambda slot, append: cache.view(slot, ctx.block_tables, append),
            cache.state_of)
