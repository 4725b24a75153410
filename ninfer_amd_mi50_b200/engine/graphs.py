"""Decode steps replayed from CUDA graphs.

A decode-only step launches a few hundred small kernels; issuing them from the host
costs more than running them.  The reference has an opt-in HIP-graph path for its
one-token forward, dense models only, because its MoE routing synchronises with the host
(src/models/model.hip:786-830; src/runtime/engine.cpp:151-154).  Here routing stays on the
device, so the whole step is captured: one graph per (number of rows, context bound).
A step copies its index data into the graph's fixed input buffer and replays it.

Rows beyond the live requests are padding: token 0 at position 0 of a request whose only
page is the cache's null page.  They cost a little work and touch nothing that is read.
"""

from __future__ import annotations

import gc
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import lib as klib
from ..parts.base import StepContext
from .batch import StepEntry


def row_bucket(n: int) -> int:
    """Rows a graph is built for: exact up to 8, then the next power of two."""
    if n <= 8:
        return n
    b = 16
    while b < n:
        b <<= 1
    return b


def context_bucket(n: int, limit: int) -> int:
    """Context bound a graph is built for: the next multiple of 512 (the decode attention
    launches one block of CTAs per 128 keys of this bound, so a tight bound saves idle CTAs)."""
    return min((n + 511) // 512 * 512, max(limit, 1))


class DecodeGraph:
    def __init__(self, runner, rows: int, context_bound: int):
        self.runner, self.S, self.context_bound = runner, rows, context_bound
        cache, dev = runner.cache, runner.device
        S = rows
        self.width = cache.max_pages_per_request
        sizes = [S, S, S, S + 1, S, S, S] + [S * self.width for _ in cache.groups]
        self.offsets = np.cumsum([0] + sizes)
        total = int(self.offsets[-1])
        # Two pinned staging buffers used in turn, each with the event of its last copy: the host
        # runs a step ahead of the device on purpose, so the copy out of a buffer may still be
        # queued when the next step is being prepared; a buffer is rewritten only after its own
        # last copy has finished.
        self.hosts = [torch.empty((total,), dtype=torch.int32).pin_memory() for _ in range(2)]
        self.nps = [h.numpy() for h in self.hosts]
        self.copied: List[Optional[torch.cuda.Event]] = [None, None]
        self.turn = 0
        self.dev = torch.zeros((total,), dtype=torch.int32, device=dev)
        parts = [self.dev[self.offsets[i]:self.offsets[i + 1]] for i in range(len(sizes))]
        self.ctx = StepContext(
            dtype=runner.dtype, device=dev, T=S, S=S, token_ids=parts[0], positions=parts[1],
            row_seg=parts[2], seg_row0=parts[3], seg_pos0=parts[4], seg_slot=parts[5],
            logit_rows=parts[6], seg_len_host=[1] * S, seg_pos0_host=None, max_rows_per_seg=1,
            max_context=context_bound, graph_mode=True)
        for gi, g in enumerate(cache.groups):
            self.ctx.block_tables[g.index] = parts[7 + gi].view(S, self.width)
        # the parts of the buffer that never change
        o = self.offsets
        for a in self.nps:
            a[o[2]:o[3]] = np.arange(S)
            a[o[3]:o[4]] = np.arange(S + 1)
            a[o[6]:o[7]] = np.arange(S)
            self._fill(a, [], [])
        self.dev.copy_(self.hosts[0])
        # warm up on a side stream (library handles, lazily set kernel attributes), then capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                runner.run(self.ctx)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        before = klib.launch_count()
        self.graph = torch.cuda.CUDAGraph()
        # No cyclic garbage collection while the stream captures: collecting an older engine's
        # graphs then would destroy them inside this capture, which the runtime forbids and
        # answers by invalidating the capture.
        collecting = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = runner.run(self.ctx)
        finally:
            if collecting:
                gc.enable()
        self.kernels = klib.launch_count() - before
        self.h2d_bytes = total * 4

    def _fill(self, a: np.ndarray, entries: Sequence[StepEntry], lengths: Sequence[int]) -> None:
        cache, o, S = self.runner.cache, self.offsets, self.S
        n = len(entries)
        a[o[0]:o[0] + n] = [int(e.tokens[0]) for e in entries]
        a[o[0] + n:o[1]] = 0
        a[o[1]:o[1] + n] = lengths
        a[o[1] + n:o[2]] = 0
        a[o[4]:o[4] + n] = lengths
        a[o[4] + n:o[5]] = 0
        a[o[5]:o[5] + n] = [cache.slot(e.req) for e in entries]
        a[o[5] + n:o[6]] = cache.null_slot
        for gi, g in enumerate(cache.groups):
            tbl = a[o[7 + gi]:o[8 + gi]].reshape(S, self.width)
            for s, e in enumerate(entries):
                row = cache.block_table(g.index, e.req)
                tbl[s, :len(row)] = row
                tbl[s, len(row):] = -1
            tbl[n:, 0] = g.null_page
            tbl[n:, 1:] = -1

    def run(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Pages for the new tokens are reserved already.  Returns logits [S, vocab] that stay
        valid until the next replay of this graph.  `device_tokens` (int32 [len(entries)] on the
        device) replace the entries' token ids: the tokens a step before has just drawn, which
        the host has not read yet."""
        lengths = [self.runner.cache.length(e.req) for e in entries]
        i = self.turn & 1
        self.turn += 1
        if self.copied[i] is not None:
            self.copied[i].synchronize()        # the copy that last read this buffer is done
        self._fill(self.nps[i], entries, lengths)
        self.dev.copy_(self.hosts[i], non_blocking=True)
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream(self.dev.device))
        self.copied[i] = done
        if device_tokens is not None:
            self.dev[self.offsets[0]:self.offsets[0] + len(entries)].copy_(device_tokens)
        self.graph.replay()
        klib.count_launches(self.kernels)
        return self.logits


class DecodeGraphs:
    """The runner's graphs, built on first use."""

    def __init__(self, runner, max_rows: int):
        self.runner, self.max_rows = runner, max_rows
        self.graphs: Dict[Tuple[int, int], DecodeGraph] = {}

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        return 0 < len(entries) <= self.max_rows and all(len(e.tokens) == 1 for e in entries)

    def get(self, entries: Sequence[StepEntry]) -> DecodeGraph:
        cache = self.runner.cache
        rows = row_bucket(len(entries))
        longest = max(cache.length(e.req) for e in entries) + 1
        key = (rows, context_bucket(longest, cache.max_context))
        if key not in self.graphs:
            self.graphs[key] = DecodeGraph(self.runner, *key)
        return self.graphs[key]
