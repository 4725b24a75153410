"""Turning a step's entries into the index tensors the kernels read.

An entry is (request, its next tokens, which of them want logits).  The reference's step
takes parallel arrays ``tokens / positions / seq_ids`` and finds the runs of equal
``seq_id`` itself (``build_groups``, src/models/model.hip:950-961); here the runs
(*segments*) are explicit, positions come from the cache manager's record of each
request's length, and everything is packed into one int32 buffer that crosses to the
device in a single copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import StepContext


@dataclass
class StepEntry:
    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()      # indices into `tokens` whose logits are asked for


class BatchError(ValueError):
    pass


def validate_entries(entries: Sequence[StepEntry], cache: CacheManager, vocab_size: int) -> None:
    seen = set()
    for e in entries:
        if e.req in seen:
            raise BatchError(f"request {e.req!r} appears twice in one step")
        seen.add(e.req)
        if not cache.is_open(e.req):
            raise BatchError(f"request {e.req!r} is not open")
        if len(e.tokens) == 0:
            raise BatchError(f"request {e.req!r} brings no tokens")
        toks = np.asarray(e.tokens, dtype=np.int64)     # one pass in numpy: a long portion has thousands
        bad = np.flatnonzero((toks < 0) | (toks >= vocab_size))
        if bad.size:
            raise BatchError(f"request {e.req!r}: token id {int(toks[bad[0]])} outside [0, {vocab_size})")
        for w in e.want:
            if not 0 <= int(w) < len(e.tokens):
                raise BatchError(f"request {e.req!r}: wanted place {w} outside its {len(e.tokens)} tokens")


def pack_step(entries: Sequence[StepEntry], cache: CacheManager, dtype: torch.dtype,
              device: torch.device, *, table_width: Optional[int] = None) -> StepContext:
    """Build the step's metadata.  Pages for the new tokens must be reserved already."""
    S = len(entries)
    # numpy pieces, not Python lists: a 2,048-token portion was 0.85 ms of list building here
    pieces_tok, pieces_pos, pieces_seg = [], [], []
    seg_row0 = [0]
    seg_pos0: List[int] = []
    seg_slot: List[int] = []
    logit_rows: List[int] = []
    seg_len: List[int] = []
    for s, e in enumerate(entries):
        n = len(e.tokens)
        pos0 = cache.length(e.req)
        row0 = seg_row0[-1]
        pieces_tok.append(np.asarray(e.tokens, dtype=np.int32))
        pieces_pos.append(np.arange(pos0, pos0 + n, dtype=np.int32))
        pieces_seg.append(np.full(n, s, dtype=np.int32))
        seg_row0.append(row0 + n)
        seg_pos0.append(pos0)
        seg_slot.append(cache.slot(e.req))
        seg_len.append(n)
        logit_rows += [row0 + int(w) for w in e.want]
    T = seg_row0[-1]
    # block tables, one per cache group, padded to a common width with -1
    tables = []
    for g in cache.groups:
        rows = [cache.block_table(g.index, e.req) for e in entries]
        width = table_width or max(1, max(len(r) for r in rows))
        tbl = np.full((S, width), -1, dtype=np.int32)
        for i, r in enumerate(rows):
            if len(r) > width:
                raise BatchError("a block table is wider than the step's table width")
            tbl[i, :len(r)] = r
        tables.append((g.index, width, tbl.reshape(-1)))
    sizes = [T, T, T, S + 1, S, S, len(logit_rows)] + [S * w for _, w, _ in tables]
    small = lambda v: np.asarray(v, dtype=np.int32)
    flat_all = np.concatenate(pieces_tok + pieces_pos + pieces_seg +
                              [small(seg_row0), small(seg_pos0), small(seg_slot), small(logit_rows)] +
                              [f for _, _, f in tables])
    buf = torch.from_numpy(flat_all)
    host_bytes = buf.numel() * 4
    if device.type == "cuda":
        buf = buf.pin_memory().to(device, non_blocking=True)
    parts = list(torch.split(buf, sizes))
    ctx = StepContext(
        dtype=dtype, device=device, T=T, S=S,
        token_ids=parts[0], positions=parts[1], row_seg=parts[2], seg_row0=parts[3],
        seg_pos0=parts[4], seg_slot=parts[5], logit_rows=parts[6],
        seg_len_host=seg_len, seg_pos0_host=seg_pos0,
        max_rows_per_seg=max(seg_len) if seg_len else 0,
        max_context=max((p + n for p, n in zip(seg_pos0, seg_len)), default=0))
    ctx.scratch["h2d_bytes"] = host_bytes
    for (gi, width, _), t in zip(tables, parts[7:]):
        ctx.block_tables[gi] = t.view(S, width)
    return ctx
