"""A step's index data on the host: rows, positions, segments, wanted rows and block tables as
the kernels read them; what a step refuses; and the row and context counts a decode graph is
built for."""

import pytest
import torch

from ninfer_amd_mi50_b200.cache import CacheManager
from ninfer_amd_mi50_b200.engine.batch import BatchError, StepEntry, pack_step, validate_entries
from ninfer_amd_mi50_b200.engine.graphs import context_bucket, row_bucket
from ninfer_amd_mi50_b200.parts.base import CacheSpec

FULL = CacheSpec("full", 2, 16)
WIN = CacheSpec("window", 2, 16, 40)


def manager(specs=(FULL, WIN), pages=16, reqs=4, page=16, ctx=256):
    return CacheManager(list(specs), [None] * len(specs), page_size=page, num_pages=pages, max_requests=reqs,
                        max_context=ctx, allocate=False)


def test_rows_positions_segments_and_tables():
    m = manager()
    m.open("a"); m.open("b"); m.open("c")
    m.reserve("a", 37); m.commit("a", 37)              # a holds 37 tokens: its next rows start at 37
    m.reserve("c", 5); m.commit("c", 5)
    entries = [StepEntry("a", [11, 12, 13], [2]), StepEntry("b", [21, 22, 23, 24, 25], []),
               StepEntry("c", [31], [0])]
    for e in entries:
        m.reserve(e.req, m.length(e.req) + len(e.tokens))
    ctx = pack_step(entries, m, torch.float32, torch.device("cpu"))
    assert (ctx.T, ctx.S) == (9, 3)
    assert ctx.token_ids.tolist() == [11, 12, 13, 21, 22, 23, 24, 25, 31]
    assert ctx.positions.tolist() == [37, 38, 39, 0, 1, 2, 3, 4, 5]
    assert ctx.row_seg.tolist() == [0, 0, 0, 1, 1, 1, 1, 1, 2]
    assert ctx.seg_row0.tolist() == [0, 3, 8, 9]
    assert ctx.seg_pos0.tolist() == [37, 0, 5]
    assert ctx.seg_slot.tolist() == [m.slot("a"), m.slot("b"), m.slot("c")]
    assert ctx.logit_rows.tolist() == [2, 8]           # a's third token, c's only one
    assert ctx.seg_len_host == [3, 5, 1] and ctx.seg_pos0_host == [37, 0, 5]
    assert ctx.max_rows_per_seg == 5 and ctx.max_context == 40
    assert all(t.dtype == torch.int32 for t in (ctx.token_ids, ctx.positions, ctx.row_seg, ctx.logit_rows))
    for g in m.groups:
        tbl = ctx.block_tables[g.index]
        assert tbl.shape[0] == 3
        for i, e in enumerate(entries):
            held = m.block_table(g.index, e.req)
            assert tbl[i, :len(held)].tolist() == list(held)
            assert (tbl[i, len(held):] == -1).all()    # beyond a request's pages: no page
    # a holds ceil(40 / 16) = 3 pages of the full group, all different
    full = ctx.block_tables[m.groups[0].index][0, :3].tolist()
    assert len(set(full)) == 3 and min(full) >= 0


def test_a_fixed_table_width_pads_and_refuses():
    m = manager()
    m.open("a")
    m.reserve("a", 40)
    e = [StepEntry("a", list(range(40)), [39])]
    ctx = pack_step(e, m, torch.float32, torch.device("cpu"), table_width=8)
    assert all(t.shape == (1, 8) for t in ctx.block_tables.values())
    with pytest.raises(BatchError, match="wider"):
        pack_step(e, m, torch.float32, torch.device("cpu"), table_width=2)


def test_what_a_step_refuses():
    m = manager()
    m.open("a")
    ok = StepEntry("a", [1, 2], [1])
    validate_entries([ok], m, 100)
    for bad, what in [([ok, StepEntry("a", [3], [])], "twice"),
                      ([StepEntry("z", [1], [])], "not open"),
                      ([StepEntry("a", [], [])], "no tokens"),
                      ([StepEntry("a", [100], [])], "token id"),
                      ([StepEntry("a", [-1], [])], "token id"),
                      ([StepEntry("a", [1, 2], [2])], "wanted place")]:
        with pytest.raises(BatchError, match=what):
            validate_entries(bad, m, 100)


def test_graph_buckets():
    assert [row_bucket(n) for n in (1, 2, 7, 8)] == [1, 2, 7, 8]            # exact up to 8 rows
    assert [row_bucket(n) for n in (9, 16, 17, 32, 33, 64, 65)] == [16, 16, 32, 32, 64, 64, 128]
    assert context_bucket(1, 4096) == 512 and context_bucket(512, 4096) == 512
    assert context_bucket(513, 4096) == 1024
    assert context_bucket(4000, 4096) == 4096 and context_bucket(5000, 4096) == 4096   # never beyond the limit
    for n in range(1, 300):
        assert row_bucket(n) >= n
