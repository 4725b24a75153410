"""The scheduler's decisions, with a fake step: admission, portions under a budget,
decode first, finishing, and what happens when pages run out."""

import pytest

from ninfer_amd_mi50_b200.cache import CacheManager
from ninfer_amd_mi50_b200.engine.scheduler import Request, Scheduler
from ninfer_amd_mi50_b200.parts.base import CacheSpec
from ninfer_amd_mi50_b200.sampling import SamplingParams


def make(pages=8, reqs=4, budget=32, chunk=16, ctx=256, page=16):
    cache = CacheManager([CacheSpec("full", 1, 16)], [None], page_size=page, num_pages=pages,
                         max_requests=reqs, max_context=ctx, allocate=False)
    return cache, Scheduler(cache, max_batched_tokens=budget, prefill_chunk=chunk, max_context=ctx)


def req(i, n, max_new=4, stop=()):
    return Request(i, list(range(100 * i, 100 * i + n)), SamplingParams(temperature=0, max_new_tokens=max_new),
                   set(stop))


def run_step(cache, sch, token=lambda r: 7):
    """What the engine does around the model: commit lengths, hand back sampled tokens."""
    batch = sch.schedule()
    for s in batch:
        cache.commit(s.request.id, s.request.computed + len(s.tokens))
    sch.update(batch, [token(s.request) for s in batch if s.sample])
    cache.check()
    return batch


def test_prompt_is_cut_into_portions_under_the_budget():
    cache, sch = make(budget=24, chunk=16)
    sch.add(req(1, 40))
    sch.add(req(2, 10))
    b = run_step(cache, sch)
    assert [(s.request.id, len(s.tokens), s.sample) for s in b] == [(1, 16, False), (2, 8, False)]
    b = run_step(cache, sch)
    assert [(s.request.id, len(s.tokens), s.sample) for s in b] == [(1, 16, False), (2, 2, True)]
    b = run_step(cache, sch)      # request 2 decodes first, then request 1's last portion
    assert [(s.request.id, len(s.tokens), s.sample) for s in b] == [(2, 1, True), (1, 8, True)]
    assert b[1].tokens == list(range(132, 140))
    e = sch.entries(b)
    assert e[0].want == [0] and e[1].want == [7]


def test_decode_until_length_then_pages_come_back():
    cache, sch = make()
    sch.add(req(1, 5, max_new=3))
    steps = 0
    while not sch.idle:
        run_step(cache, sch)
        steps += 1
    r = sch.finished[0]
    assert steps == 3 and r.generated == [7, 7, 7] and r.finish_reason == "length"
    assert cache.pages_free() == [8] and not cache.requests
    assert sch.stats.prompt_tokens == 5 and sch.stats.decode_tokens == 2


def test_stop_id_and_context_limit():
    cache, sch = make(ctx=8)
    sch.add(req(1, 3, max_new=50, stop=(9,)))
    seq = iter([7, 9])
    while not sch.idle:
        run_step(cache, sch, token=lambda r: next(seq))
    assert sch.finished[0].finish_reason == "stop" and sch.finished[0].generated == [7, 9]
    sch.add(req(2, 6, max_new=50))
    while not sch.idle:
        run_step(cache, sch)
    assert sch.finished[1].finish_reason == "context" and len(sch.finished[1].tokens) == 8
    with pytest.raises(ValueError, match="max_context"):
        sch.add(req(3, 8))


def test_admission_is_first_come_first_served_and_bounded_by_slots():
    cache, sch = make(reqs=2, budget=64)
    for i in (1, 2, 3):
        sch.add(req(i, 4, max_new=2))
    b = run_step(cache, sch)
    assert [s.request.id for s in b] == [1, 2] and [r.id for r in sch.waiting] == [3]
    run_step(cache, sch)          # 1 and 2 finish (2 new tokens each); slot free again
    b = run_step(cache, sch)
    assert [s.request.id for s in b] == [3]


def test_out_of_pages_preempts_the_youngest_and_recomputes_it():
    cache, sch = make(pages=4, budget=64, chunk=64, reqs=3)
    sch.add(req(1, 30, max_new=40))      # 2 pages, grows into a 3rd at 32 and a 4th at 48
    sch.add(req(2, 14, max_new=40))      # 1 page, needs a 2nd at 16
    run_step(cache, sch)
    assert {r.id for r in sch.running} == {1, 2} and cache.pages_free() == [1]
    order = []
    for _ in range(80):
        if sch.idle:
            break
        b = run_step(cache, sch)
        order.append([(s.request.id, len(s.tokens)) for s in b])
    fin = {r.id: r for r in sch.finished}
    assert sch.stats.preemptions >= 1 and fin[2].preemptions >= 1 and fin[1].preemptions == 0
    # the older request ran every step until it finished
    assert fin[1].finish_reason in ("length", "out_of_cache")
    # the preempted one was recomputed from prompt + generated in one portion, then went on
    assert any(rid == 2 and n > 14 for step in order for rid, n in step)
    assert fin[2].finish_reason == "length" and len(fin[2].generated) == 40
    assert cache.pages_free() == [4]


def test_a_request_that_cannot_fit_alone_ends_with_out_of_cache():
    cache, sch = make(pages=2, budget=64, chunk=64)
    sch.add(req(1, 20, max_new=100))
    while not sch.idle:
        run_step(cache, sch)
    r = sch.finished[0]
    # both pages full: 32 tokens in the cache, and the 33rd, just sampled, has nowhere to go
    assert r.finish_reason == "out_of_cache" and r.computed == 32 and len(r.tokens) == 33
    assert cache.pages_free() == [2]
    # a prompt whose first portion is larger than the whole pool never starts
    sch.add(req(2, 50))
    assert run_step(cache, sch) == []
    assert sch.finished[1].finish_reason == "out_of_cache" and sch.idle


def test_sampling_is_independent_of_preemption():
    """The same requests with a roomy and with a tight pool generate the same tokens when the
    'model' is a function of the request's tokens so far."""
    def tok(r):
        return (sum(r.tokens) * 31 + len(r.tokens)) % 97

    outs = []
    for pages in (32, 5):
        cache, sch = make(pages=pages, budget=48, chunk=16, reqs=3)
        for i, n in ((1, 20), (2, 33), (3, 9)):
            sch.add(req(i, n, max_new=25))
        while not sch.idle:
            run_step(cache, sch, token=tok)
        outs.append({r.id: r.generated for r in sch.finished})
        assert all(r.finish_reason == "length" for r in sch.finished)
    assert outs[0] == outs[1]


def test_running_ahead_is_decided_without_the_coming_token():
    """`schedule_ahead` names the next decode batch before this one's tokens are known: only
    when every running request decodes and nobody waits; requests that finish by length with
    the coming token are left out; a request that stops on a stop token after all is skipped
    by `update`, and no page is lost either way."""
    cache, sch = make(pages=16, reqs=4, budget=32, chunk=16)
    sch.add(req(1, 5, max_new=3))
    sch.add(req(2, 7, max_new=6, stop=(9,)))
    b = sch.schedule()                                   # both prompts whole: not a decode step
    assert sch.schedule_ahead(b) is None
    for s in b:
        cache.commit(s.request.id, s.request.computed + len(s.tokens))
    sch.update(b, [7, 7])
    b = sch.schedule()                                   # first pure decode step (token 2 of each)
    assert [len(s.tokens) for s in b] == [1, 1]
    for s in b:
        cache.commit(s.request.id, s.request.computed + 1)
    nxt = sch.schedule_ahead(b)
    # request 1 has one token and gets its second now; max_new 3 -> it still runs ahead
    assert [s.request.id for s in nxt] == [1, 2] and all(s.sample and len(s.tokens) == 1 for s in nxt)
    for s in nxt:
        cache.commit(s.request.id, s.request.computed + 2)
    sch.update(b, [7, 9])                                # request 2 stops on its stop token
    assert [r.id for r in sch.finished] == [2]
    cache.check()
    # the step that ran ahead: request 2's row is ignored, request 1 gets its third token and ends
    done = sch.update(nxt, [7, 123])
    assert [r.id for r in done] == [1] and sch.finished[-1].generated == [7, 7, 7]
    assert sch.finished[0].generated == [7, 9]
    assert sch.idle and cache.pages_free() == [16]
    cache.check()
    # a request about to finish by length is left out of the step ahead
    sch.add(req(3, 4, max_new=2))
    sch.add(req(4, 4, max_new=5))
    b = sch.schedule()
    for s in b:
        cache.commit(s.request.id, s.request.computed + len(s.tokens))
    sch.update(b, [7, 7])
    b = sch.schedule()
    for s in b:
        cache.commit(s.request.id, s.request.computed + 1)
    nxt = sch.schedule_ahead(b)
    assert [s.request.id for s in nxt] == [4]
    # somebody waiting: no running ahead
    sch.add(req(5, 4))
    for s in nxt:
        cache.commit(s.request.id, s.request.computed + 2)
    sch.update(b, [7, 7])
    sch.update(nxt, [7])
    b = sch.schedule()
    assert any(len(s.tokens) > 1 for s in b) and sch.schedule_ahead(b) is None
