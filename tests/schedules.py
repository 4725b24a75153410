"""Ways of cutting the same requests into steps.  Every schedule asks for the logits at
every position, so that the result can be laid beside the plain model's whole-sequence
logits position by position.

A schedule is a list of steps; a step is ``{"entries": [{"id", "tokens", "want"}], "end": [ids]}``,
which is also the record format of ``bin/trace_run`` (plus its "step" number).
"""

from typing import Dict, List, Sequence

CUTS = [7, 2, 13, 2, 5, 31, 3, 64, 2, 17]


def _entry(rid, toks):
    return {"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}


def whole(reqs: Dict[str, Sequence[int]]) -> List[dict]:
    """Each request alone, all of it in one step."""
    return [{"entries": [_entry(r, t)], "end": [r]} for r, t in reqs.items()]


def tail_decoded(reqs, tail: int = 32) -> List[dict]:
    """Each request alone: all but the last `tail` tokens in one step, then one by one."""
    steps = []
    for r, t in reqs.items():
        head = max(1, len(t) - tail)
        steps.append({"entries": [_entry(r, t[:head])], "end": []})
        for i in range(head, len(t)):
            steps.append({"entries": [_entry(r, t[i:i + 1])], "end": []})
        steps[-1]["end"] = [r]
    return steps


def portions(reqs, cuts=CUTS) -> List[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for r, t in reqs.items():
        i, c = 0, 0
        while i < len(t):
            n = min(cuts[c % len(cuts)], len(t) - i)
            steps.append({"entries": [_entry(r, t[i:i + n])], "end": []})
            i += n
            c += 1
        steps[-1]["end"] = [r]
    return steps


def mixed(reqs, max_live: int = 4, page: int = 64, pool_tokens: int = 0, tail: int = 12,
          cuts=CUTS) -> List[dict]:
    """Up to `max_live` requests at a time, portions of some beside single tokens of
    others.  A request is admitted only when the pool (``pool_tokens``, counted in whole
    pages per request) has room for all of it, so with a small pool later requests take
    the pages that earlier ones gave back."""
    names = list(reqs)
    waiting = list(names)
    live: List[str] = []
    done = {r: 0 for r in names}
    turn = {r: i for i, r in enumerate(names)}
    steps = []

    def held(r):
        return (len(reqs[r]) + page - 1) // page * page

    while waiting or live:
        while waiting and len(live) < max_live:
            r = waiting[0]
            if pool_tokens and sum(held(x) for x in live) + held(r) > pool_tokens:
                if not live:
                    raise ValueError("pool too small for one request")
                break
            live.append(waiting.pop(0))
        entries = []
        for r in live:
            left = len(reqs[r]) - done[r]
            if left <= tail:
                n = 1
            else:
                n = min(cuts[turn[r] % len(cuts)], left - tail)
                turn[r] += 1
            # a live request sits out a step now and then
            if (len(steps) + turn[r]) % 5 == 4 and len(live) > 1 and entries:
                continue
            entries.append(_entry(r, reqs[r][done[r]:done[r] + n]))
            done[r] += n
        end = [r for r in live if done[r] == len(reqs[r])]
        steps.append({"entries": entries, "end": end})
        live = [r for r in live if r not in end]
    return steps


def run_schedule(runner, steps, routing: Dict[str, Dict[int, List]] = None) -> Dict[str, List]:
    """Drive a ModelRunner through a schedule; return per-request lists of logits rows.

    `routing`, if given, is filled with the experts the engine chose:
    routing[request][layer] = int64 tensor [request's tokens, k], layer by sparse layer."""
    import torch
    from ninfer_amd_mi50_b200.engine import StepEntry
    from ninfer_amd_mi50_b200.parts.feedforward import SparseMoeSwiglu
    got: Dict[str, List] = {}
    sparse_calls = [c.layer for c in runner.model.order
                    if isinstance(runner.model.blocks[c.layer].feed_forward, SparseMoeSwiglu)]
    chosen: Dict[str, Dict[int, List]] = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if not runner.cache.is_open(e["id"]):
                runner.open(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        if routing is not None:
            SparseMoeSwiglu.record_routing = []
        try:
            out = runner.step(entries)
            record = SparseMoeSwiglu.record_routing
        finally:
            SparseMoeSwiglu.record_routing = None
        r = row = 0
        for e in st["entries"]:
            n = len(e["want"])
            got.setdefault(e["id"], []).append(out[r:r + n].float().cpu())
            r += n
            if routing is not None:
                assert len(record) == len(sparse_calls)
                for layer, idx in zip(sparse_calls, record):
                    chosen.setdefault(e["id"], {}).setdefault(layer, []).append(
                        idx[row:row + len(e["tokens"])].long().cpu())
            row += len(e["tokens"])
        for rid in st["end"]:
            runner.close(rid)
        runner.cache.check()
    if routing is not None:
        for rid, layers in chosen.items():
            routing[rid] = {l: torch.cat(v) for l, v in layers.items()}
    return {k: torch.cat(v) for k, v in got.items()}
