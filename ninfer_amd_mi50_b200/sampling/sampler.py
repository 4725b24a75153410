"""Choosing the next token from a row of logits.

The reference samples on the host from a copy of the logits (``sample_logits``,
src/runtime/engine.cpp:18-82): repetition penalty -> greedy if temperature <= 0 -> divide
by the temperature -> top-k -> softmax -> top-p -> inverse-CDF draw.  `Sampler` does the same
with device kernels; `sample_reference` is the host restatement used as the kernels' twin
and by ``Ninfer.sample`` when it is handed host logits.

Random draws are counter-based: the uniform number for a request's n-th new token depends
on (seed, n) only, so preempting a request and recomputing it later does not change what it
generates.  (The reference seeds a fresh Mersenne twister with ``seed + step`` per draw,
engine.cpp:166-169; the idea is the same, the generator is not.)
"""

from __future__ import annotations

from collections import Counter
from typing import List, Optional, Sequence

import torch

from .. import kernels
from .params import SamplingParams

_MASK = (1 << 64) - 1


def uniform_draw(seed: int, counter: int) -> float:
    """A float32-exact uniform number in [0, 1) from (seed, counter): splitmix64 mixing."""
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def check_params(p: SamplingParams, vocab: int) -> None:
    if p.greedy:
        return
    k = min(max(p.top_k, 1), vocab)
    if k > kernels.SAMPLE_MAX_TOP_K and not (k >= vocab and p.top_p >= 1.0):
        raise ValueError(
            f"top_k={p.top_k} is above {kernels.SAMPLE_MAX_TOP_K}; the device sampler takes a "
            f"larger top_k only as 'no limit' (top_k >= vocab) together with top_p >= 1")
    if p.repetition_penalty <= 0:
        raise ValueError("repetition_penalty must be positive")


def sample_reference(logits: Sequence[float], p: SamplingParams, recent: Sequence[int] = (),
                     draw: float = 0.0) -> int:
    """Host twin: same policy, same tie rules, same draw."""
    l = torch.as_tensor(logits, dtype=torch.float32).clone()
    V = l.numel()
    if p.repetition_penalty != 1.0:
        for tok in recent:
            if 0 <= tok < V:
                l[tok] = l[tok] / p.repetition_penalty if l[tok] > 0 else l[tok] * p.repetition_penalty
    if p.greedy:
        return int(torch.argmax(l))          # first maximum
    l = l * torch.tensor(1.0 / p.temperature, dtype=torch.float32)
    k = min(max(p.top_k, 1), V)
    if k >= V and p.top_p >= 1.0:
        e = torch.exp(l - l.max())
        cum = torch.cumsum(e, 0)
        hit = torch.nonzero(cum >= draw * e.sum())
        return int(hit[0]) if len(hit) else V - 1
    order = sorted(range(V), key=lambda i: (-float(l[i]), i))[:k]
    vals = l[order]
    prob = torch.exp(vals - vals[0])
    prob = prob / prob.sum()
    keep = k
    if p.top_p < 1.0:
        cum = 0.0
        for i in range(k):
            cum += float(prob[i])
            if cum >= p.top_p:
                keep = i + 1
                break
    prob = prob[:keep] / prob[:keep].sum()
    cum = 0.0
    for i in range(keep):
        cum += float(prob[i])
        if draw <= cum:
            return order[i]
    return order[keep - 1]


class Sampler:
    """Device sampling for a batch of rows with per-row parameters."""

    def __init__(self, vocab_size: int, device):
        self.vocab_size, self.device = vocab_size, torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               recent: Optional[Sequence[Sequence[int]]] = None,
               counters: Optional[Sequence[int]] = None) -> torch.Tensor:
        """logits float32 [R, V] on the device -> int32 [R] on the device.

        `recent[r]` are the ids the repetition penalty looks at (prompt and generated);
        `counters[r]` is the index of the token being drawn, the RNG counter."""
        R = logits.shape[0]
        if R == 0:
            return torch.empty((0,), dtype=torch.int32, device=self.device)
        dev = self.device
        # repetition penalty on a copy (the caller may still want the raw logits)
        pen_rows = [r for r in range(R) if params[r].repetition_penalty != 1.0 and recent and recent[r]]
        if pen_rows:
            logits = logits.clone()
            ids, counts, row_of = [], [], []
            for r in pen_rows:
                for tok, c in Counter(int(t) for t in recent[r]).items():
                    ids.append(tok); counts.append(c); row_of.append(r)
            mk = lambda v, dt: torch.tensor(v, dtype=dt).to(dev)
            pen = mk([p.repetition_penalty for p in params], torch.float32)
            kernels.repetition_penalty(logits, mk(ids, torch.int32), mk(counts, torch.int32),
                                       mk(row_of, torch.int32), pen)
        if all(p.greedy for p in params):
            return kernels.argmax_rows(logits)
        out = kernels.argmax_rows(logits)
        rows = [r for r in range(R) if not params[r].greedy]
        for r in rows:
            check_params(params[r], self.vocab_size)
        sel = torch.tensor(rows, dtype=torch.long, device=dev)
        sub = logits.index_select(0, sel) if len(rows) < R else logits
        temp = torch.tensor([params[r].temperature for r in rows], dtype=torch.float32).to(dev)
        topk = torch.tensor([params[r].top_k for r in rows], dtype=torch.int32).to(dev)
        topp = torch.tensor([params[r].top_p for r in rows], dtype=torch.float32).to(dev)
        draws = torch.tensor([uniform_draw(params[r].seed, counters[r] if counters else 0) for r in rows],
                             dtype=torch.float32).to(dev)
        picked = kernels.sample_rows(sub.contiguous(), temp, topk, topp, draws)
        if len(rows) == R:
            return picked
        out.index_copy_(0, sel, picked)
        return out
