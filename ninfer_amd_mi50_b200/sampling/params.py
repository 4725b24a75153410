"""Sampling parameters, with the reference's names, meanings and defaults
(``SamplingParams``, src/runtime/engine.h:15-22; CLI flags src/apps/ninfer.cpp:55-76)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 0.7          # <= 0: greedy (first maximum)
    top_k: int = 50                   # clamped to [1, vocab]
    top_p: float = 0.95               # >= 1: no nucleus cut
    repetition_penalty: float = 1.0   # 1: off (the CLI's default is 1.05, as in the reference)
    seed: int = 0                     # 0: a fresh seed per request
    max_new_tokens: int = 512

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0
