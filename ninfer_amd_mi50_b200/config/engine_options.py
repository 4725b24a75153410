"""Engine options: what a user chooses at start-up, as opposed to what config.json fixes.

`max_context`, `prefill_chunk` and `num_sequences` keep the names and meanings of the
reference's ``ModelOptions`` (src/models/model.h:37-50) and C options struct
(src/api/ninfer_c_api.h:20-28), and its defaults but one: a prompt's portion is 2,048 tokens,
not 512.  Every portion reads every expert's weights once, so on a B200 a prompt in portions of
512 runs at 63 K tokens/s, in portions of 2,048 at 149-167 K, of 8,192 at 185 K (A2.7B sizes).  The paged cache adds `page_size` and `cache_tokens`,
the scheduler adds `max_batched_tokens`, and `dtype` picks the bfloat16 serving path or
the all-32-bit path.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"          # "bfloat16" | "float32"
    max_context: int = 32768         # most tokens one request may hold
    prefill_chunk: int = 2048        # largest portion of one prompt in one step
    num_sequences: int = 1           # most live requests
    page_size: int = 64              # tokens per cache page
    cache_tokens: Optional[int] = None   # pool size in tokens (default: num_sequences * max_context)
    max_batched_tokens: Optional[int] = None  # token budget of one step
    use_graph: bool = True           # replay decode-only steps from CUDA graphs
    run_ahead: bool = True           # launch the next decode step before reading this one's tokens
    status_every: int = 64           # decode steps between two reads of the kernels' status flags
    clear_reused_pages: bool = True  # zero a cache page when it is handed out a second time
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {self.dtype!r}")
        self.dtype = DTYPES[self.dtype]
        # the reference treats non-positive values as "use the default"
        # (src/api/ninfer_c_api.cpp:54-82)
        if self.max_context <= 0:
            self.max_context = 32768
        if self.prefill_chunk <= 0:
            self.prefill_chunk = 2048
        if self.num_sequences <= 0:
            self.num_sequences = 1
        if self.page_size <= 0 or self.page_size % 16:
            raise ValueError(f"page_size must be a positive multiple of 16, got {self.page_size}")
        if self.cache_tokens is None:
            self.cache_tokens = self.num_sequences * self.pages_for(self.max_context) * self.page_size
        if self.max_batched_tokens is None:
            self.max_batched_tokens = max(self.prefill_chunk, self.num_sequences)
        if self.max_batched_tokens < 1:
            raise ValueError("max_batched_tokens must be at least 1")

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    @property
    def num_pages(self) -> int:
        return self.pages_for(int(self.cache_tokens))
