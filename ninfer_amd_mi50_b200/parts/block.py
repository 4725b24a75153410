"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

Pre-norm, as the reference runs a layer (src/models/model.hip:206-444):
``x1 = norm1(h)`` -> mixer -> ``h += o`` fused with ``x2 = norm2(h)`` (model.hip:311) ->
feed-forward -> ``h += ffn``.  The last sum is left pending so that it fuses with the next
block's first norm, which is what the reference's ``fused_residual_rmsnorm`` does one
stage earlier.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from ..registry import register_part
from .base import Block, CacheView, FeedForward, Fetch, Mixer, Norm, StepContext, TensorSpec, summed


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, feed_forward: FeedForward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()]

    def load(self, fetch: Fetch) -> None:
        for p in self.parts():
            p.load(fetch)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts())

    def check_limits(self, dtype, max_context, page_size) -> None:
        for p in self.parts():
            p.check_limits(dtype, max_context, page_size)

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: Optional[CacheView], state: Optional[torch.Tensor]
                ) -> Optional[torch.Tensor]:
        if not self.norm1.takes_unsummed:
            pending = summed(pending)
        x1 = self.norm1.add_norm(h, pending, ctx.dtype)
        a = self.mixer.forward(x1, ctx, cache, state)
        x2 = self.norm2.add_norm(h, a, ctx.dtype)
        return self.feed_forward.forward(x2, ctx)
