"""The generic decoder: embedding, a list of blocks run in a given order, final norm,
output head.

Reference counterpart: ``Impl::forward_batch`` (src/models/model.hip:994-1032) with
``begin_rows`` (embedding gather, 697-724), the per-layer loop (1021-1025) and
``finalize`` (727-755: final RMSNorm and LM head only on the rows whose logits are
wanted; the head is the embedding matrix when ``tie_word_embeddings``, 497-499).
Which blocks exist and in which order they run is data (`ModelPlan`), not code.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from .. import kernels
from ..config.model_config import LayerCall, ModelPlan
from ..registry import build_part, part_class
from .base import CacheSpec, CacheView, Fetch, StateSpec, StepContext, TensorSpec, summed


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        self.plan = plan
        self.vocab_size, self.hidden_size = plan.vocab_size, plan.hidden_size
        self.blocks = []
        for spec in plan.layers:
            norm1 = build_part("norm", spec.norm, prefix=spec.name_of("norm1"))
            mixer = build_part("mixer", spec.mixer, prefix=spec.name_of("mixer"))
            norm2 = build_part("norm", spec.norm, prefix=spec.name_of("norm2"))
            ffn = build_part("feed_forward", spec.feed_forward, prefix=spec.name_of("feed_forward"))
            self.blocks.append(part_class("block", spec.arrangement)(norm1, mixer, norm2, ffn))
        self.final_norm = build_part("norm", plan.final_norm, prefix=plan.final_norm_name)
        self.order: List[LayerCall] = list(plan.order)
        for call in self.order:
            if not (0 <= call.layer < len(self.blocks) and 0 <= call.cache < len(self.blocks)):
                raise ValueError(f"execution order names a layer that does not exist: {call}")
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    # ---- what the model needs ---------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        V, H = self.vocab_size, self.hidden_size
        specs = [TensorSpec(self.plan.embedding_name, (V, H))]
        for b in self.blocks:
            specs += b.tensor_specs()
        specs += self.final_norm.tensor_specs()
        if not self.plan.tie_word_embeddings:
            specs.append(TensorSpec(self.plan.head_name, (V, H)))
        return specs

    def load(self, fetch: Fetch) -> None:
        self.embedding = fetch(self.plan.embedding_name)
        for b in self.blocks:
            b.load(fetch)
        self.final_norm.load(fetch)
        self.head = self.embedding if self.plan.tie_word_embeddings else fetch(self.plan.head_name)

    def cache_specs(self) -> List[Optional[CacheSpec]]:
        """Slot i belongs to layer i; None if that layer keeps nothing in pages."""
        return [b.cache_spec() for b in self.blocks]

    def state_specs(self) -> List[Optional[StateSpec]]:
        return [b.state_spec() for b in self.blocks]

    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe

    def check_limits(self, dtype: torch.dtype, max_context: int, page_size: int) -> None:
        for b in self.blocks:
            b.check_limits(dtype, max_context, page_size)
        self.final_norm.check_limits(dtype, max_context, page_size)

    def weight_bytes(self) -> int:
        n = sum(b.weight_bytes() for b in self.blocks) + self.final_norm.weight_bytes()
        return n + self.head.numel() * self.head.element_size()

    # ---- one pass over the step's rows --------------------------------------------------
    def forward(self, ctx: StepContext,
                cache_view: Callable[[int, bool], Optional[CacheView]],
                state_of: Callable[[int], Optional[torch.Tensor]]) -> torch.Tensor:
        """Run every row of the step; return float32 logits [R, vocab] for ctx.logit_rows."""
        h = torch.empty((ctx.T, self.hidden_size), dtype=torch.float32, device=ctx.device)
        kernels.embed_rows(self.embedding, ctx.token_ids, h)
        pending = None
        for call in self.order:
            pending = self.blocks[call.layer].forward(
                h, pending, ctx, cache_view(call.cache, call.append), state_of(call.layer))
        R = ctx.logit_rows.numel()
        if R == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=ctx.device)
        if not self.final_norm.takes_unsummed:
            pending = summed(pending)
        x = self.final_norm.add_norm_rows(h, pending, ctx.logit_rows, ctx.dtype)
        return kernels.linear(x, self.head, out_dtype=torch.float32)
