"""Grouped-query causal attention over a paged cache.

Order of work, as in ``Shard::layer_start`` (src/models/model.hip:206-306):
``qkv = x Wqkv^T`` with q, k, v concatenated on rows at load (model.hip:530-545), row
layout ``[q: Hq*D | k: Hkv*D | v: Hkv*D]``; rotate q and k; write k and v at
(request, position); attention; ``o = attn Wo^T``.  Query head ``h`` reads key/value head
``h // (Hq / Hkv)`` (src/ops/attention.hip:27-28), scores are scaled by ``1/sqrt(D)``
(model.hip:285), key ``j`` is visible to a row at position ``p`` iff ``j <= p``
(attention.hip:216).  The reference loads no q/k/v bias; Qwen2-MoE has one, added before
the rotation.  With a window ``w`` a key is visible iff ``p - w < j <= p``.
"""

from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import kernels
from ..config.model_config import PartSpec
from ..registry import build_part, register_part
from .base import CacheSpec, CacheView, Fetch, Mixer, StepContext, TensorSpec


@register_part("mixer", "paged_gqa_attention")
class PagedGqaAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position: PartSpec, prefix: str,
                 window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        kernels.check_head_dim(head_dim)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.num_kv_heads, self.head_dim = int(num_kv_heads), int(head_dim)
        self.qkv_bias, self.window, self.prefix = bool(qkv_bias), window, prefix
        self.position = build_part("position", position)
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.w_qkv = self.b_qkv = self.w_o = None

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        specs = [TensorSpec(p + "q_proj.weight", (self.q_width, H)),
                 TensorSpec(p + "k_proj.weight", (self.kv_width, H)),
                 TensorSpec(p + "v_proj.weight", (self.kv_width, H)),
                 TensorSpec(p + "o_proj.weight", (H, self.q_width))]
        if self.qkv_bias:
            specs += [TensorSpec(p + "q_proj.bias", (self.q_width,), role="vector"),
                      TensorSpec(p + "k_proj.bias", (self.kv_width,), role="vector"),
                      TensorSpec(p + "v_proj.bias", (self.kv_width,), role="vector")]
        return specs

    def load(self, fetch: Fetch) -> None:
        p = self.prefix
        self.w_qkv = torch.cat([fetch(p + f"{n}_proj.weight") for n in "qkv"], dim=0).contiguous()
        self.w_o = fetch(p + "o_proj.weight")
        if self.qkv_bias:
            self.b_qkv = torch.cat([fetch(p + f"{n}_proj.bias") for n in "qkv"]).contiguous()

    def weight_bytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        return n + (self.b_qkv.numel() * 4 if self.b_qkv is not None else 0)

    # ---- cache ------------------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        kind = "window" if self.window else "full"
        return CacheSpec(kind, self.num_kv_heads, self.head_dim, self.window)

    def check_limits(self, dtype: torch.dtype, max_context: int, page_size: int) -> None:
        kernels.check_attention_limits(dtype, self.head_dim, max_context, page_size)

    # ---- forward ----------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        assert cache is not None, "attention needs a cache slot"
        Hq, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        table = self.position.rotary_table(x.device)
        bias = self.b_qkv
        if table is None:
            # an encoding that is not a half-split rotation: bias first, then its own hook
            qkv = kernels.linear(x, self.w_qkv)
            if bias is not None:
                qkv.add_(bias.to(qkv.dtype))
                bias = None
            q = qkv[:, :self.q_width].unflatten(1, (Hq, D))
            k = qkv[:, self.q_width:self.q_width + self.kv_width].unflatten(1, (Hkv, D))
            self.position.apply(q, k, ctx.positions)
            kernels.rope_append(qkv, None, ctx.positions, ctx.row_seg, None, 0, Hq, Hkv, D,
                                cache.pages, cache.block_table, cache.page_size, cache.append)
        else:
            # projection, bias, rotation and the write of k, v at (request, position): one kernel
            # on small bfloat16 steps, two otherwise
            inv_freq, rot = table
            qkv = kernels.linear_rope_append(x, self.w_qkv, bias, ctx.positions, ctx.row_seg, inv_freq, rot,
                                             Hq, Hkv, D, cache.pages, cache.block_table, cache.page_size,
                                             cache.append)
        out = kernels.paged_attention(qkv, Hq, Hkv, D, cache.pages, cache.block_table,
                                      cache.page_size, ctx, self.window or 0, self.scale)
        return kernels.linear(out, self.w_o)
