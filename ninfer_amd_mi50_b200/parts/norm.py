"""RMS normalisation, fused with the residual sum.

``inv = rsqrt(mean(x^2) + eps); y = x * inv * w`` with the weight multiplying directly
(src/ops/kernels.hip:17-41); the sum ``h += r`` happens in the same pass
(``fused_residual_rmsnorm_kernel``, src/ops/kernels.hip:100-129).  Here the residual
stream stays in float32 between layers, so the sum, the mean of squares and the product
are all 32-bit in both modes.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..registry import register_part
from .base import Fetch, Norm, RoutedSum, TensorSpec, summed


@register_part("norm", "rms_norm")
class RmsNorm(Norm):
    graph_safe = True
    takes_unsummed = True

    def __init__(self, size: int, eps: float, prefix: str):
        self.size, self.eps, self.prefix = int(size), float(eps), prefix
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.prefix + "weight", (self.size,), role="vector", init="norm")]

    def load(self, fetch: Fetch) -> None:
        self.weight = fetch(self.prefix + "weight")

    def weight_bytes(self) -> int:
        return self.size * 4

    def _fusable(self, delta, out_dtype, rows: int) -> bool:
        return (isinstance(delta, RoutedSum) and out_dtype == torch.bfloat16
                and kernels.can_fuse_combine_norm(delta.y, self.size, rows, delta.wts.shape[1]))

    def add_norm(self, h, delta, out_dtype):
        out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
        if self._fusable(delta, out_dtype, h.shape[0]):
            # the experts' weighted sum, the residual add and the norm in one kernel
            kernels.moe_combine_add_rmsnorm(delta.y, delta.plan, delta.wts, delta.shared, delta.gate, h, None,
                                            self.weight, self.eps, out)
        else:
            kernels.add_rmsnorm(h, summed(delta), self.weight, self.eps, out)
        return out

    def add_norm_rows(self, h, delta, rows, out_dtype):
        out = torch.empty((rows.numel(), h.shape[1]), dtype=out_dtype, device=h.device)
        if self._fusable(delta, out_dtype, rows.numel()):
            kernels.moe_combine_add_rmsnorm(delta.y, delta.plan, delta.wts, delta.shared, delta.gate, h, rows,
                                            self.weight, self.eps, out)
        else:
            kernels.add_rmsnorm_rows(h, summed(delta), rows, self.weight, self.eps, out)
        return out
