"""Rotary position embedding, half-split pairing.

For ``i < D/2``: ``angle = float(pos) * inv_freq[i]``, ``inv_freq[i] = theta^(-2i/D)``
evaluated in single precision on the host (src/models/model.hip:636-639);
``x'[i] = x[i] cos - x[i + D/2] sin``, ``x'[i + D/2] = x[i] sin + x[i + D/2] cos``
(src/ops/kernels.hip:73-94).  Applied to every query and key head, never to values.
The rotation itself runs inside the fused rotate-and-append kernel; this part owns the
table and the parameters.
"""

from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from ..registry import register_part
from .base import PositionEncoding


def rotary_inverse_frequencies(head_dim: int, theta: float, rotary_dim: Optional[int] = None
                               ) -> torch.Tensor:
    """float32 [rotary_dim / 2]: powf(theta, -2 i / D) with float operands."""
    rot = head_dim if rotary_dim is None else rotary_dim
    i = np.arange(rot // 2, dtype=np.float32)
    expo = (np.float32(-2.0) * i / np.float32(rot)).astype(np.float32)
    inv = np.power(np.float64(np.float32(theta)), expo.astype(np.float64)).astype(np.float32)
    return torch.from_numpy(inv)


@register_part("position", "rotary_half_split")
class RotaryHalfSplit(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None):
        self.head_dim, self.theta = int(head_dim), float(theta)
        self.rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and in (0, {head_dim}]")
        self._table = {}

    def rotary_table(self, device: torch.device) -> Optional[Tuple[torch.Tensor, int]]:
        key = str(device)
        if key not in self._table:
            self._table[key] = rotary_inverse_frequencies(
                self.head_dim, self.theta, self.rotary_dim).to(device)
        return self._table[key], self.rotary_dim


@register_part("position", "none")
class NoPosition(PositionEncoding):
    """No position information enters queries or keys."""

    def __init__(self, head_dim: int = 0):
        self.head_dim = head_dim

    def apply(self, q, k, positions) -> None:
        return None
