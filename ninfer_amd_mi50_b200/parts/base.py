"""Interfaces that every part of a layer implements, and the step's shared metadata.

A part knows its own sizes and constants (constructor arguments that come from the
configuration through a `PartSpec`) and the names of its own tensors below a prefix.
It does not know which model it is in, how many layers there are, or what the other
parts of its block are.

Reference counterpart: ``Shard::layer_start`` / ``layer_mid`` / ``end_layer``
(src/models/model.hip:206-444) hard-wire one attention and one MLP/MoE into a
function; here the same stages are objects chosen layer by layer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------------------
# Tensors a part needs from the checkpoint
# --------------------------------------------------------------------------------------

@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part asks for.

    role:  "matrix" - held in the engine dtype (bfloat16 or float32);
           "vector" - norm weights and biases, held in float32 in both modes (a
                      bfloat16 value widens exactly; a tensor stored in 32-bit stays so);
           "router" - routing matrices, held in float32 for the same reason;
           "table"  - integer tables, held as int32.
    init:  distribution for the random-weights mode: "linear" N(0, 0.02),
           "norm" 1 + N(0, 0.05).
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "linear"


Fetch = Callable[[str], torch.Tensor]   # tensor name -> device tensor in its role's dtype


# --------------------------------------------------------------------------------------
# What a mixer asks of the cache manager
# --------------------------------------------------------------------------------------

@dataclass(frozen=True)
class CacheSpec:
    """What one cache slot keeps per token, in pages.

    kind "full": every entry stays until the request ends.
    kind "window": only the last `window` entries are read; pages that the window has
    passed go back to the pool.

    The usual form is keys and values of `num_kv_heads` heads of `head_dim`: a page is
    ``[2, num_kv_heads, page_size, head_dim]`` (keys, then values; one head's keys of a page are
    one contiguous run), which is what the attention kernels read.  A mixer that keeps
    something else per token (one compressed latent row, keys and values of different widths
    packed side by side) gives `row_width` instead: a page is then ``[page_size, row_width]``
    and the mixer reads and writes it itself.  The cache manager only ever asks `page_shape`.
    """
    kind: str
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    row_width: int = 0

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        if self.row_width:
            return (page_size, self.row_width)
        return (2, self.num_kv_heads, page_size, self.head_dim)

    def elements_per_token(self) -> int:
        return self.row_width if self.row_width else 2 * self.num_kv_heads * self.head_dim

    def group_key(self) -> Tuple:
        return (self.kind, self.num_kv_heads, self.head_dim, self.window, self.row_width)


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one tensor of `shape` per live request."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheView:
    """What a mixer call sees of one cache slot during a step."""
    spec: CacheSpec
    pages: torch.Tensor          # [num_pages + 1, *spec.page_shape(page_size)]
    block_table: torch.Tensor    # int32 [S, width]: page of (segment, position // page_size)
    page_size: int
    append: bool = True


# --------------------------------------------------------------------------------------
# The step's metadata, shared by all parts
# --------------------------------------------------------------------------------------

@dataclass
class StepContext:
    """Everything about a step that is not the hidden state.

    Rows are the step's tokens in order; a *segment* is one request's run of rows
    (a portion of a prompt, or one decoded token).  All index tensors are int32 on the
    device.  `seg_len_host` / `seg_pos0_host` are host copies for grid sizing; they are
    absent in graph mode, where only the bounds `max_rows_per_seg` and `max_context`
    may shape a launch.
    """
    dtype: torch.dtype
    device: torch.device
    T: int
    S: int
    token_ids: torch.Tensor        # [T]
    positions: torch.Tensor        # [T] absolute position of each row in its request
    row_seg: torch.Tensor          # [T] segment of each row
    seg_row0: torch.Tensor         # [S + 1] first row of each segment
    seg_pos0: torch.Tensor         # [S] tokens the request held before this step
    seg_slot: torch.Tensor         # [S] state slot of each segment's request
    logit_rows: torch.Tensor       # [R] rows whose logits are wanted
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)  # per cache group
    seg_len_host: Optional[List[int]] = None
    seg_pos0_host: Optional[List[int]] = None
    max_rows_per_seg: int = 1
    max_context: int = 0           # bound on pos0 + rows over the segments of this step
    graph_mode: bool = False
    scratch: Dict[str, torch.Tensor] = field(default_factory=dict)
    _tiles: Dict[object, Tuple[torch.Tensor, int]] = field(default_factory=dict)

    @property
    def all_single(self) -> bool:
        """Every segment brings exactly one row (a decode-only step)."""
        return self.max_rows_per_seg == 1

    def query_tiles(self, rows_per_tile: int) -> Tuple[torch.Tensor, int]:
        """Tiles of at most `rows_per_tile` consecutive rows of one segment.

        Returns (int32 [n, 2] of (segment, first row), n).  Built on the host from the
        segment lengths; not available in graph mode.
        """
        if rows_per_tile in self._tiles:
            return self._tiles[rows_per_tile]
        if self.seg_len_host is None:
            raise RuntimeError("query_tiles needs host segment lengths (not in graph mode)")
        flat: List[int] = []
        row = 0
        for s, n in enumerate(self.seg_len_host):
            for r in range(0, n, rows_per_tile):
                flat += [s, row + r]
            row += n
        n_tiles = len(flat) // 2
        t = torch.tensor(flat, dtype=torch.int32).reshape(n_tiles, 2).to(self.device)
        self._tiles[rows_per_tile] = (t, n_tiles)
        return t, n_tiles


    def single_rows(self) -> Tuple[Optional[torch.Tensor], int]:
        """Rows of the segments that bring exactly one row (decoded tokens, or a prompt's last
        token arriving alone), as (int32 tensor on the device, count); (None, 0) if there are
        none.  Attention serves such a row with its split-key kernel whatever else the step
        holds.  Built on the host; not available in graph mode."""
        if "single" in self._tiles:
            return self._tiles["single"]
        if self.seg_len_host is None:
            raise RuntimeError("single_rows needs host segment lengths (not in graph mode)")
        rows, row = [], 0
        for n in self.seg_len_host:
            if n == 1:
                rows.append(row)
            row += n
        out = (torch.tensor(rows, dtype=torch.int32).to(self.device), len(rows)) if rows else (None, 0)
        self._tiles["single"] = out
        return out

    def paired_query_tiles(self, rows_per_tile: int, window: int, keys_per_block: int,
                           pair: bool = True, min_rows: int = 1) -> Tuple[torch.Tensor, int]:
        """Query tiles two to a CTA, a heavy one with a light one.

        A tile late in a long prompt reads many more keys than an early one; giving each CTA
        the i-th heaviest and the i-th lightest tile makes CTAs about equally long.  Returns
        (int32 [n_pairs, 2, 2] of (segment, first row), second entry (-1, -1) if there is
        none; n_pairs).  With `pair` false every CTA gets one tile, heaviest first.  Segments
        with fewer than `min_rows` rows are left out (they are served elsewhere)."""
        key = ("pairs", rows_per_tile, window, keys_per_block, pair, min_rows)
        if key in self._tiles:
            return self._tiles[key]
        if self.seg_len_host is None or self.seg_pos0_host is None:
            raise RuntimeError("paired_query_tiles needs host segment lengths (not in graph mode)")
        tiles = []
        row = 0
        for s, (n, pos0) in enumerate(zip(self.seg_len_host, self.seg_pos0_host)):
            for r in range(0, n if n >= min_rows else 0, rows_per_tile):
                first = pos0 + r
                last = pos0 + min(r + rows_per_tile, n) - 1
                lo = max(0, first - window + 1) if window > 0 else 0
                work = last // keys_per_block - lo // keys_per_block + 1
                tiles.append((work, s, row + r))
            row += n
        tiles.sort(key=lambda t: -t[0])
        flat: List[int] = []
        if not pair:
            # one tile a CTA, heaviest first: the device hands CTAs to SMs as they fall free, so
            # the light tiles fill the end
            for _, s, r in tiles:
                flat += [s, r, -1, -1]
        i, j = (0, len(tiles) - 1) if pair else (1, 0)
        while i <= j:
            flat += [tiles[i][1], tiles[i][2]]
            flat += [tiles[j][1], tiles[j][2]] if j > i else [-1, -1]
            i, j = i + 1, j - 1
        n_pairs = len(flat) // 4
        t = torch.tensor(flat, dtype=torch.int32).reshape(n_pairs, 2, 2).to(self.device)
        self._tiles[key] = (t, n_pairs)
        return t, n_pairs


# --------------------------------------------------------------------------------------
# Part interfaces
# --------------------------------------------------------------------------------------

class Part:
    """Common to all parts: which tensors it needs and how it takes them."""

    # True if `forward` only launches work on the current stream from device-side data
    # (no host reads of the step's contents), so that a step may be captured in a CUDA graph.
    graph_safe = False

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, fetch: Fetch) -> None:
        """Pull this part's tensors (`fetch(name)`), fusing or stacking as it likes."""

    def weight_bytes(self) -> int:
        """Bytes of weights one forward call reads when every row uses everything."""
        return 0

    def check_limits(self, dtype: torch.dtype, max_context: int, page_size: int) -> None:
        """Raise ValueError if this part's kernels cannot serve the engine's options.  Called
        once at start-up, so that a limit is met there and not in the middle of a request."""


@dataclass
class RoutedSum:
    """A feed-forward's output that has not been added up yet:

        out[t] = sum_j wts[t, j] * y[plan.inv[t * k + j]]  (+ sigmoid(gate[t]) * shared[t])

    A block hands it on as its pending contribution; a norm that knows the form (`takes_unsummed`)
    adds it up inside its own kernel, any other consumer calls `materialize()` first.
    """
    y: torch.Tensor                      # [T * k, hidden] expert outputs in sorted order
    plan: object                         # the routing plan (`inv` is what is used)
    wts: torch.Tensor                    # float32 [T, k]
    shared: Optional[torch.Tensor]       # [T, hidden] or None
    gate: Optional[torch.Tensor]         # float32 [T, 1] gate logits or None
    dtype: torch.dtype = torch.bfloat16

    def materialize(self) -> torch.Tensor:
        from .. import kernels
        return kernels.moe_combine(self.y, self.plan, self.wts, self.shared, self.gate, self.dtype)


def summed(delta):
    """`delta` as a tensor (None stays None)."""
    return delta.materialize() if isinstance(delta, RoutedSum) else delta


class Norm(Part):
    """Normalisation fused with the residual sum.

    The residual stream `h` is float32 in both modes; `delta` is the previous part's
    output in the engine dtype (or None).  A norm with `takes_unsummed` also accepts a
    `RoutedSum` as `delta`.
    """

    takes_unsummed = False

    def add_norm(self, h: torch.Tensor, delta: Optional[torch.Tensor],
                 out_dtype: torch.dtype) -> torch.Tensor:
        """h += delta (in place, in 32-bit); return norm(h) in `out_dtype`."""
        raise NotImplementedError

    def add_norm_rows(self, h: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                      out_dtype: torch.dtype) -> torch.Tensor:
        """norm(h[rows] + delta[rows]) without changing h."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions enter queries and keys."""

    def rotary_table(self, device: torch.device) -> Optional[Tuple[torch.Tensor, int]]:
        """(inverse frequencies float32 [rotary_dim // 2], rotary_dim) for the fused
        rotate-and-append kernel (half-split pairing), or None if the encoding is not of
        that form; then `apply` is called and the kernel appends without rotating."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encode in place: q [T, heads, D], k [T, kv_heads, D], positions int32 [T]."""
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here)."""

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheView],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        """x [T, hidden] in the engine dtype -> [T, hidden] in the engine dtype.

        `cache` is the view of the slot this call reads (and appends to when
        `cache.append`); `state` is the slab [slots, *state_spec.shape] indexed by
        `ctx.seg_slot`.
        """
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext):
        """x [T, hidden] -> [T, hidden], both in the engine dtype.  A routed feed-forward may
        return a `RoutedSum` instead of the tensor (see there); `summed()` turns either into
        the tensor."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of norms, mixer and feed-forward around the residual stream.

    The model asks the block, not the mixer, what the layer keeps between steps: pages
    (`cache_spec`) and a slab of fixed-size state per request (`state_spec`).  The usual block
    passes its mixer's answers on; an arrangement whose feed-forward (or the block itself)
    keeps state answers for it and hands `state` to whichever part it belongs to.
    """

    mixer: Mixer

    def cache_spec(self) -> Optional[CacheSpec]:
        return self.mixer.cache_spec()

    def state_spec(self) -> Optional[StateSpec]:
        return self.mixer.state_spec()

    def forward(self, h: torch.Tensor, pending, ctx: StepContext,
                cache: Optional[CacheView], state: Optional[torch.Tensor]):
        """Advance the float32 residual stream `h` in place.

        `pending` is a contribution not yet added to `h` (so that the sum fuses with the
        next norm): a tensor, a `RoutedSum` or None; the return value is this block's own
        pending contribution.
        """
        raise NotImplementedError
