"""The cache manager: paged keys and values per layer group, block tables per request,
and slots of fixed-size per-request state.

Layers whose mixers need the same kind of cache (all keys; a window of them) with the
same geometry form a *group*.  Each group has its own page pool, its own device tensor
``[layers_in_group, num_pages + 1, *page shape]`` (the page shape is the spec's: keys and values
``[2, kv_heads, page_size, head_dim]``, or rows of any width) and its own block table per request.  Page ``num_pages`` of every group is a null page that padding rows of
a replayed graph write to; it is never handed out.

A request's pages are given back when it is closed; in a window group, also as soon as
every position in a page lies before the window of all positions still to come.
Beside the pages, every live request holds one *state slot*: an index into per-layer
slabs ``[num_slots, *shape]`` for mixers that keep state of fixed size.  This
architecture has none; the slots exist so that adding such a mixer changes no engine code.

Reference counterpart: ``KVCache`` (src/runtime/kv_cache.h:13-62, kv_cache.cpp:10-52) and
the session struct ``{slot, length}`` (src/api/ninfer_c_api.cpp:28-32).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheSpec, CacheView, StateSpec
from .page_pool import OutOfPages, PagePool


class OutOfSlots(RuntimeError):
    pass


@dataclass
class CacheGroup:
    index: int
    spec: CacheSpec
    slots: List[int]                       # cache slots (layer indices) in this group
    pool: PagePool
    pages: Optional[torch.Tensor] = None   # device tensor, see module docstring

    @property
    def null_page(self) -> int:
        return self.pool.num_pages


@dataclass
class RequestEntry:
    slot: int
    length: int = 0                        # tokens committed
    reserved: int = 0                      # tokens for which pages are held
    # per group: logical page index -> physical page (-1 once released or never held)
    tables: List[List[int]] = field(default_factory=list)


class CacheManager:
    def __init__(self, cache_specs: Sequence[Optional[CacheSpec]],
                 state_specs: Sequence[Optional[StateSpec]], *, page_size: int, num_pages: int,
                 max_requests: int, max_context: int, dtype: torch.dtype = torch.float32,
                 device="cpu", allocate: bool = True, clear_reused_pages: bool = True):
        self.page_size, self.max_requests = int(page_size), int(max_requests)
        self.max_context = int(max_context)
        self.clear_reused_pages = bool(clear_reused_pages)
        self.pages_cleared = 0
        self.max_pages_per_request = (self.max_context + self.page_size - 1) // self.page_size
        self.dtype, self.device = dtype, torch.device(device)
        self.groups: List[CacheGroup] = []
        self.group_of_slot: Dict[int, Tuple[int, int]] = {}   # cache slot -> (group, index in group)
        by_key: Dict[Tuple, CacheGroup] = {}
        for slot, spec in enumerate(cache_specs):
            if spec is None:
                continue
            key = spec.group_key()
            if key not in by_key:
                g = CacheGroup(len(self.groups), spec, [], PagePool(num_pages))
                by_key[key] = g
                self.groups.append(g)
            g = by_key[key]
            self.group_of_slot[slot] = (g.index, len(g.slots))
            g.slots.append(slot)
        if allocate:
            for g in self.groups:
                g.pages = torch.zeros((len(g.slots), num_pages + 1, *g.spec.page_shape(self.page_size)),
                                      dtype=dtype, device=self.device)
        # state slots
        self._free_slots = list(range(self.max_requests - 1, -1, -1))
        self.state_specs = list(state_specs)
        self.state: Dict[int, torch.Tensor] = {}
        if allocate:
            for layer, sp in enumerate(self.state_specs):
                if sp is not None:
                    # one slot more than requests: padding rows of a replayed graph use the last
                    self.state[layer] = torch.zeros((self.max_requests + 1, *sp.shape), dtype=sp.dtype,
                                                    device=self.device)
        self.requests: Dict[Hashable, RequestEntry] = {}

    @property
    def null_slot(self) -> int:
        return self.max_requests

    # ---- sizes ---------------------------------------------------------------------
    def bytes_per_token(self) -> int:
        """Cache bytes one token occupies across all layers (window groups included)."""
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.slots) * g.spec.elements_per_token() * el for g in self.groups)

    def total_bytes(self) -> int:
        return sum(g.pages.numel() * g.pages.element_size() for g in self.groups if g.pages is not None)

    def pages_free(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    # ---- requests ------------------------------------------------------------------
    def open(self, req: Hashable) -> int:
        """Admit a request: one state slot (zeroed), no pages yet.  Returns the slot."""
        if req in self.requests:
            raise KeyError(f"request {req!r} is already open")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        for slab in self.state.values():
            slab[slot].zero_()
        self.requests[req] = RequestEntry(slot, tables=[[] for _ in self.groups])
        return slot

    def close(self, req: Hashable) -> None:
        """Give back everything the request holds."""
        ent = self.requests.pop(req)
        for g, table in zip(self.groups, ent.tables):
            g.pool.give_back([p for p in table if p >= 0])
        self._free_slots.append(ent.slot)

    def is_open(self, req: Hashable) -> bool:
        return req in self.requests

    def length(self, req: Hashable) -> int:
        return self.requests[req].length

    def slot(self, req: Hashable) -> int:
        return self.requests[req].slot

    # ---- pages ---------------------------------------------------------------------
    def _pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def _first_live_page(self, g: CacheGroup, length: int) -> int:
        """First logical page that positions >= `length` can still read."""
        if g.spec.kind != "window":
            return 0
        first_key = max(0, length - int(g.spec.window) + 1)
        return first_key // self.page_size

    def pages_needed(self, req: Hashable, new_length: int) -> List[int]:
        """Per group, pages that `reserve(req, new_length)` would take."""
        ent = self.requests[req]
        need_to = self._pages_for(new_length)
        out = []
        for g, table in zip(self.groups, ent.tables):
            out.append(max(0, need_to - len(table)))
        return out

    def can_reserve(self, req: Hashable, new_length: int) -> bool:
        if new_length > self.max_context:
            return False
        return all(n <= g.pool.num_free for n, g in zip(self.pages_needed(req, new_length), self.groups))

    def reserve(self, req: Hashable, new_length: int) -> None:
        """Hold pages for positions < new_length in every group, or change nothing."""
        ent = self.requests[req]
        if new_length > self.max_context:
            raise OutOfPages(f"request {req!r}: {new_length} tokens exceed max_context={self.max_context}")
        need = self.pages_needed(req, new_length)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"request {req!r}: group {g.index} needs {n} pages, "
                                 f"{g.pool.num_free} free")
        for n, g, table in zip(need, self.groups, ent.tables):
            first_new = len(table)
            taken, again = g.pool.take_marking_reuse(n)
            table.extend(taken)
            if not (again and self.clear_reused_pages and g.pages is not None):
                continue
            # A page that is handed out again still holds its earlier owner's entries.  Kernels
            # that copy whole pages multiply what lies beyond the new owner's position by a zero
            # probability, which keeps a result right only while those entries are finite; zeros
            # are.  Pages that this reservation covers to their last row are overwritten by the
            # step before anything reads them; the one it covers in part is zeroed here - on the
            # stream, so after whatever still reads it for its earlier owner (a step launched ahead).
            for i, p in enumerate(taken):
                covered_to = (first_new + i + 1) * self.page_size
                if covered_to > new_length and p in again:
                    g.pages[:, p].zero_()
                    self.pages_cleared += 1
        ent.reserved = max(ent.reserved, new_length)

    def commit(self, req: Hashable, new_length: int) -> None:
        """The step wrote positions < new_length; release what a window has passed."""
        ent = self.requests[req]
        if new_length > ent.reserved:
            raise AssertionError(f"commit to {new_length} beyond the reserved {ent.reserved}")
        ent.length = new_length
        for g, table in zip(self.groups, ent.tables):
            first = self._first_live_page(g, new_length)
            dead = [i for i in range(min(first, len(table))) if table[i] >= 0]
            if dead:
                g.pool.give_back([table[i] for i in dead])
                for i in dead:
                    table[i] = -1

    def truncate(self, req: Hashable) -> None:
        """Drop a reservation that was never committed (a step that did not run)."""
        ent = self.requests[req]
        keep = self._pages_for(ent.length)
        for g, table in zip(self.groups, ent.tables):
            extra = [p for p in table[keep:] if p >= 0]
            g.pool.give_back(extra)
            del table[keep:]
        ent.reserved = ent.length

    def block_table(self, group: int, req: Hashable) -> List[int]:
        return self.requests[req].tables[group]

    # ---- what a mixer call sees ------------------------------------------------------
    def view(self, cache_slot: int, block_tables: Dict[int, torch.Tensor], append: bool
             ) -> Optional[CacheView]:
        if cache_slot not in self.group_of_slot:
            return None
        gi, li = self.group_of_slot[cache_slot]
        g = self.groups[gi]
        return CacheView(g.spec, g.pages[li], block_tables[gi], self.page_size, append)

    def state_of(self, layer: int) -> Optional[torch.Tensor]:
        return self.state.get(layer)

    # ---- invariants (used by tests) ----------------------------------------------------
    def check(self) -> None:
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen = {}
            for req, ent in self.requests.items():
                for p in ent.tables[gi]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise AssertionError(f"page {p} of group {gi} held by {seen[p]!r} and {req!r}")
                    seen[p] = req
            if len(seen) != g.pool.num_held:
                raise AssertionError(f"group {gi}: {g.pool.num_held} pages held, "
                                     f"{len(seen)} found in block tables (a page was lost)")
        slots = [e.slot for e in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a state slot is held twice or is both held and free")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise AssertionError("a state slot was lost")
