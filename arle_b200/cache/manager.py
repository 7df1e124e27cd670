"""The cache manager: paged keys and values, block tables, and state slots.

Layers are sorted into *groups* by what their mixer needs (number of kv heads,
head size, and whether all keys are kept or only a window).  Each group has its
own pages, its own allocator and its own block table per request, because a
window group gives pages back while the request lives and a full group does not.
cklxx/arle has one group: one table per slot shared by all KV layers
(crates/cuda-kernels/src/paged_kv.rs:63-70; infer/src/scheduler/cuda/core/construction.rs:194-202).

Page layout inside a group: one array per stream of the group's need (keys and
values for attention), each ``[layer, page, head, slot_in_page, width]``, the
reference's head-major page (paged_kv.rs:330-355).  A mixer with another per-token
record (one compressed vector, keys and values of different widths) names its
streams in its ``CacheNeed`` and gets arrays of those shapes under the same tables.

A request holds one *slot* for its life.  The slot indexes the host-side block
tables and the per-request state arrays that mixers may ask for (``StateNeed``);
those are zeroed when the slot is handed out.  Attention needs no such state, so
for Qwen3 the arrays are empty, but the slots are handed out and returned all the
same.

Growth is atomic over a whole step: ``append`` first counts the pages every
group needs for every request of the step and raises ``OutOfPages`` with nothing
changed if any group falls short.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheNeed, StateNeed
from .pages import OutOfPages, PagePool


class NoFreeSlot(RuntimeError):
    pass


@dataclass
class LayerCacheView:
    """What a mixer sees of its cache layer during one step."""

    streams: List[torch.Tensor]     # one [pages, heads, page_size, width] per stream of the mixer's CacheNeed
    page_size: int
    block_table: torch.Tensor       # int32 [rows of the step, max pages]; -1 where a window has passed
    slot_mapping: torch.Tensor      # int32 [tokens of the step]: page * page_size + slot_in_page
    writable: bool = True

    @property
    def k(self) -> torch.Tensor:    # attention's names for its two streams
        return self.streams[0]

    @property
    def v(self) -> torch.Tensor:
        return self.streams[1]


class CacheGroup:
    def __init__(self, need: CacheNeed, layers: List[int], page_size: int, num_pages: int, max_slots: int,
                 max_pages_per_request: int, dtype: torch.dtype, device):
        self.need = need
        self.layers = layers                      # cache-layer ids served by this group
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.arrays = [torch.zeros((len(layers), num_pages, heads, page_size, width), dtype=dtype, device=device)
                       for heads, width in need.arrays()]
        # host block tables, one row per slot; logical page -> physical page, -1 = not held
        self.table = np.full((max_slots, max_pages_per_request), -1, dtype=np.int32)
        self.first_held = np.zeros(max_slots, dtype=np.int64)     # first logical page still held
        self.num_logical = np.zeros(max_slots, dtype=np.int64)    # logical pages ever given to the slot

    def pages_for(self, slot: int, old_tokens: int, new_tokens: int) -> int:
        return max(0, -(-new_tokens // self.page_size) - int(self.num_logical[slot]))

    def bytes_per_page(self) -> int:
        return len(self.layers) * self.need.elements_per_token() * self.page_size * self.arrays[0].element_size()


class CacheManager:
    def __init__(self, cache_needs: Sequence[CacheNeed], state_needs: Sequence[StateNeed], page_size: int,
                 num_pages: int, max_slots: int, max_tokens_per_request: int, dtype: torch.dtype, device="cuda"):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_tokens_per_request = max_tokens_per_request
        self.device = torch.device(device)
        max_pages = -(-max_tokens_per_request // page_size)
        self.max_pages_per_request = max_pages          # columns of every host block table
        by_key: Dict[tuple, List[int]] = {}
        for layer, need in enumerate(cache_needs):
            by_key.setdefault(need.group_key(), []).append(layer)
        self.groups: List[CacheGroup] = []
        self.layer_to_group: Dict[int, Tuple[int, int]] = {}
        for key, layers in by_key.items():
            g = CacheGroup(cache_needs[layers[0]], layers, page_size, num_pages, max_slots, max_pages, dtype, self.device)
            for j, layer in enumerate(layers):
                self.layer_to_group[layer] = (len(self.groups), j)
            self.groups.append(g)
        self.states = [torch.zeros((max_slots, *n.shape), dtype=n.dtype, device=self.device) for n in state_needs]
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._slot_of: Dict[object, int] = {}
        self._tokens: Dict[object, int] = {}

    # --------------------------------------------------------------- requests
    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def has_request(self, rid) -> bool:
        return rid in self._slot_of

    def live_requests(self):
        return list(self._slot_of)

    def add_request(self, rid) -> int:
        if rid in self._slot_of:
            raise ValueError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.max_slots} request slots are in use")
        slot = self._free_slots.pop()
        self._slot_of[rid] = slot
        self._tokens[rid] = 0
        for s in self.states:
            s[slot].zero_()
        return slot

    def slot(self, rid) -> int:
        return self._slot_of[rid]

    def num_tokens(self, rid) -> int:
        return self._tokens[rid]

    def free_request(self, rid) -> None:
        slot = self._slot_of.pop(rid)
        del self._tokens[rid]
        for g in self.groups:
            lo, hi = int(g.first_held[slot]), int(g.num_logical[slot])
            g.pool.free(int(p) for p in g.table[slot, lo:hi])
            g.table[slot, :hi] = -1
            g.first_held[slot] = 0
            g.num_logical[slot] = 0
        self._free_slots.append(slot)

    # ----------------------------------------------------------------- growth
    def pages_needed(self, rid, n_new: int) -> List[int]:
        """Pages each group would have to allocate to take n_new more tokens of rid."""
        slot, old = self._slot_of[rid], self._tokens[rid]
        return [g.pages_for(slot, old, old + n_new) for g in self.groups]

    def pages_for_new_request(self, n_tokens: int) -> List[int]:
        return [-(-n_tokens // self.page_size) for _ in self.groups]

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def total_pages(self) -> List[int]:
        return [g.pool.num_pages for g in self.groups]

    def can_append(self, items: Sequence[Tuple[object, int]]) -> bool:
        need = [0] * len(self.groups)
        for rid, n in items:
            for gi, p in enumerate(self.pages_needed(rid, n)):
                need[gi] += p
        return all(n <= g.pool.num_free for n, g in zip(need, self.groups))

    def append(self, items: Sequence[Tuple[object, int]]) -> None:
        """Give every (request, n_new_tokens) of a step room for its tokens, or raise
        OutOfPages / ValueError with nothing changed."""
        need = [0] * len(self.groups)
        seen = set()
        for rid, n in items:
            if rid in seen:
                raise ValueError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            if n <= 0:
                raise ValueError("a step entry needs at least one token")
            if self._tokens[rid] + n > self.max_tokens_per_request:
                raise ValueError(f"request {rid!r} would hold {self._tokens[rid] + n} tokens, "
                                 f"more than the {self.max_tokens_per_request} a request may hold")
            for gi, p in enumerate(self.pages_needed(rid, n)):
                need[gi] += p
        for gi, g in enumerate(self.groups):
            if need[gi] > g.pool.num_free:
                raise OutOfPages(need[gi], g.pool.num_free, f"pages of cache group {gi}")
        for rid, n in items:
            slot = self._slot_of[rid]
            new_total = self._tokens[rid] + n
            for g in self.groups:
                k = g.pages_for(slot, self._tokens[rid], new_total)
                if k:
                    at = int(g.num_logical[slot])
                    g.table[slot, at:at + k] = g.pool.alloc(k)
                    g.num_logical[slot] = at + k
            self._tokens[rid] = new_total

    def release_passed(self, rid) -> int:
        """Give back the pages of window groups that no later query of rid can see:
        a query at position p >= tokens sees keys >= p - window + 1, so a page whose
        last token lies before tokens - window + 1 is done.  Returns pages freed."""
        slot, n = self._slot_of[rid], self._tokens[rid]
        freed = 0
        for g in self.groups:
            w = g.need.window
            if w is None:
                continue
            first_needed_token = max(0, n - w + 1)
            upto = min(first_needed_token // g.page_size, int(g.num_logical[slot]))
            lo = int(g.first_held[slot])
            if upto > lo:
                g.pool.free(int(p) for p in g.table[slot, lo:upto])
                g.table[slot, lo:upto] = -1
                g.first_held[slot] = upto
                freed += upto - lo
        return freed

    def truncate(self, rid, n_tokens: int) -> None:
        """Forget the tokens of rid beyond n_tokens (pages wholly beyond go back).
        Used when a step fails after its pages were reserved."""
        slot = self._slot_of[rid]
        if n_tokens > self._tokens[rid]:
            raise ValueError("truncate cannot grow a request")
        for g in self.groups:
            keep = max(-(-n_tokens // g.page_size), int(g.first_held[slot]))
            hi = int(g.num_logical[slot])
            if hi > keep:
                g.pool.free(int(p) for p in g.table[slot, keep:hi])
                g.table[slot, keep:hi] = -1
                g.num_logical[slot] = keep
        self._tokens[rid] = n_tokens

    # ------------------------------------------------------------ step tables
    def slot_mapping(self, group: int, rid, start: int, n: int) -> np.ndarray:
        """Physical token slots (page * page_size + offset) of tokens start..start+n-1."""
        g = self.groups[group]
        pos = np.arange(start, start + n, dtype=np.int64)
        pages = g.table[self._slot_of[rid], pos // g.page_size].astype(np.int64)
        if (pages < 0).any():
            raise RuntimeError(f"request {rid!r}: a token of this step has no page in group {group}")
        return (pages * g.page_size + pos % g.page_size).astype(np.int32)

    def block_rows(self, group: int, rids: Sequence[object], width: Optional[int] = None) -> np.ndarray:
        g = self.groups[group]
        slots = [self._slot_of[r] for r in rids]
        if width is None:
            width = max(1, int(max(g.num_logical[s] for s in slots))) if slots else 1
        return g.table[slots, :width]

    def layer_view(self, cache_layer: int, block_table: torch.Tensor, slot_mapping: torch.Tensor,
                   writable: bool) -> LayerCacheView:
        gi, j = self.layer_to_group[cache_layer]
        g = self.groups[gi]
        return LayerCacheView([a[j] for a in g.arrays], g.page_size, block_table, slot_mapping, writable)

    def group_of_layer(self, cache_layer: int) -> int:
        return self.layer_to_group[cache_layer][0]

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_page() for g in self.groups) // self.page_size

    # ------------------------------------------------------------- invariants
    def check(self) -> None:
        """No page lost, none held twice: the held pages of every group are exactly
        the entries of the live requests' tables."""
        live_slots = set(self._slot_of.values())
        if len(live_slots) != len(self._slot_of) or live_slots & set(self._free_slots):
            raise AssertionError("slot bookkeeping is inconsistent")
        if len(live_slots) + len(self._free_slots) != self.max_slots:
            raise AssertionError("a slot is lost")
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = []
            for s in range(self.max_slots):
                row = g.table[s]
                live = row[row >= 0]
                if s not in live_slots and live.size:
                    raise AssertionError(f"group {gi}: free slot {s} still lists pages")
                held.extend(int(p) for p in live)
                lo, hi = int(g.first_held[s]), int(g.num_logical[s])
                if (row[lo:hi] < 0).any() or (row[:lo] >= 0).any() or (row[hi:] >= 0).any():
                    raise AssertionError(f"group {gi}: slot {s} table does not match its bounds")
            if len(held) != len(set(held)):
                raise AssertionError(f"group {gi}: a page is held twice")
            if len(held) + g.pool.num_free != g.pool.num_pages:
                raise AssertionError(f"group {gi}: {g.pool.num_pages - len(held) - g.pool.num_free} page(s) lost")
