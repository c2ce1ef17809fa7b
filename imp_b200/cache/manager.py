"""The cache manager: pages of keys and values with a block table per request,
one pool per group of layers with the same needs, and slots of fixed-size state.

What the reference has (src/memory/): one pool for all attention layers with a
LIFO free list that hands out page 0 first (kv_cache.cu:74-79, 97-116), a map
from sequence id to its page list with all-or-nothing allocation
(kv_cache_manager.cpp:37-69), `free_sequence` at the end of a request, and a
pool of fixed-size state indexed by `request id % max_sequences`
(ssm_state.h:16-49), which can collide.  What differs here:

* layers are grouped by what they need of the cache (all keys; a window of
  them; fixed-size state); each paged group has a pool and block tables of its
  own, shared by the layers of the group (one page id addresses the same slot
  in each of them);
* a windowed group gives a page back as soon as every later query is past it;
* state slots come from a free list, so two live requests never share one;
* nothing is evicted behind a request's back: `reserve` either gets all the
  pages or raises `OutOfPages` and leaves everything as it was; what to do then
  is the scheduler's decision.

The bookkeeping is host-only and needs no GPU; `allocate_storage` makes the
device tensors.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np


class OutOfPages(RuntimeError):
    """Not enough free pages (or state slots) for what was asked."""


class CacheError(RuntimeError):
    """Misuse of the cache manager (unknown request, double free, ...)."""


# ---------------------------------------------------------------------------
# What a mixer may ask of the cache
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values per token: [kv_heads, head_dim] each.  window == 0 keeps every token;
    window == W keeps what a query at position p may still see: positions > p - W."""

    num_kv_heads: int
    head_dim: int
    window: int = 0

    kind = "paged"


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per request: one tensor of `shape` per layer, zero at a request's start."""

    shape: Tuple[int, ...]
    dtype: str = "float32"

    kind = "state"


# ---------------------------------------------------------------------------
# Page pool
# ---------------------------------------------------------------------------
class PagePool:
    """Free list over `num_pages` page ids.  LIFO; page 0 comes out first."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("page pool is empty")
        p = self._free.pop()
        self._held[p] = True
        return p

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} is outside the pool of {self.num_pages}")
        if not self._held[page]:
            raise CacheError(f"page {page} freed twice")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]


class SlotPool(PagePool):
    """Free list over fixed-size state slots (same discipline as pages)."""


# ---------------------------------------------------------------------------
# Groups
# ---------------------------------------------------------------------------
class PagedGroup:
    """Layers that share page ids: same kv heads, head size and window.

    Block tables live in one int32 matrix [slots, max_pages_per_seq] (-1 = no page), so that a
    batch's table is one gather by slot.  Invariant: for a live request of committed length n, every
    entry in [first_live_page(n), n_entries) holds a page and every entry outside holds -1.
    """

    def __init__(self, gid: int, spec: PagedKVSpec, layers: List[int], page_size: int, num_pages: int,
                 num_slots: int, max_pages_per_seq: int):
        self.gid = gid
        self.spec = spec
        self.layers = layers
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.table_np = np.full((num_slots, max_pages_per_seq), -1, dtype=np.int32)
        self.n_entries = np.zeros(num_slots, dtype=np.int64)   # logical pages per slot (held or given back)
        self.slot_of: Dict[Hashable, int] = {}
        self.storage = None  # torch tensor [n_layers, 2, num_pages, kv_heads, page_size, head_dim]

    @property
    def tables(self) -> Dict[Hashable, "np.ndarray"]:
        """request -> its block table (a view: page id per logical page, -1 = already given back)."""
        return {rid: self.table_np[s, :self.n_entries[s]] for rid, s in self.slot_of.items()}

    def ensure_width(self, n_logical: int) -> None:
        """Widen the table matrix so that a row can hold `n_logical` logical pages."""
        width = self.table_np.shape[1]
        if n_logical > width:
            wider = np.full((self.table_np.shape[0], max(n_logical, 2 * width)), -1, dtype=np.int32)
            wider[:, :width] = self.table_np
            self.table_np = wider

    def table(self, rid: Hashable):
        s = self.slot_of[rid]
        return self.table_np[s, :self.n_entries[s]]

    def first_live_page(self, length: int) -> int:
        """Index of the first logical page a query at position >= `length` can still read."""
        if self.spec.window <= 0:
            return 0
        first_pos = max(0, length - self.spec.window + 1)
        return first_pos // self.page_size

    def pages_needed_n(self, n_entries: int, cur_len: int, new_len: int) -> int:
        """Pages to allocate for a request with `n_entries` logical pages to grow from cur_len to new_len."""
        n_logical = (new_len + self.page_size - 1) // self.page_size
        return max(0, n_logical - max(n_entries, self.first_live_page(cur_len)))

    def pages_needed(self, table, cur_len: int, new_len: int) -> int:
        return self.pages_needed_n(len(table), cur_len, new_len)


class StateGroup:
    """Layers with the same fixed-size state; slot ids are shared by all state groups."""

    def __init__(self, gid: int, spec: StateSpec, layers: List[int]):
        self.gid = gid
        self.spec = spec
        self.layers = layers
        self.storage = None  # torch tensor [n_layers, n_slots, *shape]


@dataclass
class LayerCacheRef:
    """Where a layer's cache lives: its group and its index inside the group's storage."""

    group: int
    index: int
    kind: str


class CacheManager:
    """Pages, block tables and state slots for all live requests.

    `layer_specs[i]` is what layer i asks for (a PagedKVSpec, a StateSpec or None).
    Layers that read another layer's cache are passed as None and resolved by the model.
    """

    def __init__(self, layer_specs: Sequence[Optional[object]], page_size: int, num_pages: int,
                 num_state_slots: int = 1, max_pages_per_seq: Optional[int] = None):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_pages_per_seq = max_pages_per_seq or num_pages
        n_slots = max(1, num_state_slots)
        self.paged: List[PagedGroup] = []
        self.state: List[StateGroup] = []
        self.layer_ref: List[Optional[LayerCacheRef]] = []
        by_spec: Dict[object, object] = {}
        for layer, spec in enumerate(layer_specs):
            if spec is None:
                self.layer_ref.append(None)
                continue
            grp = by_spec.get(spec)
            if grp is None:
                if isinstance(spec, PagedKVSpec):
                    grp = PagedGroup(len(self.paged), spec, [], page_size, num_pages, n_slots, self.max_pages_per_seq)
                    self.paged.append(grp)
                elif isinstance(spec, StateSpec):
                    grp = StateGroup(len(self.state), spec, [])
                    self.state.append(grp)
                else:
                    raise TypeError(f"layer {layer}: unknown cache spec {spec!r}")
                by_spec[spec] = grp
            grp.layers.append(layer)
            self.layer_ref.append(LayerCacheRef(grp.gid, len(grp.layers) - 1, spec.kind))
        self.slots = SlotPool(n_slots)
        self._slot_of: Dict[Hashable, int] = {}
        self._length: Dict[Hashable, int] = {}     # tokens committed per request
        self._reserved: Dict[Hashable, int] = {}   # tokens reserved (>= committed) per request

    # ------------------------------------------------------------------ requests
    def live_requests(self):
        return list(self._length)

    def has(self, rid: Hashable) -> bool:
        return rid in self._length

    def length(self, rid: Hashable) -> int:
        return self._length[rid]

    def add_request(self, rid: Hashable) -> int:
        """Register a request and give it a state slot.  Returns the slot."""
        if rid in self._length:
            raise CacheError(f"request {rid!r} is already live")
        try:
            slot = self.slots.alloc()
        except OutOfPages:
            raise OutOfPages("no free state slot") from None
        self._slot_of[rid] = slot
        self._length[rid] = 0
        self._reserved[rid] = 0
        for g in self.paged:
            g.slot_of[rid] = slot
            g.n_entries[slot] = 0
        return slot

    def slot_of(self, rid: Hashable) -> int:
        return self._slot_of[rid]

    def pages_needed(self, rid: Hashable, new_len: int) -> int:
        """Most pages any group lacks for `rid` to grow to `new_len` tokens."""
        cur = self._length[rid]
        slot = self._slot_of[rid]
        return max((g.pages_needed_n(int(g.n_entries[slot]), cur, new_len) for g in self.paged), default=0)

    def pages_for_new_request(self, n_tokens: int) -> int:
        """Pages per group that a fresh request needs for its first `n_tokens` tokens."""
        return (n_tokens + self.page_size - 1) // self.page_size if self.paged else 0

    def free_pages(self) -> int:
        """Free pages of the scarcest group."""
        return min((g.pool.n_free for g in self.paged), default=self.num_pages)

    def can_reserve(self, rid: Hashable, new_len: int) -> bool:
        cur = self._length[rid]
        slot = self._slot_of[rid]
        return all(g.pages_needed_n(int(g.n_entries[slot]), cur, new_len) <= g.pool.n_free for g in self.paged)

    def reserve(self, rid: Hashable, new_len: int) -> None:
        """Make sure every paged group has pages for positions < new_len that later queries can see.

        All or nothing: on `OutOfPages` nothing has changed.
        """
        if rid not in self._length:
            raise CacheError(f"unknown request {rid!r}")
        cur = self._length[rid]
        if new_len < cur:
            raise CacheError(f"request {rid!r}: cannot reserve {new_len} tokens below its length {cur}")
        slot = self._slot_of[rid]
        for g in self.paged:
            n_logical = (new_len + g.page_size - 1) // g.page_size
            g.ensure_width(n_logical)
            need = g.pages_needed_n(int(g.n_entries[slot]), cur, new_len)
            if need > g.pool.n_free:
                raise OutOfPages(f"group {g.gid}: request {rid!r} needs {need} more pages for {new_len} tokens, "
                                 f"{g.pool.n_free} free")
        for g in self.paged:
            n_logical = (new_len + g.page_size - 1) // g.page_size
            row = g.table_np[slot]
            for i in range(max(int(g.n_entries[slot]), g.first_live_page(cur)), n_logical):
                row[i] = g.pool.alloc()
            if n_logical > g.n_entries[slot]:
                g.n_entries[slot] = n_logical
        self._reserved[rid] = max(self._reserved[rid], new_len)

    def commit(self, rid: Hashable, new_len: int) -> List[Tuple[int, int]]:
        """Record that `rid` now holds `new_len` tokens; give back pages no later query can read.

        Returns the (group, page) pairs that were freed.
        """
        if new_len > self._reserved[rid]:
            raise CacheError(f"request {rid!r}: commit of {new_len} tokens beyond the reserved {self._reserved[rid]}")
        if new_len < self._length[rid]:
            raise CacheError(f"request {rid!r}: length cannot shrink from {self._length[rid]} to {new_len}")
        old_len = self._length[rid]
        self._length[rid] = new_len
        freed = []
        for g in self.paged:
            if g.spec.window <= 0:
                continue
            slot = self._slot_of[rid]
            row = g.table_np[slot]
            hi = min(g.first_live_page(new_len), int(g.n_entries[slot]))
            lo = g.first_live_page(old_len)
            for i in range(min(lo, hi), hi):
                if row[i] >= 0:
                    g.pool.free(int(row[i]))
                    freed.append((g.gid, int(row[i])))
                    row[i] = -1
        return freed

    def release(self, rid: Hashable) -> None:
        """Give back everything `rid` holds: pages of every group and its state slot."""
        if rid not in self._length:
            raise CacheError(f"release of unknown request {rid!r} (released twice?)")
        for g in self.paged:
            slot = g.slot_of.pop(rid)
            row = g.table_np[slot]
            for i in range(g.first_live_page(self._length[rid]), int(g.n_entries[slot])):
                if row[i] >= 0:
                    g.pool.free(int(row[i]))
            row[:int(g.n_entries[slot])] = -1
            g.n_entries[slot] = 0
        self.slots.free(self._slot_of.pop(rid))
        del self._length[rid]
        del self._reserved[rid]

    def block_table(self, group: int, rid: Hashable) -> List[int]:
        """The request's block table in `group` as a list (page id per logical page, -1 = given back)."""
        return [int(p) for p in self.paged[group].table(rid)]

    # ---------------------------------------------------------------- invariants
    def check_invariants(self) -> None:
        """No page lost, none held twice; raises AssertionError otherwise."""
        for g in self.paged:
            seen = set()
            for rid, table in g.tables.items():
                for p in table:
                    if p < 0:
                        continue
                    assert 0 <= p < g.pool.num_pages, f"group {g.gid}: page {p} out of range"
                    assert p not in seen, f"group {g.gid}: page {p} held twice"
                    assert g.pool.is_held(p), f"group {g.gid}: page {p} in a table but marked free"
                    seen.add(p)
            assert len(seen) + g.pool.n_free == g.pool.num_pages, \
                f"group {g.gid}: {g.pool.num_pages - len(seen) - g.pool.n_free} pages lost"
            assert len(set(g.pool._free)) == len(g.pool._free), f"group {g.gid}: a page is on the free list twice"
        slots = list(self._slot_of.values())
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert len(slots) + self.slots.n_free == self.slots.num_pages, "a state slot was lost"

    # ------------------------------------------------------------------- storage
    def allocate_storage(self, dtype, device) -> None:
        """Create the device tensors of every group (zero-filled, as the reference's pool: kv_cache.cu:53)."""
        import torch

        for g in self.paged:
            s = g.spec
            g.storage = torch.zeros((len(g.layers), 2, g.pool.num_pages, s.num_kv_heads, g.page_size, s.head_dim),
                                    dtype=dtype, device=device)
        for g in self.state:
            sdt = getattr(torch, g.spec.dtype)
            g.storage = torch.zeros((len(g.layers), self.slots.num_pages, *g.spec.shape), dtype=sdt, device=device)

    def storage_bytes(self, element_size: int) -> int:
        total = 0
        for g in self.paged:
            s = g.spec
            total += len(g.layers) * 2 * g.pool.num_pages * s.num_kv_heads * g.page_size * s.head_dim * element_size
        return total

    def layer_storage(self, layer: int):
        """(kind, tensor) of one layer: paged -> [2, pages, kv_heads, page_size, head_dim]; state -> [slots, *shape]."""
        ref = self.layer_ref[layer]
        if ref is None:
            return None, None
        grp = self.paged[ref.group] if ref.kind == "paged" else self.state[ref.group]
        return ref.kind, grp.storage[ref.index]

    def zero_state(self, slot: int) -> None:
        for g in self.state:
            if g.storage is not None:
                g.storage[:, slot].zero_()
