"""The cache manager: paged keys and values with a block table per request and per layer group,
and slots for per-request state of fixed size.

Layers that need the same kind of cache (all keys, or a window of them, with the same number of
key/value heads and head size) form a *group*. A group has pages of its own (one ``PagePool``),
and every request has one block table per group: position ``p`` of the request lives in page
``table[p // page_size]`` at row ``p % page_size`` in each layer of the group. Pages are given
back when a request is closed, when a reservation is rolled back, or, in a window group, when the
window has moved past them (their table entry becomes ``-1``); freed pages are handed out again.

Everything here is host bookkeeping; the device memory the ids refer to belongs to the engine.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from .pages import OutOfPages, PagePool


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer needs of the paged cache. ``window`` None keeps all keys; an integer w keeps
    only the keys of the last w positions (a query at p reads positions p-w+1 .. p)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    @property
    def group_key(self) -> Tuple:
        return ("window", self.window, self.num_kv_heads, self.head_dim) if self.window else \
               ("full", None, self.num_kv_heads, self.head_dim)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size that a mixer reads and rewrites each step."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass
class LayerGroup:
    index: int
    need: CacheNeed
    layers: List[int]
    pool: PagePool


class StateSlots:
    """Slot ids for fixed-size per-request state; slot 0 is handed out first, freed slots again."""

    def __init__(self, n_slots: int):
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._held = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free state slot")
        s = self._free.pop()
        self._held.add(s)
        return s

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise RuntimeError(f"StateSlots.release: slot {slot} is not allocated")
        self._held.remove(slot)
        self._free.append(slot)

    def check_invariants(self) -> None:
        assert len(set(self._free)) == len(self._free)
        assert not (self._held & set(self._free))
        assert len(self._held) + len(self._free) == self.n_slots


@dataclass
class PageCopy:
    """A page whose contents must be copied on the device (copy-on-write) before the next step."""
    group: int
    src: int
    dst: int


class RequestCache:
    """What one live request holds: a block table per group, its length and its state slot."""

    def __init__(self, key: Hashable, n_groups: int, max_pages: int, state_slot: int, fresh_state: bool):
        self.key = key
        self.length = 0                     # positions whose keys/values are in the cache
        self.reserved = 0                   # positions covered by pages (>= length)
        self.tables = [np.full(max_pages, -1, dtype=np.int32) for _ in range(n_groups)]
        self.n_pages = [0] * n_groups       # table entries in use (holes included)
        self.first_live = [0] * n_groups    # window groups: first table index still held
        self.state_slot = state_slot
        self.fresh_state = fresh_state      # True until the first step ran (state must start from zero)
        self.closed = False

    def n_pages_min(self) -> int:
        return min(self.n_pages) if self.n_pages else 1 << 30


class CacheManager:
    def __init__(self, needs: Dict[int, CacheNeed], page_size: int, pages_per_group: int,
                 max_position: int, max_requests: int, state_layers: Sequence[int] = ()):
        """``needs`` maps the index of each layer that owns pages to its need; ``state_layers`` are
        the layers that own a state slot (one slot id per request serves all of them)."""
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        self.page_size = page_size
        self.max_position = max_position
        self.max_pages_per_request = (max_position + page_size - 1) // page_size
        self.groups: List[LayerGroup] = []
        self.group_of_layer: Dict[int, int] = {}
        by_key: Dict[Tuple, LayerGroup] = {}
        for layer in sorted(needs):
            key = needs[layer].group_key
            if key not in by_key:
                by_key[key] = LayerGroup(len(self.groups), needs[layer], [], PagePool(pages_per_group))
                self.groups.append(by_key[key])
            by_key[key].layers.append(layer)
            self.group_of_layer[layer] = by_key[key].index
        self.state_layers = list(state_layers)
        self.slots = StateSlots(max_requests)
        self.max_requests = max_requests
        self.requests: Dict[Hashable, RequestCache] = {}

    # ------------------------------------------------------------------ requests
    def open(self, key: Hashable) -> RequestCache:
        if key in self.requests:
            raise KeyError(f"request {key!r} is already open")
        slot = self.slots.allocate()
        rc = RequestCache(key, len(self.groups), self.max_pages_per_request, slot, True)
        self.requests[key] = rc
        return rc

    def close(self, rc: RequestCache) -> None:
        """Gives back everything the request holds."""
        if rc.closed:
            raise RuntimeError(f"request {rc.key!r} was closed twice")
        for g, group in enumerate(self.groups):
            for i in range(rc.n_pages[g]):
                if rc.tables[g][i] >= 0:
                    group.pool.release(int(rc.tables[g][i]))
                    rc.tables[g][i] = -1
            rc.n_pages[g] = 0
        self.slots.release(rc.state_slot)
        rc.closed = True
        rc.length = rc.reserved = 0
        del self.requests[rc.key]

    # ------------------------------------------------------------------ pages
    def pages_needed(self, rc: RequestCache, n_new: int) -> int:
        """Pages a reservation of ``n_new`` more positions would take from the tightest group
        (copy-on-write pages included)."""
        worst = 0
        ps = self.page_size
        want = (rc.length + n_new + ps - 1) // ps
        for g, group in enumerate(self.groups):
            need = max(0, want - rc.n_pages[g])
            if n_new > 0:
                for i in range(rc.length // ps, min(rc.n_pages[g], want)):
                    p = int(rc.tables[g][i])
                    if p >= 0 and group.pool.ref_count(p) > 1:
                        need += 1
            worst = max(worst, need)
        return worst

    def free_pages(self) -> int:
        """Free pages of the tightest group."""
        return min((g.pool.free_count for g in self.groups), default=1 << 30)

    def reserve(self, rc: RequestCache, n_new: int) -> List[PageCopy]:
        """Makes positions ``length .. length+n_new-1`` writable in every group. All or nothing:
        on ``OutOfPages`` everything taken on the way is given back and nothing has changed.
        Returns the page copies (copy-on-write of shared pages) to perform before writing."""
        if rc.closed:
            raise RuntimeError("reserve on a closed request")
        if n_new < 0:
            raise ValueError("n_new must be >= 0")
        if rc.length + n_new > self.max_position:
            raise IndexError(f"position {rc.length + n_new - 1} is beyond the context length {self.max_position}")
        ps = self.page_size
        want = (rc.length + n_new + ps - 1) // ps
        taken: List[Tuple[int, int, int]] = []          # (group, table index, previous entry)
        copies: List[PageCopy] = []
        old_n = list(rc.n_pages)
        try:
            for g, group in enumerate(self.groups):
                table = rc.tables[g]
                if n_new > 0:                            # shared pages that will be written: copy first
                    for i in range(rc.length // ps, min(rc.n_pages[g], want)):
                        p = int(table[i])
                        if p >= 0 and group.pool.ref_count(p) > 1:
                            fresh = group.pool.allocate()
                            taken.append((g, i, p))
                            table[i] = fresh
                            copies.append(PageCopy(g, p, fresh))
                while rc.n_pages[g] < want:
                    fresh = group.pool.allocate()
                    i = rc.n_pages[g]
                    taken.append((g, i, -1))
                    table[i] = fresh
                    rc.n_pages[g] += 1
        except OutOfPages:
            for g, i, prev in reversed(taken):
                self.groups[g].pool.release(int(rc.tables[g][i]))
                rc.tables[g][i] = prev
            rc.n_pages = old_n
            raise
        for c in copies:                                 # the shared originals lose this request's reference
            self.groups[c.group].pool.release(c.src)
        rc.reserved = max(rc.reserved, rc.length + n_new)
        return copies

    def advance(self, rc: RequestCache, n_new: int) -> None:
        """The step that wrote ``n_new`` positions is done: the request is longer now, and window
        groups give back the pages that no later query can read."""
        if rc.length + n_new > rc.n_pages_min() * self.page_size:
            raise RuntimeError("advance beyond the reserved pages")
        rc.length += n_new
        rc.fresh_state = False
        ps = self.page_size
        for g, group in enumerate(self.groups):
            w = group.need.window
            if not w:
                continue
            first_needed = max(0, rc.length - w + 1)     # lowest position a query at >= length reads
            dead = first_needed // ps                    # pages wholly below it
            for i in range(rc.first_live[g], min(dead, rc.n_pages[g])):
                if rc.tables[g][i] >= 0:
                    group.pool.release(int(rc.tables[g][i]))
                    rc.tables[g][i] = -1
            rc.first_live[g] = max(rc.first_live[g], min(dead, rc.n_pages[g]))

    def rollback(self, rc: RequestCache) -> None:
        """Gives back pages reserved beyond the current length (a step that was not run)."""
        ps = self.page_size
        keep = (rc.length + ps - 1) // ps
        for g, group in enumerate(self.groups):
            while rc.n_pages[g] > keep:
                i = rc.n_pages[g] - 1
                if rc.tables[g][i] >= 0:
                    group.pool.release(int(rc.tables[g][i]))
                    rc.tables[g][i] = -1
                rc.n_pages[g] -= 1
        rc.reserved = rc.length

    def truncate(self, rc: RequestCache, length: int) -> None:
        """Rewinds a request to its first ``length`` positions (the reference's Sequence::truncate,
        src/model/kv_cache.cpp:96-104): pages wholly beyond them are given back, the rows of the last
        kept page beyond ``length`` are simply written again later. A window group cannot be rewound
        past positions whose pages it has already given back; per-request state cannot be rewound at
        all (it would have to be recomputed)."""
        if rc.closed or not (0 <= length <= rc.length):
            raise ValueError(f"truncate: {length} is outside the {rc.length} cached positions of {rc.key!r}")
        if length == rc.length:
            return
        if self.state_layers:
            raise RuntimeError("truncate: a request with per-request state cannot be rewound")
        ps = self.page_size
        for g, group in enumerate(self.groups):
            w = group.need.window
            if w and max(0, length - w + 1) // ps < rc.first_live[g]:
                raise RuntimeError(f"truncate: the window group has given back pages that position {length} would read")
        keep = (length + ps - 1) // ps
        for g, group in enumerate(self.groups):
            while rc.n_pages[g] > keep:
                i = rc.n_pages[g] - 1
                if rc.tables[g][i] >= 0:
                    group.pool.release(int(rc.tables[g][i]))
                    rc.tables[g][i] = -1
                rc.n_pages[g] -= 1
        rc.length = rc.reserved = length

    def adopt(self, rc: RequestCache, group: int, pages: Sequence[int]) -> None:
        """Starts an empty request on full pages that already hold its first positions (a prefix
        cache hit). The caller has retained each page for this request."""
        if rc.length != 0 or any(rc.n_pages):
            raise RuntimeError("adopt: the request is not empty")
        if len(self.groups) != 1 or self.groups[0].need.window or self.state_layers:
            raise RuntimeError("adopt: only models with one full-attention group and no state can share pages")
        for i, p in enumerate(pages):
            rc.tables[group][i] = p
        rc.n_pages[group] = len(pages)
        rc.length = rc.reserved = len(pages) * self.page_size
        rc.fresh_state = False

    def fork(self, src: RequestCache, key: Hashable, length: Optional[int] = None) -> RequestCache:
        """Opens a request that starts on the first ``length`` cached positions of ``src`` (all of
        them by default) and shares the pages that hold them (the reference pairs KvPool::retain
        with Sequence::adopt and truncate for this, tools/multiseq_check_main.cpp:279-286). Neither
        request sees what the other writes afterwards: ``reserve`` copies a shared page before a
        request writes into it (copy-on-write)."""
        if len(self.groups) != 1 or self.groups[0].need.window or self.state_layers:
            raise RuntimeError("fork: only models with one full-attention group and no state can share pages")
        n = src.length if length is None else int(length)
        if src.closed or not (0 < n <= src.length):
            raise ValueError(f"fork: length {n} is outside the {src.length} cached positions of {src.key!r}")
        rc = self.open(key)
        pages = (n + self.page_size - 1) // self.page_size
        pool = self.groups[0].pool
        for i in range(pages):
            p = int(src.tables[0][i])
            pool.retain(p)
            rc.tables[0][i] = p
        rc.n_pages[0] = pages
        rc.length = rc.reserved = n
        rc.fresh_state = False
        return rc

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost, none held by two tables without two references, none freed twice."""
        for g, group in enumerate(self.groups):
            group.pool.check_invariants()
            held: Dict[int, int] = {}
            for rc in self.requests.values():
                for i in range(rc.n_pages[g]):
                    p = int(rc.tables[g][i])
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            for p, n in held.items():
                assert group.pool.ref_count(p) >= n, f"group {g} page {p}: {n} holders, {group.pool.ref_count(p)} refs"
        self.slots.check_invariants()
        slots = [rc.state_slot for rc in self.requests.values()]
        assert len(slots) == len(set(slots)), "a state slot is held twice"

