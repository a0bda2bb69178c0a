"""Prefix cache: full pages of finished or running requests, found again by their tokens.

Semantics of the reference (src/model/prefix_cache.h:5-66, src/model/prefix_cache.cpp:7-122): only
full pages are indexed; a page is keyed by (page id of the page before it, its exact tokens), so a
match is a walk down a chain from the start of the prompt and no hashing can confuse two prefixes;
the cache holds one reference per indexed page; eviction takes the least recently used leaf that
nobody else references, and when every such page sits above a leaf still in use it forgets that
leaf (which frees nothing yet) to expose the page above it.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

from .pages import PagePool


class _Entry:
    __slots__ = ("parent", "tokens", "tick", "children")

    def __init__(self, parent: int, tokens: Tuple[int, ...], tick: int):
        self.parent, self.tokens, self.tick, self.children = parent, tokens, tick, 0


class PrefixCache:
    def __init__(self, pool: PagePool, page_size: int):
        self.pool = pool
        self.page_size = page_size
        self._index: Dict[Tuple[int, Tuple[int, ...]], int] = {}
        self._by_page: Dict[int, _Entry] = {}
        self._clock = 0

    @property
    def entries(self) -> int:
        return len(self._by_page)

    def match(self, tokens: Sequence[int], n: int) -> List[int]:
        """Pages holding the longest indexed prefix of ``tokens[:n]`` (whole pages only). Each
        returned page has been retained for the caller."""
        ps, parent, out = self.page_size, -1, []
        i = 0
        while (i + 1) * ps <= n:
            page = self._index.get((parent, tuple(tokens[i * ps:(i + 1) * ps])))
            if page is None:
                break
            self.pool.retain(page)
            self._clock += 1
            self._by_page[page].tick = self._clock
            out.append(page)
            parent = page
            i += 1
        return out

    def insert(self, tokens: Sequence[int], n_tokens: int, table: Sequence[int]) -> int:
        """Indexes the full pages of a request whose first ``n_tokens`` positions are cached."""
        ps, parent, added = self.page_size, -1, 0
        for i in range(min(n_tokens // ps, len(table))):
            key = (parent, tuple(tokens[i * ps:(i + 1) * ps]))
            known = self._index.get(key)
            self._clock += 1
            if known is not None:          # same contents already indexed (maybe under another page id)
                self._by_page[known].tick = self._clock
                parent = known
                continue
            page = int(table[i])
            if page < 0 or page in self._by_page:
                break
            self._by_page[page] = _Entry(parent, key[1], self._clock)
            if parent >= 0:
                self._by_page[parent].children += 1
            self.pool.retain(page)
            self._index[key] = page
            parent = page
            added += 1
        return added

    def _remove(self, page: int) -> None:
        e = self._by_page.pop(page)
        del self._index[(e.parent, e.tokens)]
        if e.parent >= 0:
            self._by_page[e.parent].children -= 1
        self.pool.release(page)

    def evict(self, count: int) -> int:
        """Frees up to ``count`` pages; returns how many were freed."""
        freed = 0
        while freed < count:
            victim: Optional[int] = None
            victim_frees = False
            for page, e in self._by_page.items():
                if e.children:
                    continue
                frees = self.pool.ref_count(page) == 1
                if not frees:
                    a, above = e.parent, False
                    while a >= 0:
                        above = above or self.pool.ref_count(a) == 1
                        a = self._by_page[a].parent
                    if not above:
                        continue
                better = victim is None or (frees and not victim_frees) or \
                    (frees == victim_frees and (e.tick, page) < (self._by_page[victim].tick, victim))
                if better:
                    victim, victim_frees = page, frees
            if victim is None:
                break
            self._remove(victim)
            if victim_frees:
                freed += 1
        return freed

    def evictable(self) -> int:
        return sum(1 for p in self._by_page if self.pool.ref_count(p) == 1)

    def clear(self) -> None:
        for page in list(self._by_page):
            self.pool.release(page)
        self._by_page.clear()
        self._index.clear()
