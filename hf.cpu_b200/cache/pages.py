"""Paged key/value cache: page pools, block tables, groups of layers, and the manager.

The reference keeps one malloc per (layer, 64-token block) and a pointer table per context
(src/model.c:195-213, :244-247), grows it lazily before compute with rollback on failure
(src/model.c:309-330), and frees only with the context (src/model.c:217-230).  Here a *page id*
addresses the same slot in every layer of a *group*; groups exist because layers may need
different things of the cache (all keys, or a window of them), and each group has its own pool
and its own block table per request.  Pages go back to the pool when a request ends and, in a
windowed group, as soon as the window has passed them; the pool hands them out again.

A request may start on the full pages of another whose first tokens are the same (``fork``): the reference
shares full blocks read-only between a context and its forks and copies the partial one (src/model.c:268-301),
for the continuations of one prompt (src/ops.c:808-825) and for a prompt that begins like the previous one
(src/ops.c:771-776).  Here a shared page is held once per block table that maps it (the pool counts the holders),
nobody writes to it again because every holder only appends behind it, and the partial block is not copied but
computed again by the new request, which has to run its last prompt token in any case.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheSpec


class OutOfPages(RuntimeError):
    """The pool of some group cannot supply the pages a reservation needs; nothing was changed."""


class PagePool:
    """A stack of free page ids with a reference count per page."""

    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))     # pop() hands out 0 first
        self._ref = [0] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("page pool is empty")
        p = self._free.pop()
        assert self._ref[p] == 0
        self._ref[p] = 1
        return p

    def share(self, page: int) -> None:
        if self._ref[page] < 1:
            raise ValueError(f"page {page} is not held")
        self._ref[page] += 1

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages or self._ref[page] < 1:
            raise ValueError(f"page {page} is freed but not held")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return self._ref[page]

    def check(self) -> None:
        """Every page is either free exactly once or held: none lost, none free twice."""
        free = sorted(self._free)
        assert len(set(free)) == len(free), "a page is on the free list twice"
        for p in range(self.num_pages):
            assert (self._ref[p] == 0) == (p in set(free)), f"page {p}: refcount {self._ref[p]} vs free list"


@dataclass
class LayerCache:
    """One schedule entry's keys and values: ``[num_pages, block_size, kv_heads, head_dim]`` each."""
    group: int
    k: torch.Tensor
    v: torch.Tensor


class CacheGroup:
    """Schedule entries with the same needs share page geometry, a pool and block tables."""

    def __init__(self, index: int, spec: CacheSpec, entries: Sequence[int], num_pages: int, block_size: int,
                 dtype: torch.dtype, device: torch.device):
        self.index, self.spec, self.entries = index, spec, list(entries)
        self.block_size, self.num_pages = block_size, num_pages
        self.pool = PagePool(num_pages)
        self.storage = torch.zeros((len(self.entries), 2, num_pages, block_size, spec.num_kv_heads, spec.head_dim),
                                   dtype=dtype, device=device)
        self.tables: Dict[object, List[int]] = {}       # request -> page id per block, -1 = not mapped
        self.np_tables: Dict[object, np.ndarray] = {}   # the same at full width as int32, ready to be copied to the device

    @property
    def page_bytes(self) -> int:
        return (len(self.entries) * 2 * self.block_size * self.spec.num_kv_heads * self.spec.head_dim
                * self.storage.element_size())

    def layer_cache(self, entry: int) -> LayerCache:
        i = self.entries.index(entry)
        return LayerCache(self.index, self.storage[i, 0], self.storage[i, 1])

    def first_needed_block(self, next_pos: int) -> int:
        """Blocks before this one hold no key that a query at ``next_pos`` or later can see."""
        if self.spec.window <= 0:
            return 0
        return max(0, next_pos - self.spec.window + 1) // self.block_size

    def blocks_to_map(self, table: List[int], old_len: int, new_len: int) -> List[int]:
        """Block indices that must be mapped so positions ``old_len .. new_len-1`` can be written
        and every query among them sees its keys."""
        last = (new_len - 1) // self.block_size
        first = self.first_needed_block(old_len)
        # Blocks below len(table) are mapped unless a window has passed them, and those lie before `first`
        # (advance() released them; a step that failed after its reservation leaves its blocks mapped):
        # only blocks beyond the table are new.
        start = max(first, len(table))
        return list(range(start, last + 1))


class KVCacheManager:
    """Owns every group's pool and every request's block tables."""

    def __init__(self, entry_specs: Dict[int, CacheSpec], block_size: int, num_pages: int,
                 dtype: torch.dtype, device: torch.device, max_blocks_per_request: int):
        if block_size < 1:
            raise ValueError("block_size must be at least 1")
        self.block_size, self.max_blocks = block_size, max_blocks_per_request
        by_spec: Dict[CacheSpec, List[int]] = {}
        for entry, spec in sorted(entry_specs.items()):
            by_spec.setdefault(spec, []).append(entry)
        self.groups: List[CacheGroup] = [
            CacheGroup(i, spec, entries, num_pages, block_size, dtype, device)
            for i, (spec, entries) in enumerate(by_spec.items())]
        self._entry_cache: Dict[int, LayerCache] = {}
        for g in self.groups:
            for e in g.entries:
                self._entry_cache[e] = g.layer_cache(e)
        self.lengths: Dict[object, int] = {}

    # ---- queries --------------------------------------------------------------------------
    def entry_cache(self, entry: int) -> Optional[LayerCache]:
        return self._entry_cache.get(entry)

    def length(self, req) -> int:
        return self.lengths[req]

    def table(self, group: int, req) -> List[int]:
        return self.groups[group].tables[req]

    def pages_in_use(self) -> int:
        return sum(g.pool.used_count for g in self.groups)

    def bytes_in_use(self) -> int:
        return sum(g.pool.used_count * g.page_bytes for g in self.groups)

    def free_pages(self) -> List[int]:
        return [g.pool.free_count for g in self.groups]

    # ---- life cycle -------------------------------------------------------------------------
    def add(self, req) -> None:
        if req in self.lengths:
            raise ValueError(f"request {req!r} is already live")
        self.lengths[req] = 0
        for g in self.groups:
            g.tables[req] = []
            g.np_tables[req] = np.full(self.max_blocks, -1, dtype=np.int32)

    def pages_needed(self, req, new_len: int) -> List[int]:
        """Pages each group would have to map for ``req`` to hold ``new_len`` tokens; a request that is
        not live yet counts from nothing."""
        old = self.lengths.get(req, 0)
        return [len(g.blocks_to_map(g.tables.get(req, []), old, new_len)) for g in self.groups]

    def can_reserve(self, wants: Sequence[Tuple[object, int]]) -> bool:
        """Would reserving ``new_len`` tokens for each ``(request, new_len)`` fit, all together?"""
        need = [0] * len(self.groups)
        for req, new_len in wants:
            for i, n in enumerate(self.pages_needed(req, new_len)):
                need[i] += n
        return all(n <= g.pool.free_count for n, g in zip(need, self.groups))

    def reserve(self, req, new_len: int) -> None:
        """Map pages so that positions ``length(req) .. new_len-1`` can be written; all groups or none."""
        old = self.lengths[req]
        if new_len < old:
            raise ValueError("a reservation cannot shrink a request")
        if (new_len + self.block_size - 1) // self.block_size > self.max_blocks:
            raise OutOfPages(f"request {req!r} would hold {new_len} tokens, more than the context limit "
                             f"of {self.max_blocks * self.block_size}")
        plan = [g.blocks_to_map(g.tables[req], old, new_len) for g in self.groups]
        for g, blocks in zip(self.groups, plan):
            if len(blocks) > g.pool.free_count:
                raise OutOfPages(f"cache group {g.index} needs {len(blocks)} pages for request {req!r}, "
                                 f"{g.pool.free_count} are free")
        for g, blocks in zip(self.groups, plan):
            t = g.tables[req]
            for b in blocks:
                while len(t) <= b:
                    t.append(-1)
                t[b] = g.pool.alloc()
                g.np_tables[req][b] = t[b]

    def fork(self, src, dst, n_tokens: int) -> int:
        """``dst`` (live, holding nothing yet) starts on the pages of ``src``'s first tokens: as many full blocks of
        the first ``n_tokens`` as ``src`` has computed and, in a windowed group, still holds where a query behind
        them would look.  Returns how many tokens ``dst`` now holds (a multiple of the block size, maybe 0)."""
        if self.lengths[dst] != 0 or any(g.tables[dst] for g in self.groups):
            raise ValueError(f"request {dst!r} already holds pages")
        if src == dst:
            raise ValueError("a request cannot start on its own pages")
        n = min(int(n_tokens), self.lengths[src]) // self.block_size * self.block_size
        nb = n // self.block_size
        if nb == 0:
            return 0
        for g in self.groups:
            t = g.tables[src]
            if len(t) < nb or any(t[b] < 0 for b in range(g.first_needed_block(n), nb)):
                return 0                   # a window has passed pages of src that a query at position n still sees
        for g in self.groups:
            ts, td, first = g.tables[src], g.tables[dst], g.first_needed_block(n)
            for b in range(nb):
                page = ts[b] if b >= first else -1
                td.append(page)
                if page >= 0:
                    g.pool.share(page)
                    g.np_tables[dst][b] = page
        self.lengths[dst] = n
        return n

    def advance(self, req, new_len: int) -> None:
        """The request now holds ``new_len`` tokens; pages a window has passed go back to the pool."""
        self.lengths[req] = new_len
        for g in self.groups:
            t = g.tables[req]
            for b in range(min(g.first_needed_block(new_len), len(t))):
                if t[b] >= 0:
                    g.pool.free(t[b])
                    t[b] = -1
                    g.np_tables[req][b] = -1

    def release(self, req) -> None:
        """The request ends: every page it holds in every group goes back."""
        for g in self.groups:
            for p in g.tables.pop(req):
                if p >= 0:
                    g.pool.free(p)
            del g.np_tables[req]
        del self.lengths[req]

    def check(self) -> None:
        """No page lost, held twice or freed twice."""
        for g in self.groups:
            g.pool.check()
            holders: Dict[int, int] = {}
            for t in g.tables.values():
                pages = [p for p in t if p >= 0]
                assert len(pages) == len(set(pages)), f"group {g.index}: a page is in one block table twice"
                for p in pages:
                    holders[p] = holders.get(p, 0) + 1
            assert len(holders) == g.pool.used_count, \
                f"group {g.index}: {g.pool.used_count} pages in use but {len(holders)} in block tables"
            for p, n in holders.items():
                assert g.pool.refcount(p) == n, f"group {g.index}: page {p} is in {n} block tables, held {g.pool.refcount(p)} times"
            for req, t in g.tables.items():
                assert g.np_tables[req][:len(t)].tolist() == t and (g.np_tables[req][len(t):] == -1).all()
