"""The cache manager: pages of keys and values, a block table per request and group.

Cache entries (one per writing call of the model's run order) with the same need -
kv heads, head size, window - form a group.  A group has its own pool of page ids and
its own block table per request, so layers that keep every key and layers that keep
a window of them never compete silently for the same pages.  A page id of a group is
valid in every entry of that group.

Protocol per step, as the reference's (src/kvcache/block_manager.cpp:30-35,
include/engine/block_manager.hpp:37-60): `reserve` grows the tables to hold the new
tokens, the kernels write them, `commit` advances the length.  `commit` also gives
back the pages of a windowed group that no later query can see.  `close` returns
everything the request holds.  Prefix sharing follows the reference's design
(src/kvcache/block_manager.cpp:132-221): full pages only, matched by a chained hash and
confirmed by comparing tokens, reference counted, evicted least recently used first;
unlike the reference, evictable cached pages count as free, so a pool full of cached
prefixes cannot block admission.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .pool import OutOfPages, PagePool, StateSlots


@dataclass(frozen=True)
class CacheNeed:
    """What one cache entry stores per token: kv_heads x head_dim keys and as many values.
    window = 0 keeps every key; window = W keeps what a query can still see of the last W."""

    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass
class CacheGroup:
    need: CacheNeed
    entries: List[int]            # cache entry ids (positions in the run order) in this group
    page_size: int
    num_pages: int


@dataclass
class RequestCache:
    """What one live request holds: per group a block table (page ids, -1 = given back),
    the number of committed tokens, and a state slot."""

    request_id: object
    slot: int
    tables: List[List[int]]
    length: int = 0
    shared_tokens: int = 0        # leading tokens that came from shared prefix pages
    closed: bool = False
    fresh_state: bool = True      # the state slot still holds what its previous owner left
    _arrays: Optional[list] = None    # per group (table length, int32 array) for the step's staging

    def table_array(self, g: int):
        """The block table of group g as an int32 numpy array, rebuilt only when it changed
        (tables only grow at the end; a windowed group also turns entries into -1 in place,
        which `note_release` reports)."""
        import numpy as np
        if self._arrays is None:
            self._arrays = [None] * len(self.tables)
        table = self.tables[g]
        cached = self._arrays[g]
        if cached is None or cached[0] > len(table):
            array = np.asarray(table, dtype=np.int32)
        elif cached[0] < len(table):
            array = np.concatenate([cached[1], np.asarray(table[cached[0]:], dtype=np.int32)])
        else:
            return cached[1]
        self._arrays[g] = (len(table), array)
        return array

    def note_release(self, g: int, block: int) -> None:
        if self._arrays is not None and self._arrays[g] is not None and block < self._arrays[g][0]:
            self._arrays[g][1][block] = -1


@dataclass
class _PrefixEntry:
    parent: int
    tokens: Tuple[int, ...]
    pages: Tuple[int, ...]        # one page per group
    last_used: int


def _hash_block(parent: int, tokens: Sequence[int]) -> int:
    """Hash of (parent page's hash, this page's tokens), chained like the reference's FNV-1a
    (src/kvcache/block_manager.cpp:120-130) but with the interpreter's tuple hash; matches are
    confirmed by comparing tokens, so a collision costs a probe, not correctness."""
    return hash((parent, tuple(tokens)))


def group_needs(needs: Sequence[Optional[CacheNeed]]) -> List[Tuple[CacheNeed, List[int]]]:
    """Group cache entries by equal need, in order of first appearance."""
    grouped: Dict[CacheNeed, List[int]] = {}
    for entry, need in enumerate(needs):
        if need is not None:
            grouped.setdefault(need, []).append(entry)
    return list(grouped.items())


class CacheManager:
    def __init__(self, needs: Sequence[Optional[CacheNeed]], page_size: int,
                 num_pages, num_slots: int, enable_prefix_cache: bool = False,
                 has_state: bool = False):
        """`needs[e]` is the need of cache entry e (None for an entry without keys).
        `num_pages` is one count for every group or a list with one count per group.
        `has_state` says that some layer keeps per-request state of fixed size in the slots."""
        if page_size <= 0:
            raise ValueError("CacheManager: page_size must be positive")
        grouped = group_needs(needs)
        counts = list(num_pages) if isinstance(num_pages, (list, tuple)) else \
            [num_pages] * len(grouped)
        if len(counts) != len(grouped):
            raise ValueError(f"CacheManager: {len(grouped)} groups but {len(counts)} page counts")
        self.page_size = page_size
        self.groups = [CacheGroup(need, entries, page_size, n)
                       for (need, entries), n in zip(grouped, counts)]
        self.pools = [PagePool(g.num_pages) for g in self.groups]
        self.slots = StateSlots(num_slots)
        self.entry_group: Dict[int, Tuple[int, int]] = {}      # entry -> (group, index in group)
        for gi, group in enumerate(self.groups):
            for index, entry in enumerate(group.entries):
                self.entry_group[entry] = (gi, index)
        self.live: Dict[object, RequestCache] = {}
        # sharing a prefix needs every position's keys to be kept (no windowed group) and
        # nothing else that the shared tokens would have had to pass through: fixed-size state
        # has no copy per page, so a request that skipped tokens would start from a wrong state
        self.prefix_enabled = (enable_prefix_cache and not has_state
                               and all(g.need.window == 0 for g in self.groups))
        self._prefix: Dict[int, List[_PrefixEntry]] = {}
        # cached entries from least to most recently used, and by their page in group 0 (the
        # pages of an entry are always shared together, so group 0 speaks for all of them);
        # _idle holds the entries nobody but the cache holds, in the order in which their last
        # holder let go of them, kept up to date on every reference change: free_pages() costs
        # nothing per step and an eviction takes the first of them without walking past the
        # entries that live requests still hold
        self._lru: "OrderedDict[int, _PrefixEntry]" = OrderedDict()
        self._cached_page: Dict[int, _PrefixEntry] = {}
        self._idle: "OrderedDict[int, _PrefixEntry]" = OrderedDict()
        self._tick = 0
        self.prefix_hits = 0

    # ------------------------------------------------------------------ requests
    def open(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise RuntimeError(f"request {request_id!r} is already open")
        handle = RequestCache(request_id, self.slots.acquire(), [[] for _ in self.groups])
        self.live[request_id] = handle
        return handle

    def close(self, handle: RequestCache) -> None:
        if handle.closed:
            raise RuntimeError(f"request {handle.request_id!r} was closed twice")
        for g, table in enumerate(handle.tables):
            for page in table:
                if page >= 0:
                    self._free(g, page)
            table.clear()
        handle._arrays = None
        self.slots.release(handle.slot)
        handle.length = 0
        handle.shared_tokens = 0
        handle.closed = True
        del self.live[handle.request_id]

    def can_open(self) -> bool:
        return self.slots.num_free > 0

    # --------------------------------------------------------------------- sizes
    def blocks_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, handle: RequestCache, n_new: int) -> List[int]:
        """Pages each group must add so the request can hold `n_new` more tokens."""
        want = self.blocks_for(handle.length + n_new)
        return [max(0, want - len(table)) for table in handle.tables]

    def fits_in_held_pages(self, handle: RequestCache, n_new: int) -> bool:
        """Whether `n_new` more tokens need no new page (the common case of a decode step)."""
        want = (handle.length + n_new + self.page_size - 1) // self.page_size
        for table in handle.tables:
            if len(table) < want:
                return False
        return True

    def free_pages(self) -> List[int]:
        """Free pages per group, counting cached prefix pages nobody else holds."""
        return [pool.num_free + len(self._idle) for pool in self.pools]

    def _incref(self, g: int, page: int) -> None:
        if g == 0 and page in self._cached_page and self.pools[0].ref_count(page) == 1:
            del self._idle[id(self._cached_page[page])]       # a request shares it again
        self.pools[g].incref(page)

    def _free(self, g: int, page: int) -> None:
        self.pools[g].free(page)
        if g == 0 and page in self._cached_page and self.pools[0].ref_count(page) == 1:
            entry = self._cached_page[page]
            self._idle[id(entry)] = entry     # only the cache holds it now

    def can_reserve(self, handle: RequestCache, n_new: int,
                    budget: Optional[List[int]] = None) -> bool:
        budget = self.free_pages() if budget is None else budget
        return all(n <= b for n, b in zip(self.pages_needed(handle, n_new), budget))

    def max_tokens_per_request(self) -> int:
        """Tokens one request alone can hold (the full-attention groups bound it)."""
        full = [g.num_pages for g in self.groups if g.need.window == 0]
        if not full:
            return 1 << 62
        return min(full) * self.page_size

    # ------------------------------------------------------------ step protocol
    def reserve(self, handle: RequestCache, n_new: int) -> None:
        if self.fits_in_held_pages(handle, n_new):
            return
        needed = self.pages_needed(handle, n_new)
        if not all(n <= b for n, b in zip(needed, self.free_pages())):
            raise OutOfPages(f"request {handle.request_id!r} needs {needed} pages, "
                             f"free are {self.free_pages()}")
        for g, count in enumerate(needed):
            for _ in range(count):
                handle.tables[g].append(self._allocate(g))

    def commit(self, handle: RequestCache, n_new: int) -> None:
        handle.length += n_new
        for g, group in enumerate(self.groups):
            window = group.need.window
            if window <= 0:
                continue
            # the next query sits at position `length` and sees keys > length - window
            first_needed = handle.length - window + 1
            table = handle.tables[g]
            for block in range(min(len(table), max(0, first_needed) // self.page_size)):
                if table[block] >= 0:
                    self._free(g, table[block])
                    table[block] = -1
                    handle.note_release(g, block)

    def _allocate(self, g: int) -> int:
        if self.pools[g].num_free == 0:
            self._evict_one()
        return self.pools[g].allocate()

    # -------------------------------------------------------------- prefix cache
    def acquire_prefix(self, handle: RequestCache, tokens: Sequence[int]) -> int:
        """Share the leading full pages of `tokens` that are cached; returns tokens shared.
        Only for a request that holds nothing yet (src/kvcache/block_manager.cpp:132-173)."""
        if not self.prefix_enabled or handle.length != 0 or any(handle.tables):
            return 0
        ps = self.page_size
        parent = 0
        matched = 0
        for b in range(len(tokens) // ps):
            span = tuple(tokens[b * ps:(b + 1) * ps])
            h = _hash_block(parent, span)
            found = None
            for entry in self._prefix.get(h, ()):
                if entry.parent == parent and entry.tokens == span:
                    found = entry
                    break
            if found is None:
                break
            self._tick += 1
            found.last_used = self._tick
            self._lru.move_to_end(id(found))
            for g, page in enumerate(found.pages):
                self._incref(g, page)
                handle.tables[g].append(page)
            parent = h
            matched += ps
        handle.length = matched
        handle.shared_tokens = matched
        if matched:
            self.prefix_hits += 1
        return matched

    def release_prefix(self, handle: RequestCache) -> None:
        """Undo `acquire_prefix` for a request that has run nothing since: the shared pages are
        given back (they stay cached) and the request holds nothing again."""
        if handle.length != handle.shared_tokens:
            raise RuntimeError(f"request {handle.request_id!r} has run tokens of its own")
        if handle.shared_tokens:
            self.prefix_hits -= 1
        for g, table in enumerate(handle.tables):
            for page in table:
                if page >= 0:
                    self._free(g, page)
            table.clear()
        handle._arrays = None
        handle.length = handle.shared_tokens = 0

    def register_prefix(self, handle: RequestCache, tokens: Sequence[int]) -> None:
        """Remember the request's full pages covering `tokens` for later requests
        (src/kvcache/block_manager.cpp:175-204); the cache holds its own reference."""
        if not self.prefix_enabled:
            return
        ps = self.page_size
        full = min(min(len(t) for t in handle.tables) if handle.tables else 0,
                   min(len(tokens), handle.length) // ps)
        parent = 0
        for b in range(full):
            span = tuple(tokens[b * ps:(b + 1) * ps])
            h = _hash_block(parent, span)
            entries = self._prefix.setdefault(h, [])
            if not any(e.parent == parent and e.tokens == span for e in entries):
                pages = tuple(table[b] for table in handle.tables)
                if pages[0] in self._cached_page:
                    parent = h            # the page already backs another entry: share no further
                    continue
                for g, page in enumerate(pages):
                    self.pools[g].incref(page)
                self._tick += 1
                entry = _PrefixEntry(parent, span, pages, self._tick)
                entries.append(entry)
                self._lru[id(entry)] = entry
                self._cached_page[pages[0]] = entry
            parent = h

    def _drop_entry(self, entry: _PrefixEntry) -> None:
        h = _hash_block(entry.parent, entry.tokens)
        bucket = self._prefix[h]
        bucket.remove(entry)
        if not bucket:
            del self._prefix[h]
        del self._lru[id(entry)]
        del self._cached_page[entry.pages[0]]
        self._idle.pop(id(entry), None)
        for g, page in enumerate(entry.pages):
            self.pools[g].free(page)

    def _evict_one(self) -> bool:
        """Drop the entry that only the cache holds and that has been idle longest (the
        reference evicts by the tick of the last use among such entries,
        src/kvcache/block_manager.cpp:206-212; an entry's last holder lets go of it after its
        last use, so the order is nearly the same and costs no search)."""
        if not self._idle:
            return False
        self._drop_entry(next(iter(self._idle.values())))
        return True

    def clear_prefix_cache(self) -> None:
        for entry in list(self._lru.values()):
            self._drop_entry(entry)

    # ----------------------------------------------------------------- checking
    def check(self) -> None:
        """No page lost, none held twice without a matching reference count."""
        for g, pool in enumerate(self.pools):
            pool.check()
            holders = [0] * pool.num_pages
            for handle in self.live.values():
                for page in handle.tables[g]:
                    if page >= 0:
                        holders[page] += 1
            for entries in self._prefix.values():
                for entry in entries:
                    holders[entry.pages[g]] += 1
            for page, count in enumerate(holders):
                if count != pool.ref_count(page):
                    raise AssertionError(f"group {g} page {page}: {count} holders but "
                                         f"reference count {pool.ref_count(page)}")
        idle = {id(e) for e in self._lru.values() if self.pools[0].ref_count(e.pages[0]) == 1}
        if idle != set(self._idle) or len(self._lru) != sum(map(len, self._prefix.values())):
            raise AssertionError(f"prefix cache accounting: {len(self._idle)} idle entries listed, "
                                 f"{len(idle)} found")
