"""Cache manager: who holds which pages, and which per-request state slot. Host only; it never
touches device memory.

Kept from the reference's BlockManager (src/infer/kv/paged_cache.py:55-182): pages of ``page_size``
tokens; a block table per request; ``slot = table[pos // page_size] * page_size + pos % page_size``
(paged_cache.py:90-91); admission OK / LATER / NEVER against a watermark (paged_cache.py:95-102);
pages for the whole sequence at admission (paged_cache.py:104-123); growth by one page when a
sequence crosses a page edge (paged_cache.py:125-131); pages given back in reverse order
(paged_cache.py:133-137); prefix caching by a chain of hashes over full pages, published after the
step that filled them (paged_cache.py:141-182).

Beyond the reference: layers with different needs form *groups*, each with a pool, an allocator and
block tables of its own (a request holds one table per group); a group with a window gives pages
back as soon as every future query's window has passed them; and fixed-size per-request state lives
in numbered slots handed out at admission. Hashes are an explicit 64-bit digest, so they are equal
across processes.
"""

from __future__ import annotations

import enum
import hashlib
from array import array
from dataclasses import dataclass, field

from .allocator import OutOfPages, PageAllocator


class AllocStatus(enum.Enum):
    OK = 0
    LATER = 1      # not enough free pages (or state slots) now
    NEVER = 2      # would not fit even in an empty pool


class StateSlots:
    """Numbered slots for per-request state of fixed size; a free stack."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no per-request state slot is free")
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise RuntimeError(f"state slot {slot} is not held")
        self._held.remove(slot)
        self._free.append(slot)

    def check_invariants(self) -> None:
        if len(set(self._free)) != len(self._free) or set(self._free) & self._held:
            raise AssertionError("state slot lists are inconsistent")
        if len(self._free) + len(self._held) != self.num_slots:
            raise AssertionError("a state slot was lost")


@dataclass
class CacheHandle:
    """What one request holds. tables[g][i] is the physical page of logical page i in group g, or -1
    once a window has passed it."""

    tables: list[list[int]]
    state_slot: int = -1
    page_hashes: list[int] = field(default_factory=list)
    num_registered_pages: int = 0
    fresh_state: bool = False      # the state slot was just handed out and must be zeroed before use

    @property
    def holds_pages(self) -> bool:
        return any(p >= 0 for t in self.tables for p in t)


def chain_hash(parent: int | None, tokens: list[int]) -> int:
    """64-bit digest of (previous page's digest, this page's token ids)."""
    h = hashlib.blake2b(digest_size=8)
    h.update((parent if parent is not None else 0).to_bytes(8, "little"))
    h.update(b"\x01" if parent is not None else b"\x00")
    h.update(array("q", tokens).tobytes())
    return int.from_bytes(h.digest(), "little")


class CacheManager:
    def __init__(self, num_pages: int | list[int], page_size: int, windows: list[int | None] | None = None,
                 watermark: float = 0.01, enable_prefix_caching: bool = False, num_state_slots: int = 0):
        self.windows = list(windows) if windows is not None else [None]
        self.num_groups = len(self.windows)
        pages = num_pages if isinstance(num_pages, list) else [num_pages] * self.num_groups
        if len(pages) != self.num_groups:
            raise ValueError("one page count per group")
        if page_size < 1:
            raise ValueError("page_size must be at least 1")
        self.page_size = page_size
        self.num_pages = pages
        # Prefix hits skip computing tokens, which is only sound when every layer can read those
        # tokens back: no windowed group, no per-request state.
        self.enable_prefix_caching = bool(enable_prefix_caching) and all(w is None for w in self.windows) \
            and num_state_slots == 0 and self.num_groups > 0
        self.allocators = [PageAllocator(n, self.enable_prefix_caching, on_evict=self._evictor(g))
                           for g, n in enumerate(pages)]
        self.watermark_pages = [int(watermark * n) for n in pages]
        self.state_slots = StateSlots(num_state_slots) if num_state_slots > 0 else None
        self._hash_to_pages: dict[int, list[int]] = {}       # digest -> one page per group
        self._page_to_hash: list[dict[int, int]] = [dict() for _ in pages]
        self.prefix_hit_tokens = 0
        self.prefix_query_tokens = 0

    # --- bookkeeping ----------------------------------------------------------------------------

    def new_handle(self) -> CacheHandle:
        return CacheHandle(tables=[[] for _ in range(self.num_groups)])

    def pages_for(self, num_tokens: int) -> int:
        return -(-num_tokens // self.page_size)

    @property
    def num_free_pages(self) -> int:
        """Free pages of the tightest group."""
        return min((a.num_free for a in self.allocators), default=0)

    @property
    def all_free(self) -> bool:
        return all(a.num_free == a.num_pages for a in self.allocators) and \
            (self.state_slots is None or self.state_slots.num_free == self.state_slots.num_slots)

    def usage(self) -> float:
        return max((a.num_used / a.num_pages for a in self.allocators), default=0.0)

    def slot(self, handle: CacheHandle, group: int, pos: int) -> int:
        page = handle.tables[group][pos // self.page_size]
        if page < 0:
            raise RuntimeError(f"position {pos} lies in a page that was already given back")
        return page * self.page_size + pos % self.page_size

    # --- admission / growth / release -----------------------------------------------------------

    def admission_status(self, handle: CacheHandle, token_ids: list[int]) -> AllocStatus:
        need = self.pages_for(len(token_ids))
        for g in range(self.num_groups):
            if need + self.watermark_pages[g] > self.num_pages[g]:
                return AllocStatus.NEVER
        if self.state_slots is not None and self.state_slots.num_free < 1:
            return AllocStatus.LATER
        hits = self._num_active_prefix_hits(handle, token_ids)
        for g, alloc in enumerate(self.allocators):
            if alloc.num_free - (need - hits) < self.watermark_pages[g]:
                return AllocStatus.LATER
        return AllocStatus.OK

    def allocate(self, handle: CacheHandle, token_ids: list[int]) -> int:
        """Give a waiting request pages for all of ``token_ids`` in every group (and a state slot).
        Returns the number of leading tokens whose pages were found in the prefix cache and need
        not be computed again."""
        if handle.holds_pages or handle.state_slot >= 0:
            raise RuntimeError("the request still holds pages")
        need = self.pages_for(len(token_ids))
        shared: list[list[int]] = []
        if self.enable_prefix_caching:
            hashes = self._page_hashes(handle, token_ids)
            reusable = (len(token_ids) - 1) // self.page_size          # always compute >= 1 token
            for h in hashes[:reusable]:
                pages = self._hash_to_pages.get(h)
                if pages is None:
                    break
                shared.append(pages)
            self.prefix_query_tokens += len(token_ids)
        for g, alloc in enumerate(self.allocators):
            fresh_needed = need - len(shared)
            revive = sum(1 for pages in shared if alloc.refcount[pages[g]] == 0)
            if fresh_needed > alloc.num_free - revive:
                raise OutOfPages(f"group {g}: need {fresh_needed} pages, {alloc.num_free - revive} available")
        if self.state_slots is not None and self.state_slots.num_free < 1:
            raise OutOfPages("no per-request state slot is free")
        for g, alloc in enumerate(self.allocators):
            table = []
            for pages in shared:
                alloc.share(pages[g])
                table.append(pages[g])
            table += alloc.allocate(need - len(shared))
            handle.tables[g] = table
        if self.state_slots is not None:
            handle.state_slot = self.state_slots.allocate()
            handle.fresh_state = True
        handle.num_registered_pages = len(shared)
        self.prefix_hit_tokens += len(shared) * self.page_size
        return len(shared) * self.page_size

    def can_grow(self, handle: CacheHandle, num_tokens: int) -> bool:
        """Room for the sequence to reach ``num_tokens`` tokens?"""
        need = self.pages_for(num_tokens)
        return all(need - len(handle.tables[g]) <= a.num_free for g, a in enumerate(self.allocators))

    def grow(self, handle: CacheHandle, num_tokens: int) -> None:
        need = self.pages_for(num_tokens)
        if not self.can_grow(handle, num_tokens):
            raise OutOfPages(f"cannot grow to {num_tokens} tokens")
        for g, alloc in enumerate(self.allocators):
            extra = need - len(handle.tables[g])
            if extra > 0:
                handle.tables[g] += alloc.allocate(extra)

    def release_behind_window(self, handle: CacheHandle, num_computed: int) -> int:
        """Give back, in windowed groups, the pages no future query can read: page i goes once
        (i + 1) * page_size <= num_computed - window + 1. Returns how many pages were released."""
        released = 0
        for g, window in enumerate(self.windows):
            if window is None:
                continue
            dead = max(0, (num_computed - window + 1)) // self.page_size
            table = handle.tables[g]
            for i in range(min(dead, len(table))):
                if table[i] >= 0:
                    self.allocators[g].release([table[i]])
                    table[i] = -1
                    released += 1
        return released

    def free(self, handle: CacheHandle) -> None:
        """Give back everything the request holds. Reverse order: with caching, a prefix's tail pages
        become evictable before its head."""
        for g, alloc in enumerate(self.allocators):
            alloc.release([p for p in reversed(handle.tables[g]) if p >= 0])
            handle.tables[g] = []
        if handle.state_slot >= 0:
            self.state_slots.release(handle.state_slot)
            handle.state_slot = -1
        handle.num_registered_pages = 0
        handle.fresh_state = False

    # --- prefix caching -------------------------------------------------------------------------

    def _page_hashes(self, handle: CacheHandle, token_ids: list[int]) -> list[int]:
        hashes = handle.page_hashes
        ps = self.page_size
        for i in range(len(hashes), len(token_ids) // ps):
            hashes.append(chain_hash(hashes[-1] if hashes else None, token_ids[i * ps:(i + 1) * ps]))
        return hashes

    def _num_active_prefix_hits(self, handle: CacheHandle, token_ids: list[int]) -> int:
        """Prefix pages somebody else holds right now: reusing them costs no free page."""
        if not self.enable_prefix_caching:
            return 0
        hits = 0
        for h in self._page_hashes(handle, token_ids)[:(len(token_ids) - 1) // self.page_size]:
            pages = self._hash_to_pages.get(h)
            if pages is None:
                break
            if all(self.allocators[g].refcount[p] > 0 for g, p in enumerate(pages)):
                hits += 1
        return hits

    def register_computed(self, handle: CacheHandle, token_ids: list[int], num_computed: int) -> None:
        """After a step: publish every page the step filled, so later requests can share it."""
        if not self.enable_prefix_caching:
            return
        full = num_computed // self.page_size
        if full <= handle.num_registered_pages:
            return
        hashes = self._page_hashes(handle, token_ids)
        for i in range(handle.num_registered_pages, full):
            h = hashes[i]
            pages = [handle.tables[g][i] for g in range(self.num_groups)]
            if h not in self._hash_to_pages and all(p not in self._page_to_hash[g] for g, p in enumerate(pages)):
                self._hash_to_pages[h] = pages
                for g, p in enumerate(pages):
                    self._page_to_hash[g][p] = h
                    self.allocators[g].mark_cached(p)
        handle.num_registered_pages = full

    def _evictor(self, group: int):
        def on_evict(page: int) -> None:
            h = self._page_to_hash[group].pop(page, None)
            if h is not None:
                # The digest names one page per group; once any of them is gone the entry is dead.
                pages = self._hash_to_pages.pop(h, None)
                if pages is not None:
                    for g, p in enumerate(pages):
                        if g != group:
                            self._page_to_hash[g].pop(p, None)
        return on_evict

    def check_invariants(self) -> None:
        for a in self.allocators:
            a.check_invariants()
        if self.state_slots is not None:
            self.state_slots.check_invariants()
