"""Host-side bookkeeping of the cache: slots, pages and per-sequence lengths.

A sequence of a batch holds one *slot* from its first step until it ends; the
slot indexes the page tables and the fixed-size state.  Keys and values live in
*pages* of ``PAGE`` positions.  Layers with the same needs form a *group* with
its own page pool: a group that keeps every key grows by a page each ``PAGE``
positions; a group that keeps a window of W keys is a ring of
ceil(W / PAGE) pages per sequence and stops growing there.

Nothing here touches a device, so the rules (no slot lost, held twice or freed
twice; pages returned exactly once) are tested on the CPU.

The reference keeps one flat block per layer for a single sequence and a
free-list of blocks (src/kvcache/manager.zig:76-185,
src/kvcache/block_allocator.zig:14-102); its ``KVCacheFull`` / ``OutOfBlocks``
errors (src/models/model.zig:32-43) correspond to ``CacheFull`` here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

PAGE = 64


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot, no free page, or a sequence longer than the cache allows."""


def round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class SlotAllocator:
    """Hands out slot numbers 0..n-1, lowest free first."""

    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise CacheError("a cache needs at least one slot")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._held = set()

    def acquire(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} slots are held")
        s = self._free.pop()
        self._held.add(s)
        return s

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheError(f"slot {slot} is not held (freed twice, or never acquired)")
        self._held.remove(slot)
        self._free.append(slot)
        self._free.sort(reverse=True)

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def held(self):
        return frozenset(self._held)


class PagePool:
    """A pool of page numbers with all-or-nothing allocation."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = set()

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{n} pages wanted, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        self._held.update(out)
        return out

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            if p not in self._held:
                raise CacheError(f"page {p} is not held (freed twice)")
        for p in pages:
            self._held.remove(p)
            self._free.append(p)

    @property
    def n_free(self) -> int:
        return len(self._free)


@dataclass
class GroupGeometry:
    """Sizes of one group of cache entries.

    ``cap`` is the number of ring rows a sequence may use (a multiple of PAGE):
    position p lives in row p % cap.  ``window`` None: every key is kept and cap
    covers the longest sequence.
    """
    n_kv_heads: int
    head_dim: int
    window: Optional[int]
    cap: int
    n_pages: int
    entries: List[int] = field(default_factory=list)     # cache entry ids, in order

    @property
    def max_pages(self) -> int:
        return self.cap // PAGE

    def pages_for(self, length: int) -> int:
        return min(round_up(length, PAGE), self.cap) // PAGE


class CacheBook:
    """Slots, per-group pages and lengths; pure host state.

    ``max_tokens`` bounds the sum over live sequences of their lengths rounded
    up to PAGE; ``max_seq_len`` bounds one sequence.
    """

    def __init__(self, groups: Sequence[GroupGeometry], n_slots: int, max_seq_len: int):
        self.groups = list(groups)
        self.slots = SlotAllocator(n_slots)
        self.pools = [PagePool(g.n_pages) for g in self.groups]
        self.max_seq_len = max_seq_len
        self.length: Dict[int, int] = {}
        self.pages: Dict[int, List[List[int]]] = {}
        self.dirty: set = set()          # slots whose page-table rows changed

    def acquire(self) -> int:
        s = self.slots.acquire()
        self.length[s] = 0
        self.pages[s] = [[] for _ in self.groups]
        self.dirty.add(s)
        return s

    def reserve(self, slot: int, new_len: int) -> None:
        """Make room for positions < new_len (all groups, or none on failure)."""
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not held")
        if new_len > self.max_seq_len:
            raise CacheFull(f"a sequence of {new_len} positions exceeds the cache's "
                            f"limit of {self.max_seq_len}")
        need = [g.pages_for(new_len) - len(self.pages[slot][i])
                for i, g in enumerate(self.groups)]
        for i, n in enumerate(need):
            if n > self.pools[i].n_free:
                raise CacheFull(
                    f"slot {slot} needs {n} more pages in group {i}, "
                    f"{self.pools[i].n_free} of {self.pools[i].n_pages} are free")
        for i, n in enumerate(need):
            if n > 0:
                self.pages[slot][i].extend(self.pools[i].alloc(n))
                self.dirty.add(slot)

    def trim(self, slot: int, length: Optional[int] = None) -> None:
        """Give back the pages beyond what ``length`` positions need (default: the
        slot's recorded length): undoes a reservation whose step did not run."""
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not held")
        n = self.length[slot] if length is None else length
        for i, g in enumerate(self.groups):
            keep = g.pages_for(n)
            extra = self.pages[slot][i][keep:]
            if extra:
                self.pools[i].free(extra)
                del self.pages[slot][i][keep:]
                self.dirty.add(slot)

    def set_length(self, slot: int, length: int) -> None:
        self.length[slot] = length

    def release(self, slot: int) -> None:
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not held (freed twice, or never acquired)")
        for i, pages in enumerate(self.pages[slot]):
            self.pools[i].free(pages)
        del self.pages[slot]
        del self.length[slot]
        self.slots.release(slot)

    def live_tokens(self) -> int:
        return sum(round_up(n, PAGE) for n in self.length.values())


def plan_groups(requests: Sequence[object], max_tokens: int, max_seq_len: int,
                n_slots: int) -> Tuple[List[GroupGeometry], Dict[int, Tuple[int, int]]]:
    """Group key/value requests by what they need.

    Returns the groups and {cache entry id: (group index, index within group)}.
    ``requests[i]`` is the KVRequest of cache entry i, or something else (no
    keys and values).
    """
    from ..parts.base import KVRequest
    groups: List[GroupGeometry] = []
    index: Dict[Tuple, int] = {}
    where: Dict[int, Tuple[int, int]] = {}
    full_cap = round_up(max_seq_len, PAGE)
    budget_pages = round_up(max_tokens, PAGE) // PAGE
    for entry, r in enumerate(requests):
        if not isinstance(r, KVRequest):
            continue
        window = r.window if (r.window is not None and round_up(r.window, PAGE) < full_cap) else None
        key = (r.n_kv_heads, r.head_dim, window)
        if key not in index:
            cap = full_cap if window is None else round_up(window, PAGE)
            n_pages = min(budget_pages, n_slots * (cap // PAGE))
            index[key] = len(groups)
            groups.append(GroupGeometry(r.n_kv_heads, r.head_dim, window, cap, max(1, n_pages)))
        g = index[key]
        where[entry] = (g, len(groups[g].entries))
        groups[g].entries.append(entry)
    return groups, where
