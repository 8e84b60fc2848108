"""The cache on the device: page pools per group, page tables, fixed-size state.

Layout of one group: keys and values ``[entries, pages, PAGE, n_kv_heads,
head_dim]`` in the compute dtype, and one page table ``[slots, max_pages]``
(int32) shared by the group's entries.  Position p of the sequence in slot s is
row p % cap; its page is ``page_table[s, row // PAGE]``.  Nothing is cleared
when a slot is reused: every read is bounded by the sequence's length.

Fixed-size state is ``[entries, slots, numel]`` in 32-bit and is zeroed when a
slot is acquired.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVRequest, StateRequest
from .book import PAGE, CacheBook, CacheError, CacheFull, GroupGeometry, plan_groups, round_up


@dataclass
class KVView:
    """What an attention layer needs to reach its keys and values."""
    k_pool: torch.Tensor          # [pages, PAGE, nkv, hd] of this entry
    v_pool: torch.Tensor
    page_table: torch.Tensor      # [slots, max_pages] int32
    page: int
    cap: int
    window: Optional[int]


@dataclass
class StateView:
    state: torch.Tensor           # [slots, numel] float32 of this entry


class Cache:
    def __init__(self, requests: Sequence[object], max_tokens: int, max_seq_len: int,
                 n_slots: int, dtype: torch.dtype, device: torch.device):
        self.requests = list(requests)
        self.dtype, self.device = dtype, device
        max_seq_len = max(1, min(max_seq_len, round_up(max_tokens, PAGE)))
        self.max_seq_len = max_seq_len
        self.max_tokens = max_tokens
        groups, self.where = plan_groups(self.requests, max_tokens, max_seq_len, n_slots)
        self.book = CacheBook(groups, n_slots, max_seq_len)
        self.n_slots = n_slots
        self.k_pools: List[torch.Tensor] = []
        self.v_pools: List[torch.Tensor] = []
        self.tables: List[torch.Tensor] = []
        for g in groups:
            shape = (len(g.entries), g.n_pages, PAGE, g.n_kv_heads, g.head_dim)
            self.k_pools.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v_pools.append(torch.zeros(shape, dtype=dtype, device=device))
            self.tables.append(torch.zeros((n_slots, g.max_pages), dtype=torch.int32,
                                           device=device))
        # fixed-size state: one tensor per distinct size
        self.state_where: Dict[int, Tuple[int, int]] = {}
        sizes: Dict[int, List[int]] = {}
        for entry, r in enumerate(self.requests):
            if isinstance(r, StateRequest):
                sizes.setdefault(r.numel, []).append(entry)
        self.states: List[torch.Tensor] = []
        for numel, entries in sizes.items():
            for i, e in enumerate(entries):
                self.state_where[e] = (len(self.states), i)
            self.states.append(torch.zeros((len(entries), n_slots, numel), dtype=torch.float32,
                                           device=device))

    # ------------------------------------------------------------- lifecycle
    def acquire(self) -> int:
        s = self.book.acquire()
        for st in self.states:
            st[:, s].zero_()
        return s

    def reserve(self, slot: int, new_len: int) -> None:
        self.book.reserve(slot, new_len)

    def trim(self, slot: int) -> None:
        self.book.trim(slot)

    def release(self, slot: int) -> None:
        self.book.release(slot)

    def flush(self) -> None:
        """Copy changed page-table rows to the device (on the current stream).

        Every flush stages its rows in pinned memory of its own: a copy that has
        not run yet must not see what a later flush writes for the same slot (a
        slot released and taken again with no read in between).  The pinned
        allocator hands a block out again only after the copies from it have run."""
        if not self.book.dirty:
            return
        pinned = self.device.type == "cuda"
        for s in sorted(self.book.dirty):
            pages = self.book.pages.get(s)
            if pages is None:
                continue
            for gi, plist in enumerate(pages):
                if not plist:
                    continue
                row = torch.tensor(plist, dtype=torch.int32)
                if pinned:
                    row = row.pin_memory()
                self.tables[gi][s, :len(plist)].copy_(row, non_blocking=True)
        self.book.dirty.clear()

    # ----------------------------------------------------------------- views
    def kv_view(self, entry: int) -> KVView:
        if entry not in self.where:
            raise CacheError(f"cache entry {entry} holds no keys and values")
        gi, li = self.where[entry]
        g = self.book.groups[gi]
        return KVView(self.k_pools[gi][li], self.v_pools[gi][li], self.tables[gi], PAGE, g.cap,
                      g.window)

    def state_view(self, entry: int) -> StateView:
        if entry not in self.state_where:
            raise CacheError(f"cache entry {entry} holds no fixed-size state")
        ti, li = self.state_where[entry]
        return StateView(self.states[ti][li])

    def bytes_held(self) -> int:
        n = 0
        for t in self.k_pools + self.v_pools + self.states + self.tables:
            n += t.numel() * t.element_size()
        return n
