"""The step function: a batch of sequences, only the tokens given, from the cache.

``Runner.step`` takes, for each sequence of the batch, its cache slot and its
next tokens, and the places whose logits are wanted.  A batch either starts
(every slot is empty; whole prompts of unequal lengths run in one step) or
goes on by one token per sequence.  Tokens of all sequences lie on one ragged
axis, so nothing is padded in a prompt step; a decode batch may carry padding
entries (slot -1), which the kernels skip.

The reference has ``forward(one token)`` and ``prefill(one sequence)`` over a
single shared sequence state (src/models/gemma3.zig:331-442); its "batching"
is a host loop over single-token forwards (src/server/scheduler.zig:360-392).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ..cache import Cache, CacheError
from .batch import DECODE, PREFILL, StepContext


class StepError(ValueError):
    pass


class Runner:
    """A model with its cache; owns nothing else."""

    def __init__(self, model, max_tokens: int, max_seq_len: int, n_slots: int):
        self.model = model
        self.device, self.dtype = model.device, model.dtype
        self.cache = Cache(model.cache_requests(), max_tokens, max_seq_len, n_slots,
                           model.dtype, model.device)
        self.vocab_size = model.spec.vocab_size

    # ------------------------------------------------------------- contexts
    def _pack(self, tokens: Sequence[int], positions: Sequence[int], seq_index: Sequence[int],
              cu: Sequence[int], slots: Sequence[int], lens: Sequence[int]):
        T, B = len(tokens), len(slots)
        host = torch.empty(3 * T + 3 * B + 1, dtype=torch.int32, pin_memory=True)
        host[:T] = torch.tensor(tokens, dtype=torch.int32)
        host[T:2 * T] = torch.tensor(positions, dtype=torch.int32)
        host[2 * T:3 * T] = torch.tensor(seq_index, dtype=torch.int32)
        o = 3 * T
        host[o:o + B + 1] = torch.tensor(cu, dtype=torch.int32)
        host[o + B + 1:o + 2 * B + 1] = torch.tensor(slots, dtype=torch.int32)
        host[o + 2 * B + 1:] = torch.tensor(lens, dtype=torch.int32)
        dev = host.to(self.device, non_blocking=True)
        return (dev[:T], dev[T:2 * T], dev[2 * T:3 * T], dev[o:o + B + 1],
                dev[o + B + 1:o + 2 * B + 1], dev[o + 2 * B + 1:])

    def context(self, entries: Sequence[Tuple[int, Sequence[int]]]) -> StepContext:
        """Check a batch, reserve its cache room and build its device arrays.

        ``entries``: (slot, tokens) per sequence; slot -1 with one token is a
        padding entry of a decode batch.
        """
        if not entries:
            raise StepError("a step needs at least one sequence")
        book = self.cache.book
        real = [(s, t) for s, t in entries if s >= 0]
        seen = set()
        for s, toks in real:
            if s not in book.length:
                raise StepError(f"slot {s} is not held")
            if s in seen:
                raise StepError(f"slot {s} appears twice in one step")
            seen.add(s)
            if len(toks) == 0:
                raise StepError(f"slot {s} brings no tokens")
        V = self.vocab_size
        for s, toks in entries:
            for t in toks:
                if not 0 <= int(t) < V:
                    raise StepError(f"token id {t} is outside the vocabulary of {V}")
        starts = [book.length[s] for s, _ in real]
        if real and all(st == 0 for st in starts) and len(real) == len(entries):
            mode = PREFILL
        elif all(len(t) == 1 for _, t in entries) and all(st > 0 for st in starts):
            mode = DECODE
        else:
            raise StepError("the sequences of a step must either all start at position 0 or "
                            "all go on by exactly one token")
        # all-or-nothing reservation
        reserved = []
        try:
            for s, toks in real:
                book_len = book.length[s]
                self.cache.reserve(s, book_len + len(toks))
                reserved.append(s)
        except CacheError:
            raise
        tokens: List[int] = []
        positions: List[int] = []
        seq_index: List[int] = []
        cu = [0]
        slots, lens = [], []
        for b, (s, toks) in enumerate(entries):
            start = book.length[s] if s >= 0 else 0
            tokens.extend(int(t) for t in toks)
            positions.extend(range(start, start + len(toks)))
            seq_index.extend([b] * len(toks))
            cu.append(len(tokens))
            slots.append(s)
            lens.append(start + len(toks) if s >= 0 else 0)
        self.cache.flush()
        d = self._pack(tokens, positions, seq_index, cu, slots, lens)
        ctx = StepContext(mode=mode, n_tokens=len(tokens), batch=len(entries), tokens=d[0],
                          positions=d[1], seq_index=d[2], cu_seqlens=d[3], slots=d[4], lens=d[5],
                          max_len=max(lens), max_new=max(len(t) for _, t in entries),
                          cache=self.cache, dtype=self.dtype, device=self.device)
        return ctx

    def commit(self, entries: Sequence[Tuple[int, Sequence[int]]]) -> None:
        """Record that the step ran: lengths grow by the tokens brought."""
        for s, toks in entries:
            if s >= 0:
                self.cache.book.set_length(s, self.cache.book.length[s] + len(toks))

    # ----------------------------------------------------------------- step
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Sequence[Sequence[int]]) -> torch.Tensor:
        """Run one step; 32-bit logits [sum(len(w) for w in want), V].

        ``want[b]`` lists the places among entry b's tokens whose logits are
        returned, in the order of the entries and of ``want``.
        """
        if len(want) != len(entries):
            raise StepError("want must have one list per sequence")
        rows: List[int] = []
        off = 0
        for (s, toks), w in zip(entries, want):
            for i in w:
                if not 0 <= int(i) < len(toks):
                    raise StepError(f"wanted place {i} is outside the {len(toks)} tokens of a "
                                    "sequence")
                rows.append(off + int(i))
            off += len(toks)
        ctx = self.context(entries)
        h = self.model.hidden_states(ctx)
        self.commit(entries)
        if not rows:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        rows_dev = torch.tensor(rows, dtype=torch.int32).to(self.device)
        return self.model.logits(h, rows_dev, ctx)

    # ------------------------------------------------------------ lifecycle
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)
