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

import numpy as np
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
    def context(self, entries: Sequence[Tuple[int, Sequence[int]]]) -> StepContext:
        """Check a batch, reserve its cache room and build its device arrays.

        ``entries``: (slot, tokens) per sequence; slot -1 with one token is a
        padding entry of a decode batch.
        """
        if not entries:
            raise StepError("a step needs at least one sequence")
        book = self.cache.book
        B = len(entries)
        slots = np.fromiter((s for s, _ in entries), dtype=np.int64, count=B)
        toks = [np.asarray(t, dtype=np.int64).reshape(-1) for _, t in entries]
        counts = np.fromiter((t.size for t in toks), dtype=np.int64, count=B)
        real = slots >= 0
        seen = set()
        for s, c in zip(slots.tolist(), counts.tolist()):
            if s < 0:
                continue
            if s not in book.length:
                raise StepError(f"slot {s} is not held")
            if s in seen:
                raise StepError(f"slot {s} appears twice in one step")
            seen.add(s)
            if c == 0:
                raise StepError(f"slot {s} brings no tokens")
        tokens = np.concatenate(toks) if B else np.zeros(0, dtype=np.int64)
        V = self.vocab_size
        if tokens.size and (tokens.min() < 0 or tokens.max() >= V):
            bad = tokens[(tokens < 0) | (tokens >= V)][0]
            raise StepError(f"token id {int(bad)} is outside the vocabulary of {V}")
        starts = np.fromiter((book.length[s] if s >= 0 else 0 for s in slots.tolist()),
                             dtype=np.int64, count=B)
        if real.all() and (starts == 0).all():
            mode = PREFILL
        elif (counts == 1).all() and (starts[real] > 0).all():
            mode = DECODE
        else:
            raise StepError("the sequences of a step must either all start at position 0 or "
                            "all go on by exactly one token")
        for s, st, c in zip(slots.tolist(), starts.tolist(), counts.tolist()):
            if s >= 0:
                self.cache.reserve(s, st + c)
        self.cache.flush()
        T = int(counts.sum())
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(counts, out=cu[1:])
        seq_index = np.repeat(np.arange(B, dtype=np.int64), counts)
        positions = np.arange(T, dtype=np.int64) - cu[:-1][seq_index] + starts[seq_index]
        lens = np.where(real, starts + counts, 0)
        host = torch.empty(3 * T + 3 * B + 1, dtype=torch.int32, pin_memory=True)
        a = host.numpy()
        a[:T] = tokens
        a[T:2 * T] = positions
        a[2 * T:3 * T] = seq_index
        o = 3 * T
        a[o:o + B + 1] = cu
        a[o + B + 1:o + 2 * B + 1] = slots
        a[o + 2 * B + 1:] = lens
        dev = host.to(self.device, non_blocking=True)
        return StepContext(mode=mode, n_tokens=T, batch=B, tokens=dev[:T],
                           positions=dev[T:2 * T], seq_index=dev[2 * T:3 * T],
                           cu_seqlens=dev[o:o + B + 1], slots=dev[o + B + 1:o + 2 * B + 1],
                           lens=dev[o + 2 * B + 1:], max_len=int(lens.max()),
                           max_new=int(counts.max()), cache=self.cache, dtype=self.dtype,
                           device=self.device)

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
        rows_host = torch.tensor(rows, dtype=torch.int32).pin_memory()
        rows_dev = rows_host.to(self.device, non_blocking=True)
        return self.model.logits(h, rows_dev, ctx)

    # ------------------------------------------------------------ lifecycle
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)
