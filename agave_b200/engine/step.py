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

from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from ..cache import Cache, CacheError
from .batch import DECODE, PREFILL, Cancelled, StepContext


class StepError(ValueError):
    pass


PROMPT_GRAPHS = 4             # recorded prompt steps kept
PROMPT_GRAPH_ROWS = 64        # with at most this many wanted places
PROMPT_GRAPH_TOKENS = 16384   # and this many tokens


class _PromptGraph:
    """A recorded prompt step: packed step arrays in, logits out."""
    host: torch.Tensor
    dev: torch.Tensor
    logits: torch.Tensor
    graph: "torch.cuda.CUDAGraph"
    copied: "torch.cuda.Event"


class Runner:
    """A model with its cache and its recorded prompt steps; owns nothing else."""

    def __init__(self, model, max_tokens: int, max_seq_len: int, n_slots: int,
                 use_graphs: bool = True):
        self.use_graphs = use_graphs
        self._prompt_graphs: "OrderedDict[tuple, _PromptGraph]" = OrderedDict()
        self._prompt_seen: dict = {}
        self.model = model
        self.device, self.dtype = model.device, model.dtype
        self.cache = Cache(model.cache_requests(), max_tokens, max_seq_len, n_slots,
                           model.dtype, model.device)
        self.cancel_flag = None        # a threading.Event an eager step checks between blocks
        self.vocab_size = model.spec.vocab_size

    # ------------------------------------------------------------- contexts
    def _plan(self, entries: Sequence[Tuple[int, Sequence[int]]]):
        """Check a batch and reserve its cache room; the step's arrays on the host."""
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
        reserved = []
        try:
            for s, st, c in zip(slots.tolist(), starts.tolist(), counts.tolist()):
                if s >= 0:
                    self.cache.reserve(s, st + c)
                    reserved.append(s)
        except CacheError:
            # the step does not run: what its earlier sequences reserved goes back
            for s in reserved:
                self.cache.trim(s)
            raise
        self.cache.flush()
        T = int(counts.sum())
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(counts, out=cu[1:])
        seq_index = np.repeat(np.arange(B, dtype=np.int64), counts)
        positions = np.arange(T, dtype=np.int64) - cu[:-1][seq_index] + starts[seq_index]
        lens = np.where(real, starts + counts, 0)
        return dict(mode=mode, T=T, B=B, tokens=tokens, positions=positions, seq_index=seq_index,
                    cu=cu, slots=slots, lens=lens, max_len=int(lens.max()),
                    max_new=int(counts.max()))

    @staticmethod
    def _packed_size(T: int, B: int, n_rows: int) -> int:
        return 3 * T + 3 * B + 1 + n_rows

    def _fill(self, plan, rows: Sequence[int], host: torch.Tensor) -> None:
        T, B = plan["T"], plan["B"]
        a = host.numpy()
        a[:T] = plan["tokens"]
        a[T:2 * T] = plan["positions"]
        a[2 * T:3 * T] = plan["seq_index"]
        o = 3 * T
        a[o:o + B + 1] = plan["cu"]
        a[o + B + 1:o + 2 * B + 1] = plan["slots"]
        a[o + 2 * B + 1:o + 3 * B + 1] = plan["lens"]
        if len(rows):
            a[o + 3 * B + 1:] = rows

    def _context_on(self, plan, dev: torch.Tensor) -> Tuple[StepContext, torch.Tensor]:
        """The step's context over a packed device buffer, and the wanted rows."""
        T, B = plan["T"], plan["B"]
        o = 3 * T
        ctx = StepContext(mode=plan["mode"], n_tokens=T, batch=B, tokens=dev[:T],
                          positions=dev[T:2 * T], seq_index=dev[2 * T:3 * T],
                          cu_seqlens=dev[o:o + B + 1], slots=dev[o + B + 1:o + 2 * B + 1],
                          lens=dev[o + 2 * B + 1:o + 3 * B + 1], max_len=plan["max_len"],
                          max_new=plan["max_new"], cache=self.cache, dtype=self.dtype,
                          device=self.device)
        return ctx, dev[o + 3 * B + 1:]

    def context(self, entries: Sequence[Tuple[int, Sequence[int]]]) -> StepContext:
        """Check a batch, reserve its cache room and build its device arrays.

        ``entries``: (slot, tokens) per sequence; slot -1 with one token is a
        padding entry of a decode batch.
        """
        plan = self._plan(entries)
        host = torch.empty(self._packed_size(plan["T"], plan["B"], 0), dtype=torch.int32,
                           pin_memory=True)
        self._fill(plan, (), host)
        return self._context_on(plan, host.to(self.device, non_blocking=True))[0]

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

        A prompt step whose sizes (tokens, sequences, greatest length, wanted
        places) were seen before runs from a recorded CUDA graph: the kernels
        read lengths, positions and page tables from device arrays, so only these
        four numbers are fixed in a recording.
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
        plan = self._plan(entries)
        T, B = plan["T"], plan["B"]
        key = (T, B, plan["max_len"], len(rows))
        graph = None
        timed = kernels._perf is not None      # operations are timed launch by launch
        if (self.use_graphs and not timed and plan["mode"] == PREFILL
                and 0 < len(rows) <= PROMPT_GRAPH_ROWS and T <= PROMPT_GRAPH_TOKENS):
            graph = self._prompt_graphs.get(key)
            if graph is None and self._prompt_seen.get(key, 0) >= 1:
                try:
                    graph = self._record_prompt(plan, rows, key)
                except RuntimeError:
                    # a part that cannot be recorded (one that reads device data on the
                    # host, say): these sizes keep running launch by launch
                    torch.cuda.synchronize()
                    self._prompt_seen[key] = -(1 << 60)
            self._prompt_seen[key] = self._prompt_seen.get(key, 0) + 1
            if len(self._prompt_seen) > 4096:
                self._prompt_seen.clear()
        if graph is not None:
            self._prompt_graphs.move_to_end(key)
            graph.copied.synchronize()       # the staging buffer's last copy has been made
            self._fill(plan, rows, graph.host)
            graph.dev.copy_(graph.host, non_blocking=True)
            graph.copied.record()
            graph.graph.replay()
            self.commit(entries)
            return graph.logits.clone()
        host = torch.empty(self._packed_size(T, B, len(rows)), dtype=torch.int32, pin_memory=True)
        self._fill(plan, rows, host)
        ctx, rows_dev = self._context_on(plan, host.to(self.device, non_blocking=True))
        ctx.cancel = self.cancel_flag
        if timed:
            ctx.lens_host = plan["lens"]
            kernels._perf.n_tokens += T
        try:
            logits = self.model.run_step(ctx, rows_dev if rows else None)
        except Cancelled:
            # nothing is committed: lengths stay, the room reserved for the step goes back
            for s, _ in entries:
                if s >= 0:
                    self.cache.trim(s)
            raise
        self.commit(entries)
        if not rows:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        return logits

    def _record_prompt(self, plan, rows: Sequence[int], key) -> "_PromptGraph":
        """Record the prompt step of these sizes.  Recording runs nothing; the caller
        replays it.  The oldest recording goes when there are too many."""
        g = _PromptGraph()
        n = self._packed_size(plan["T"], plan["B"], len(rows))
        g.host = torch.empty(n, dtype=torch.int32, pin_memory=True)
        g.dev = torch.zeros(n, dtype=torch.int32, device=self.device)
        self._fill(plan, rows, g.host)
        g.dev.copy_(g.host)
        g.copied = torch.cuda.Event()
        g.copied.record()
        torch.cuda.synchronize()
        g.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g.graph):
            ctx, rows_dev = self._context_on(plan, g.dev)
            g.logits = self.model.run_step(ctx, rows_dev)
        while len(self._prompt_graphs) >= PROMPT_GRAPHS:
            self._prompt_graphs.popitem(last=False)
        self._prompt_graphs[key] = g
        return g

    # ------------------------------------------------------------ lifecycle
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)
