"""The decisions of the generation loop, free of any device.

Requests are served in batches: a batch's prompts run together in one step,
then every live sequence gets one token per step; a sequence that meets a
stop token, its token limit or the end of the cache leaves the batch (its slot
is given back at once), and when the batch is empty the next one starts.
Nothing joins a running batch.

What follows the reference (src/main.zig:2234-2461): the first token comes
from the prompt step's last logits; a stop token ends the sequence and is not
returned (2366-2369); ``max_new_tokens`` bounds the tokens returned.  The
reference's halt after six equal tokens in a row (2400-2407) is a console
heuristic and is not repeated here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from ..cache.book import PAGE, round_up

STOP, LENGTH, CONTEXT, CANCELLED = "stop", "length", "context", "cancelled"


@dataclass
class RequestState:
    index: int
    prompt: List[int]
    max_new: int
    output: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    slot: int = -1
    clamped: bool = False       # max_new was cut to what the cache can hold

    @property
    def done(self) -> bool:
        return self.finish_reason is not None


class GenerationPlan:
    """Which requests form the next batch, and what each sampled token means."""

    def __init__(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 stop_token_ids: Sequence[int], max_batch: int, max_tokens: int,
                 max_seq_len: int):
        if max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")
        if max_batch < 1:
            raise ValueError("max_batch must be >= 1")
        self.stop = frozenset(int(t) for t in stop_token_ids)
        self.max_batch, self.max_tokens, self.max_seq_len = max_batch, max_tokens, max_seq_len
        self.requests: List[RequestState] = []
        for i, p in enumerate(prompts):
            p = [int(t) for t in p]
            if not p:
                raise ValueError(f"prompt {i} is empty")
            if len(p) > max_seq_len:
                raise ValueError(f"prompt {i} has {len(p)} tokens, the cache holds sequences "
                                 f"of at most {max_seq_len}")
            if round_up(len(p), PAGE) > round_up(max_tokens, PAGE):
                raise ValueError(f"prompt {i} has {len(p)} tokens, the cache holds {max_tokens}")
            # a sequence of n positions can be followed by one more sampled token
            room = max_seq_len - len(p) + 1
            self.requests.append(RequestState(i, p, min(max_new_tokens, room),
                                              clamped=max_new_tokens > room))
        self._next = 0
        self.batch: List[RequestState] = []

    # -------------------------------------------------------------- batches
    def _worst_case(self, r: RequestState) -> int:
        # positions the sequence may come to hold: the last sampled token is never fed back
        return round_up(min(self.max_seq_len, len(r.prompt) + max(0, r.max_new - 1)), PAGE)

    def next_batch(self) -> List[RequestState]:
        """Start the next batch (the running one must be empty); [] when all are served."""
        if any(not r.done for r in self.batch):
            raise RuntimeError("the running batch has live sequences")
        self.batch = []
        budget = round_up(self.max_tokens, PAGE)
        used = 0
        while self._next < len(self.requests) and len(self.batch) < self.max_batch:
            r = self.requests[self._next]
            if r.max_new == 0:
                r.finish_reason = LENGTH
                self._next += 1
                continue
            need = self._worst_case(r)
            if used + need > budget:
                if not self.batch:
                    # alone it still does not fit: let it run until the cache ends
                    need = budget - used
                    r.max_new = min(r.max_new, need - len(r.prompt) + 1)
                    r.clamped = True
                else:
                    break
            used += need
            self.batch.append(r)
            self._next += 1
        return list(self.batch)

    def live(self) -> List[RequestState]:
        return [r for r in self.batch if not r.done]

    # --------------------------------------------------------------- tokens
    def accept(self, sampled: Dict[int, int]) -> List[RequestState]:
        """Take the token sampled for each live request (by request index).

        Returns the requests that ended with this token.
        """
        ended = []
        for r in self.live():
            t = int(sampled[r.index])
            if t in self.stop:
                r.finish_reason = STOP
            else:
                r.output.append(t)
                if len(r.output) >= r.max_new:
                    r.finish_reason = CONTEXT if r.clamped else LENGTH
            if r.done:
                ended.append(r)
        return ended

    def cancel(self) -> List[RequestState]:
        """End every request that has not finished (the running batch and those not
        yet started) with the reason "cancelled"; returns the live ones of the batch."""
        ended = self.live()
        for r in self.requests:
            if not r.done:
                r.finish_reason = CANCELLED
        self._next = len(self.requests)
        return ended

    @property
    def finished(self) -> bool:
        return self._next >= len(self.requests) and not self.live()

    def outputs(self) -> List[List[int]]:
        return [r.output for r in self.requests]
