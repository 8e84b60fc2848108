"""Next-token choice on the device.

Options and their meaning are the reference's (src/main.zig:333-338,
src/ops/math.zig:209-372): ``temperature`` 0 is arg max (first index on
ties); otherwise logits are divided by the temperature, cut to the ``top_k``
greatest (0 = off), turned into weights, cut to the ``top_p`` nucleus (1 =
off) and one token is drawn.  ``repeat_penalty`` (1 = off) divides positive
logits of already generated tokens and multiplies the others, from the second
generated token on (src/main.zig:2350-2352).  ``seed`` fixes the draws; the
draw of a sequence depends on (seed, sequence id, number of tokens generated
so far) only, not on the batch it runs in.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels

HISTORY_CAP = 4096        # ids remembered per sequence (src/main.zig:92)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repeat_penalty: float = 1.0
    seed: Optional[int] = None

    def validate(self) -> "SamplingParams":
        # the reference's own checks (src/main.zig:555-573)
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if self.repeat_penalty <= 0:
            raise ValueError("repeat_penalty must be > 0")
        return self

    @property
    def greedy(self) -> bool:
        return self.temperature == 0

    def resolved_seed(self) -> int:
        return self.seed if self.seed is not None else time.time_ns() & 0xFFFFFFFFFFFF


class Sampler:
    """Holds the per-slot history and launches the sampling kernels."""

    def __init__(self, n_slots: int, device: torch.device):
        self.device = device
        self.hist = torch.zeros((n_slots, HISTORY_CAP), dtype=torch.int32, device=device)
        self.hist_len = torch.zeros((n_slots,), dtype=torch.int32, device=device)

    def reset(self, slot: int) -> None:
        self.hist_len[slot] = 0

    def note_inputs(self, tokens: torch.Tensor, slots: torch.Tensor) -> None:
        """A decode step's input tokens are the tokens generated the step before."""
        kernels.history_append(tokens, slots, self.hist, self.hist_len)

    def choose(self, logits: torch.Tensor, out: torch.Tensor, params: SamplingParams, seed: int,
               slots: torch.Tensor, seq_ids: torch.Tensor, steps: torch.Tensor,
               penalise: bool, dev_params: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out[b] = token chosen from logits[b]; logits may be changed in place.

        With ``dev_params`` (``kernels.sampling_words`` on the device) the
        temperature, top_k, top_p, seed and penalty are read from there when the
        kernels run; ``params`` then only says which kernels are launched (greedy
        or not, penalty or not), so a recording serves every other setting."""
        if penalise and params.repeat_penalty != 1.0:
            kernels.repeat_penalty(logits, slots, self.hist, self.hist_len, params.repeat_penalty,
                                   dev_params)
        if params.greedy:
            kernels.argmax(logits, out)
        else:
            kernels.sample(logits, out, params.temperature, params.top_k, params.top_p, seed,
                           seq_ids, steps, dev_params)
        return out
