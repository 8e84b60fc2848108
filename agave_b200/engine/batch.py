"""What one step hands to every layer.

A step is either the whole prompts of a batch (every sequence starts at
position 0; lengths differ) or one new token for each sequence of a batch.
The tokens of all sequences lie on one ragged axis of T tokens; the arrays
below say whose each token is and where it stands.  All arrays are int32 on
the device and are the only per-step inputs of the kernels, so a decode step
whose arrays live in fixed buffers can be replayed as a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch

PREFILL, DECODE = "prefill", "decode"


class Cancelled(RuntimeError):
    """A step was stopped between two blocks because its cancel flag was set
    (the reference checks its flag at the same place, src/models/gemma3.zig:342,435)."""


@dataclass
class StepContext:
    mode: str                     # PREFILL or DECODE
    n_tokens: int                 # T
    batch: int                    # B (padding entries included)
    tokens: torch.Tensor          # [T]
    positions: torch.Tensor       # [T] position of each token in its sequence
    seq_index: torch.Tensor       # [T] batch entry of each token
    cu_seqlens: torch.Tensor      # [B + 1] first token of each entry on the ragged axis
    slots: torch.Tensor           # [B] cache slot of each entry; negative = padding
    lens: torch.Tensor            # [B] sequence length after this step
    max_len: int                  # host copy of the greatest length after this step
    max_new: int                  # host copy of the greatest number of tokens an entry brings
    cache: object                 # agave_b200.cache.Cache
    dtype: torch.dtype
    device: torch.device
    # per-step scratch shared between layers
    cancel: object = None         # a threading.Event (or None): set = stop between blocks
    lens_host: object = None      # the lengths on the host, when per-operation timing wants them
    rope_tables: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)
    step_kv: Dict[int, Tuple] = field(default_factory=dict)

    def new(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)
