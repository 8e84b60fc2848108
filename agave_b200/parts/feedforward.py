"""Dense gated feed-forward: down(act(gate x) * up x), no biases
(src/models/gemma3.zig:840-872); the activation and the product are the
epilogue of the gate/up kernel.

Interface of a feed-forward part:
  ``param_specs(spec, hidden) -> {local name: ParamSpec}``      (class method)
  ``load(tensors, dtype, device)``
  ``forward(x [T, hidden], ctx) -> y [T, hidden]`` (or ``[S, T, hidden]`` 32-bit
  partial sums, which the norm that follows adds)
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.base import GatedFeedForwardSpec
from .base import ParamSpec, register_feed_forward
from .linear import GatedLinear, Linear


class GatedFeedForward:
    def __init__(self, spec: GatedFeedForwardSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        self.spec, self.hidden_size = spec, hidden_size
        self.gate_up: Optional[GatedLinear] = None
        self.down: Optional[Linear] = None

    @classmethod
    def param_specs(cls, spec: GatedFeedForwardSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        ff = spec.intermediate_size
        return {
            "gate_proj.weight": ParamSpec((ff, hidden_size)),
            "up_proj.weight": ParamSpec((ff, hidden_size)),
            "down_proj.weight": ParamSpec((hidden_size, ff)),
        }

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def mat(name):
            return tensors[name].to(device=device, dtype=dtype).contiguous()
        self.gate_up = GatedLinear(mat("gate_proj.weight"), mat("up_proj.weight"),
                                   self.spec.activation)
        self.down = Linear(mat("down_proj.weight"), role="down")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return self.down.partial(self.gate_up(x))


register_feed_forward("gated_dense", GatedFeedForward)
