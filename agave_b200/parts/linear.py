"""Projections: a weight [out, in] and the kernel choice for it.

The 32-bit path always runs the FFMA kernel (one dot product per output, in
ascending k: a token's result does not depend on its company at all).  The
bfloat16 path runs the tcgen05 kernel when the shape qualifies and otherwise
the FFMA kernel on bfloat16 data.  On the tcgen05 path the number of ranges K
is cut into follows the number of tokens, so a token's 32-bit sums are added in
an order that depends on the batch size: equal up to rounding, not bit for bit.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


class Linear:
    def __init__(self, weight: torch.Tensor, role: str = "linear"):
        assert weight.dim() == 2 and weight.is_contiguous()
        self.weight = weight
        self.role = role               # the operation's name in per-operation timing
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype,
                              device=x.device)
        kernels.linear(x, self.weight, out, op=self.role)
        return out

    def partial(self, x: torch.Tensor, cheap_sum: bool = False) -> torch.Tensor:
        """x w^T for a consumer that sums over a leading axis itself: [S, T, N]
        32-bit partial sums over ranges of K on the tensor-core path (S may be
        1), else the plain [T, N] result.  ``cheap_sum``: the consumer adds the
        partial sums in loads it makes anyway, so more of them are welcome."""
        return kernels.linear_partial(x, self.weight, cheap_sum, op=self.role)


class GatedLinear:
    """act(x wg^T) * (x wu^T) in one kernel."""

    def __init__(self, w_gate: torch.Tensor, w_up: torch.Tensor, activation: str,
                 role: str = "gate_up"):
        assert w_gate.shape == w_up.shape
        self.w_gate, self.w_up, self.activation, self.role = w_gate, w_up, activation, role
        self.out_features, self.in_features = w_gate.shape

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=x.dtype, device=x.device)
        kernels.linear(x, self.w_gate, out, w2=self.w_up, activation=self.activation,
                       op=self.role)
        return out
