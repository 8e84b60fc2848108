"""RMS norm: x * w / sqrt(mean(x^2) + eps), statistics in 32-bit.

The weight is kept in 32-bit; a zero-centred norm stores w and multiplies by
1 + w, which is formed once at load time (the reference does the same when it
warms its norm cache, src/models/gemma3.zig:908-954).

Interface of a norm part (what a block needs):
  ``forward(h, out, rows=None)``      out = norm(h[rows]) for the 32-bit stream h
  ``residual(h, y, nxt, x_out)``      h += self(y); x_out = nxt(h) if nxt
  ``after_residual(h, y, x_out)``     h += y; x_out = self(h)
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import NormSpec
from .base import ParamSpec, register_norm


class RMSNorm:
    def __init__(self, spec: NormSpec, width: int, dtype: torch.dtype, device: torch.device):
        self.spec, self.width = spec, width
        self.eps = float(spec.eps)
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, spec: NormSpec, width: int) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((width,), "norm", zero_centered=spec.zero_centered)}

    def load(self, tensors: Dict[str, torch.Tensor], device: torch.device) -> None:
        w = tensors["weight"].to(device=device, dtype=torch.float32)
        self.weight = (w + 1.0 if self.spec.zero_centered else w).contiguous()

    def forward(self, h: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        kernels.norm_residual(h, None, None, self.weight, out, eps_next=self.eps, rows=rows)
        return out

    def residual(self, h: torch.Tensor, y: torch.Tensor, nxt, x_out) -> None:
        """h += self(y); x_out = nxt(h) if nxt (one launch when nxt is an RMS norm)."""
        if nxt is None or isinstance(nxt, RMSNorm):
            fused_residual(h, y, self, nxt, x_out)
        else:
            fused_residual(h, y, self, None, None)
            nxt.forward(h, x_out)

    def after_residual(self, h: torch.Tensor, y: torch.Tensor, x_out: torch.Tensor) -> None:
        """h += y; x_out = self(h)."""
        fused_residual(h, y, None, self, x_out)


def fused_residual(h: torch.Tensor, y: torch.Tensor, post: Optional[RMSNorm],
                   nxt: Optional[RMSNorm], x_out: Optional[torch.Tensor]) -> None:
    """h += post(y) (or y); x_out = nxt(h): one launch for RMS norms."""
    kernels.norm_residual(
        h, y, post.weight if post is not None else None,
        nxt.weight if nxt is not None else None, x_out if nxt is not None else None,
        eps_post=post.eps if post is not None else 0.0,
        eps_next=nxt.eps if nxt is not None else 0.0)


register_norm("rmsnorm", RMSNorm)
