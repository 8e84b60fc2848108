"""Rotary position encoding as a table of angles per step.

A position part turns the step's positions into ``(cos, sin)`` tables
``[T, rotary_dim / 2]`` (32-bit); the attention kernels rotate the pairs
(i, i + rotary_dim / 2) of every head with them.  The tables of one spec are
made once per step and shared by all layers that use that spec.  Any encoding
that is a rotation of such pairs fits this interface by giving other tables.

angle = (p / factor) * theta^(-2 i / rotary_dim): src/backend/kernels/cpu/rope.zig:11-27,
src/models/gemma3.zig:884-902.  Angles are formed in 64-bit on the device.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import kernels
from ..config.base import RotarySpec
from .base import register_position


class RotaryEmbedding:
    def __init__(self, spec: RotarySpec, head_dim: int):
        self.spec = spec
        self.rotary_dim = spec.rotary_dim or head_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most "
                             f"head_dim {head_dim}")
        self._key = ("rotary", float(spec.theta), float(spec.factor), self.rotary_dim)

    def tables(self, ctx) -> Tuple[torch.Tensor, torch.Tensor]:
        hit = ctx.rope_tables.get(self._key)
        if hit is None:
            half = self.rotary_dim // 2
            cos = ctx.new(ctx.n_tokens, half, dtype=torch.float32)
            sin = ctx.new(ctx.n_tokens, half, dtype=torch.float32)
            kernels.rope_table(ctx.positions, self.rotary_dim, self.spec.theta, self.spec.factor,
                               cos, sin)
            hit = ctx.rope_tables[self._key] = (cos, sin)
        return hit


register_position("rotary", RotaryEmbedding)
