"""One layer: mixer and feed-forward between norms, over a 32-bit residual stream.

"sandwich" (src/models/gemma3.zig:708-709,824-826,835-836,876-878):
    h += post_mixer_norm(mixer(pre_mixer_norm(h)))
    h += post_ffn_norm(ffn(pre_ffn_norm(h)))
"pre": the same without the two post norms.

The residual sum, the norm of the branch and the norm that feeds the next
branch are one kernel launch, so a block receives its input already normed
(``x``) and returns the input of whatever runs next, normed with that part's
own input norm (``next_norm``; None after the last block).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.base import BlockSpec
from .base import ParamSpec, feed_forward_class, mixer_class, norm_class, register_block
from .norm import fused_residual


class Block:
    def __init__(self, spec: BlockSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if spec.arrangement not in ("sandwich", "pre"):
            raise ValueError(f"unknown block arrangement {spec.arrangement!r}")
        self.spec, self.hidden_size, self.dtype, self.device = spec, hidden_size, dtype, device
        N = norm_class(spec.norm.kind)
        self.sandwich = spec.arrangement == "sandwich"
        self.pre_mixer_norm = N(spec.norm, hidden_size, dtype, device)
        self.pre_ffn_norm = N(spec.norm, hidden_size, dtype, device)
        self.post_mixer_norm = N(spec.norm, hidden_size, dtype, device) if self.sandwich else None
        self.post_ffn_norm = N(spec.norm, hidden_size, dtype, device) if self.sandwich else None
        self.mixer = mixer_class(spec.mixer.kind)(spec.mixer, hidden_size, dtype, device)
        self.ffn = feed_forward_class(spec.feed_forward.kind)(spec.feed_forward, hidden_size,
                                                              dtype, device)

    @classmethod
    def param_specs(cls, spec: BlockSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        N = norm_class(spec.norm.kind)
        names = ["pre_mixer_norm", "pre_ffn_norm"]
        if spec.arrangement == "sandwich":
            names += ["post_mixer_norm", "post_ffn_norm"]
        out: Dict[str, ParamSpec] = {}
        for n in names:
            for k, v in N.param_specs(spec.norm, hidden_size).items():
                out[f"{n}.{k}"] = v
        for k, v in mixer_class(spec.mixer.kind).param_specs(spec.mixer, hidden_size).items():
            out[f"mixer.{k}"] = v
        F = feed_forward_class(spec.feed_forward.kind)
        for k, v in F.param_specs(spec.feed_forward, hidden_size).items():
            out[f"ffn.{k}"] = v
        return out

    @property
    def entry_norm(self):
        """The norm that feeds this block's first branch."""
        return self.pre_mixer_norm

    def cache_request(self):
        return self.mixer.cache_request()

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def sub(prefix):
            n = len(prefix) + 1
            return {k[n:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
        for name in ("pre_mixer_norm", "pre_ffn_norm", "post_mixer_norm", "post_ffn_norm"):
            part = getattr(self, name)
            if part is not None:
                part.load(sub(name), device)
        self.mixer.load(sub("mixer"), dtype, device)
        self.ffn.load(sub("ffn"), dtype, device)

    def forward(self, h: torch.Tensor, x: torch.Tensor, ctx, cache_entry: int,
                writes_cache: bool, next_norm) -> Optional[torch.Tensor]:
        """h: [T, H] 32-bit stream (updated in place); x = pre_mixer_norm(h)."""
        y = self.mixer.forward(x, ctx, cache_entry, writes_cache)
        x2 = ctx.new(*x.shape)
        _join(h, y, self.post_mixer_norm, self.pre_ffn_norm, x2)
        d = self.ffn.forward(x2, ctx)
        x3 = ctx.new(*x.shape) if next_norm is not None else None
        _join(h, d, self.post_ffn_norm, next_norm, x3)
        return x3


register_block("sequential", Block)


def _join(h, y, post, nxt, x_out) -> None:
    """h += post(y) (or y when there is no post norm); x_out = nxt(h) if nxt."""
    if post is not None:
        post.residual(h, y, nxt, x_out)
    elif nxt is not None:
        nxt.after_residual(h, y, x_out)
    else:
        fused_residual(h, y, None, None, None)
