"""Grouped-query softmax attention over the paged cache, as a mixer part.

Interface of a mixer part (what a block needs):
  ``param_specs(spec, hidden) -> {local name: ParamSpec}``      (class method)
  ``cache_request() -> KVRequest | StateRequest | None``
  ``load(tensors, dtype, device)``
  ``forward(x [T, hidden], ctx, cache_entry, writes_cache) -> y [T, hidden]``
  (y may also be ``[S, T, hidden]`` 32-bit partial sums; the norm that follows
  adds them)

Order of operations (src/models/gemma3.zig:714-820): q, k, v projections (one
fused product here), per-head RMS norm of q and k, rotation, store of k and v,
attention with the spec's scale and window, output projection.

Prompts are attended from the step's own keys and values (every sequence of a
prompt step starts at position 0), so a window ring never has to hold a whole
prompt; decoding attends from the cache after the new key is stored (where the
sizes allow, the decode attention kernel takes the projection's partial sums and does
the norm, the rotation and that store itself).  A call
that does not write the cache reads what the owning call stored: during a
prompt step through ``ctx.step_kv``, during decoding through the cache.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import AttentionSpec
from ..engine.batch import DECODE, PREFILL
from .base import KVRequest, ParamSpec, position_class, register_mixer
from .linear import Linear


class AttentionMixer:
    def __init__(self, spec: AttentionSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.spec, self.hidden_size, self.dtype, self.device = spec, hidden_size, dtype, device
        self.position = (position_class(spec.position.kind)(spec.position, spec.head_dim)
                         if spec.position is not None else None)
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.q_norm_weight = self.k_norm_weight = None

    @classmethod
    def param_specs(cls, spec: AttentionSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        q, kv = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        p = {
            "q_proj.weight": ParamSpec((q, hidden_size)),
            "k_proj.weight": ParamSpec((kv, hidden_size)),
            "v_proj.weight": ParamSpec((kv, hidden_size)),
            "o_proj.weight": ParamSpec((hidden_size, q)),
        }
        if spec.qk_norm is not None:
            zc = spec.qk_norm.zero_centered
            p["q_norm.weight"] = ParamSpec((spec.head_dim,), "norm", zero_centered=zc)
            p["k_norm.weight"] = ParamSpec((spec.head_dim,), "norm", zero_centered=zc)
        return p

    def cache_request(self):
        return KVRequest(self.spec.n_kv_heads, self.spec.head_dim, self.spec.window)

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def mat(name):
            return tensors[name].to(device=device, dtype=dtype)
        # one product for q | k | v: rows of q first, then k, then v
        self.qkv = Linear(torch.cat([mat("q_proj.weight"), mat("k_proj.weight"),
                                     mat("v_proj.weight")], dim=0).contiguous(), role="qkv")
        self.out = Linear(mat("o_proj.weight").contiguous(), role="out_proj")
        if self.spec.qk_norm is not None:
            add = 1.0 if self.spec.qk_norm.zero_centered else 0.0
            self.q_norm_weight = (tensors["q_norm.weight"].to(device=device, dtype=torch.float32)
                                  + add).contiguous()
            self.k_norm_weight = (tensors["k_norm.weight"].to(device=device, dtype=torch.float32)
                                  + add).contiguous()

    def forward(self, x: torch.Tensor, ctx, cache_entry: int, writes_cache: bool) -> torch.Tensor:
        s = self.spec
        nh, nkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
        T = x.shape[0]
        cos = sin = None
        rotary_dim = 0
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            rotary_dim = self.position.rotary_dim
        view = ctx.cache.kv_view(cache_entry)
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        window = s.window or 0
        if ctx.mode == PREFILL and kernels.qkv_prefill_supported(x, self.qkv.weight, hd,
                                                                 rotary_dim):
            # a prompt step on the tensor cores: norm, rotation, the cache store and the
            # transposed values are the epilogue of the q/k/v product
            qkv = ctx.new(T, (nh + 2 * nkv) * hd)
            vt = None
            if writes_cache and kernels.attention_prefill_wants_transposed_values(qkv, hd):
                vt = kernels.prefill_values_scratch(T, ctx.batch, nkv, hd, qkv.device)
            pools = dict(k_pool=view.k_pool, v_pool=view.v_pool, page_table=view.page_table,
                         slots=ctx.slots, lens=ctx.lens, page=view.page,
                         cap=view.cap) if writes_cache else {}
            kernels.qkv_prefill(x, self.qkv.weight, qkv, nh, nkv, hd, self.q_norm_weight,
                                self.k_norm_weight, eps, cos, sin, ctx.positions, ctx.seq_index,
                                vt=vt, cu_seqlens=ctx.cu_seqlens, **pools)
            return self._attend_prompt(qkv, vt, ctx, cache_entry, writes_cache, window)
        proj = self.qkv.partial(x, cheap_sum=True)
        part = proj if proj.dim() == 3 else None
        if (ctx.mode == DECODE and part is not None and
                kernels.attention_decode_fused_supported(self.dtype, hd, rotary_dim)):
            # decoding: norm, rotation and the store of the new key and value happen inside
            # the attention kernel, on the projection's partial sums
            out = ctx.new(T, nh * hd)
            kernels.attention_decode_fused(part, self.q_norm_weight, self.k_norm_weight, eps, cos,
                                           sin, writes_cache, out, view, ctx, nh, nkv, hd, s.scale,
                                           window)
            return self.out.partial(out)
        qkv = proj if part is None else ctx.new(T, (nh + 2 * nkv) * hd)
        if writes_cache:
            # a prompt step on the tcgen05 attention kernel reads the values transposed:
            # the same launch writes that copy
            vt = None
            if ctx.mode == PREFILL and kernels.attention_prefill_wants_transposed_values(qkv, hd):
                vt = kernels.prefill_values_scratch(T, ctx.batch, nkv, hd, qkv.device)
            kernels.qk_norm_rope_store(
                qkv, nh, nkv, hd, self.q_norm_weight, self.k_norm_weight, eps, cos, sin,
                rotary_dim, ctx.positions, view.k_pool, view.v_pool, view.page_table, ctx.slots,
                ctx.lens, ctx.seq_index, view.page, view.cap, partial=part, vt=vt,
                cu_seqlens=ctx.cu_seqlens, max_len=ctx.max_new)
        else:
            kernels.qk_norm_rope_store(qkv, nh, nkv, hd, self.q_norm_weight, self.k_norm_weight,
                                       eps, cos, sin, rotary_dim, ctx.positions, partial=part)
        if ctx.mode == PREFILL:
            return self._attend_prompt(qkv, vt if writes_cache else None, ctx, cache_entry,
                                       writes_cache, window)
        out = ctx.new(T, nh * hd)
        kernels.attention_decode(qkv[:, :nh * hd], out, view, ctx, nh, nkv, hd, s.scale, window)
        return self.out.partial(out)

    def _attend_prompt(self, qkv: torch.Tensor, vt, ctx, cache_entry: int, writes_cache: bool,
                       window: int) -> torch.Tensor:
        """Prompt attention from the step's own keys and values, then the output projection."""
        s = self.spec
        nh, nkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
        if writes_cache:
            k = qkv[:, nh * hd:(nh + nkv) * hd]
            v = qkv[:, (nh + nkv) * hd:]
            ctx.step_kv[cache_entry] = (k, v, vt)
        else:
            k, v, vt = ctx.step_kv[cache_entry]
        out = ctx.new(qkv.shape[0], nh * hd)
        kernels.attention_prefill(qkv[:, :nh * hd], k, v, out, ctx, nh, nkv, hd, s.scale, window,
                                  vt=vt)
        return self.out.partial(out)


register_mixer("attention", AttentionMixer)
