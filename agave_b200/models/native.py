"""The C++ host side of a step, for models whose blocks are the standard arrangement.

``NativeStep.build(model)`` describes a loaded ``DecoderModel`` to the CUDA library
(``csrc/host_step.cu``): pointers and sizes of every block, the rotation table kinds, the
cache pools and the run order.  ``run`` then executes a whole step (embedding, every
block, final norm, head) with one call into the library, which makes the dispatch
decisions and launches the kernels itself.  It returns None from ``build`` for a model it
cannot describe (a part registered from outside, a block of another kind, a call that
reads another call's cache, a position encoding added to the stream); such models run
through the Python parts, launch by launch.

Both paths launch the same kernels with the same arguments; ``AGAVE_B200_NATIVE_STEP=0``
turns this one off.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import kernels
from ..config.base import AttentionSpec, GatedFeedForwardSpec
from ..engine.batch import DECODE, PREFILL
from ..parts.attention import AttentionMixer
from ..parts.block import Block
from ..parts.feedforward import GatedFeedForward
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEmbedding

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


class _BlockDesc(ctypes.Structure):
    _fields_ = [(n, _P) for n in ("w_pre_mixer", "w_post_mixer", "w_pre_ffn", "w_post_ffn",
                                  "w_qkv", "w_out", "wq_norm", "wk_norm", "w_gate", "w_up",
                                  "w_down")] + \
               [(n, _F) for n in ("eps", "qk_eps", "scale")] + \
               [(n, _I) for n in ("nh", "nkv", "hd", "window", "rotary_dim", "rope_slot", "ff",
                                  "act")]


class _CacheDesc(ctypes.Structure):
    _fields_ = [("k_pool", _P), ("v_pool", _P), ("page_table", _P), ("max_pages", _I),
                ("page", _I), ("cap", _I), ("pool_pages", _I)]


class _StepDesc(ctypes.Structure):
    _fields_ = [(n, _P) for n in ("tokens", "positions", "seq_index", "cu_seqlens", "slots", "lens",
                                  "workspace", "rows", "logits", "argmax_out",
                                  "decode_counters")] + \
               [("workspace_bytes", ctypes.c_longlong)] + \
               [(n, _I) for n in ("mode", "T", "B", "max_len", "max_new", "n_rows")]


def _ptr(t: Optional[torch.Tensor]):
    return t.data_ptr() if t is not None else None


ENABLED = os.environ.get("AGAVE_B200_NATIVE_STEP", "1") != "0"


def standard_blocks(model) -> bool:
    """Whether every block of the model is the standard arrangement of the library's own
    parts (RMS norms, attention mixer with or without rotation, gated feed-forward), every
    call writes its own cache entry and nothing is added to the stream: what the C++ step
    function and the few-token decode path know how to run."""
    if model.head is None or model.stream_position is not None:
        return False
    if any(not c.writes_cache for c in model.spec.schedule):
        return False
    for b in model.blocks:
        if type(b) is not Block or type(b.mixer) is not AttentionMixer or \
                type(b.ffn) is not GatedFeedForward:
            return False
        if not isinstance(b.mixer.spec, AttentionSpec) or \
                not isinstance(b.ffn.spec, GatedFeedForwardSpec):
            return False
        for n in (b.pre_mixer_norm, b.pre_ffn_norm, b.post_mixer_norm, b.post_ffn_norm):
            if n is not None and type(n) is not RMSNorm:
                return False
        if b.mixer.position is not None and type(b.mixer.position) is not RotaryEmbedding:
            return False
    return type(model.final_norm) is RMSNorm


class NativeStep:
    def __init__(self, handle, lib, model, keep):
        self._handle, self._lib, self.model = handle, lib, model
        self._keep = keep                      # what the library points into
        self._cache_set = False

    def __del__(self):
        try:
            if self._handle:
                self._lib.agv_model_destroy(self._handle)
        except Exception:
            pass

    # ----------------------------------------------------------------- build
    @classmethod
    def build(cls, model) -> Optional["NativeStep"]:
        if not ENABLED or not standard_blocks(model):
            return None
        spec = model.spec
        lib = kernels.library()
        lib.agv_model_create.restype = ctypes.c_void_p
        lib.agv_model_workspace_bytes.restype = ctypes.c_longlong
        handle = lib.agv_model_create(
            kernels.dtype_code(model.dtype), spec.hidden_size, spec.vocab_size,
            _F(spec.embed_scale), _P(model.embed_table.data_ptr()),
            _P(model.final_norm.weight.data_ptr()), _F(model.final_norm.eps),
            _P(model.head.weight.data_ptr()))
        if not handle:
            raise kernels.KernelError(lib.agv_last_error().decode("utf-8", "replace"))
        handle = ctypes.c_void_p(handle)
        ropes = {}
        for b in model.blocks:
            m, s = b.mixer, b.mixer.spec
            slot = -1
            if m.position is not None:
                key = m.position._key
                if key not in ropes:
                    rs = m.position.spec
                    ropes[key] = lib.agv_model_add_rope(handle, ctypes.c_double(rs.theta),
                                                        ctypes.c_double(rs.factor),
                                                        m.position.rotary_dim)
                    if ropes[key] < 0:
                        kernels._check(ropes[key])
                slot = ropes[key]
            d = _BlockDesc(
                w_pre_mixer=_ptr(b.pre_mixer_norm.weight),
                w_post_mixer=_ptr(b.post_mixer_norm.weight) if b.post_mixer_norm else None,
                w_pre_ffn=_ptr(b.pre_ffn_norm.weight),
                w_post_ffn=_ptr(b.post_ffn_norm.weight) if b.post_ffn_norm else None,
                w_qkv=_ptr(m.qkv.weight), w_out=_ptr(m.out.weight),
                wq_norm=_ptr(m.q_norm_weight), wk_norm=_ptr(m.k_norm_weight),
                w_gate=_ptr(b.ffn.gate_up.w_gate), w_up=_ptr(b.ffn.gate_up.w_up),
                w_down=_ptr(b.ffn.down.weight), eps=b.pre_mixer_norm.eps,
                qk_eps=s.qk_norm.eps if s.qk_norm is not None else 0.0, scale=s.scale,
                nh=s.n_heads, nkv=s.n_kv_heads, hd=s.head_dim, window=s.window or 0,
                rotary_dim=m.position.rotary_dim if m.position is not None else 0,
                rope_slot=slot, ff=b.ffn.spec.intermediate_size,
                act=kernels.ACT[b.ffn.spec.activation])
            rc = lib.agv_model_add_block(handle, ctypes.byref(d))
            if rc < 0:
                kernels._check(rc)
        for call in spec.schedule:
            kernels._check(lib.agv_model_add_call(handle, call.block, call.cache))
        return cls(handle, lib, model, keep=None)

    def _set_caches(self, cache) -> None:
        """The cache pools of every entry the run order names (fixed for the cache's life)."""
        for call in self.model.spec.schedule:
            v = cache.kv_view(call.cache)
            d = _CacheDesc(k_pool=v.k_pool.data_ptr(), v_pool=v.v_pool.data_ptr(),
                           page_table=v.page_table.data_ptr(), max_pages=v.page_table.shape[1],
                           page=v.page, cap=v.cap, pool_pages=v.k_pool.shape[0])
            kernels._check(self._lib.agv_model_set_cache(self._handle, call.cache, ctypes.byref(d)))
        self._cache_set = cache

    # ------------------------------------------------------------------- run
    def run(self, ctx, rows: Optional[torch.Tensor], logits: Optional[torch.Tensor] = None,
            argmax_out: Optional[torch.Tensor] = None) -> None:
        """One whole step on torch's current stream: logits [len(rows), V] (32-bit) or, into
        ``argmax_out`` (int32), the index of each row's greatest logit."""
        if self._cache_set is not ctx.cache:
            self._set_caches(ctx.cache)
        mode = 0 if ctx.mode == PREFILL else 1
        n_rows = rows.numel() if rows is not None else 0
        need = self._lib.agv_model_workspace_bytes(self._handle, mode, ctx.n_tokens, ctx.batch,
                                                   ctx.max_len, ctx.max_new, n_rows,
                                                   1 if argmax_out is not None else 0)
        if need < 0:
            kernels._check(int(need))
        ws = torch.empty(int(need), dtype=torch.uint8, device=ctx.device)
        nh = max(b.mixer.spec.n_heads for b in self.model.blocks)
        counters = kernels._decode_counters(ctx.device, ctx.batch * nh)
        d = _StepDesc(tokens=ctx.tokens.data_ptr(), positions=ctx.positions.data_ptr(),
                      seq_index=ctx.seq_index.data_ptr(), cu_seqlens=ctx.cu_seqlens.data_ptr(),
                      slots=ctx.slots.data_ptr(), lens=ctx.lens.data_ptr(),
                      workspace=ws.data_ptr(), rows=_ptr(rows), logits=_ptr(logits),
                      argmax_out=_ptr(argmax_out), decode_counters=counters.data_ptr(),
                      workspace_bytes=int(need), mode=mode, T=ctx.n_tokens, B=ctx.batch,
                      max_len=ctx.max_len, max_new=ctx.max_new, n_rows=n_rows)
        n = ctypes.c_int(0)
        rc = self._lib.agv_model_step(self._handle, ctypes.byref(d), ctypes.byref(n),
                                      kernels._stream())
        kernels._launches += n.value - 1          # (_stream() counted one)
        kernels._check(rc)
