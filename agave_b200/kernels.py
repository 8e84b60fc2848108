"""Python face of the CUDA library: one function per exported kernel launcher.

Each function takes torch CUDA tensors, checks what the C side cannot see
(device, dtype, contiguity), and launches on torch's current stream, so the
calls can be recorded into a CUDA graph.  There is no fallback: without the
compiled library, or on a tensor that is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from . import perf as _perf_mod
from .csrc import build as _build

F32, BF16 = 0, 1
ACT = {"gelu_tanh": 0, "silu": 1}

_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The loaded CUDA library (compiled on first use)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.library_path()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"the CUDA library {path} could not be loaded: {e}") from None
                lib.agv_last_error.restype = ctypes.c_char_p
                lib.agv_attention_prefill_tc_vt_cols.restype = ctypes.c_longlong
                if os.environ.get("AGAVE_B200_DEPENDENT_LAUNCH", "1") == "0":
                    # kernels then start only after the one before has ended, which
                    # makes per-kernel durations in a profiler additive
                    lib.agv_set_dependent_launch(0)
                _lib = lib
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(library().agv_last_error().decode("utf-8", "replace"))


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} has no kernels (float32 and bfloat16 do)")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("a tensor handed to a CUDA kernel is not on a CUDA device")
    return ctypes.c_void_p(t.data_ptr())


NVTX = os.environ.get("AGAVE_B200_NVTX", "0") == "1"     # name every launch for a profiler
_launches = 0
_perf = None          # an active agave_b200.perf.PerfCounters, or None


def _span(op: str, nbytes: int = 0, flops: int = 0):
    """A timing span around one launch while operations are being timed."""
    if _perf is None or torch.cuda.is_current_stream_capturing():
        # (a recording holds no timing events)
        return _perf_mod.NvtxSpan(op) if NVTX else _perf_mod.NULL_SPAN
    return _perf.span(op, nbytes, flops)


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)



_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    # called exactly once per kernel launch: the count is what bench.py reports
    global _launches
    _launches += 1
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))     # the same handle, without the
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)   # Stream object around it


def launch_count() -> int:
    """Kernels of this library launched (or recorded into a graph) so far."""
    return _launches


def _dense(t: torch.Tensor, what: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")


def _f32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{what} must be float32, got {t.dtype}")


def device_arch() -> int:
    rc = library().agv_device_arch()
    if rc < 0:
        _check(rc)
    return rc


# ------------------------------------------------------------------ embedding
def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """out[t, :] = table[tokens[t], :] * scale, 32-bit."""
    _i32(tokens, "tokens"); _f32(out, "out"); _dense(table, "table"); _dense(out, "out")
    T, (V, H) = tokens.numel(), table.shape
    assert out.shape == (T, H)
    with _span("embed", T * H * table.element_size() + _nbytes(out)):
        _check(library().agv_embed(_ptr(tokens), _ptr(table), dtype_code(table.dtype), _ptr(out),
                                   T, H, V, ctypes.c_float(scale), _stream()))


def rope_table(positions: torch.Tensor, rotary_dim: int, theta: float, factor: float,
               cos: torch.Tensor, sin: torch.Tensor) -> None:
    """cos, sin [T, rotary_dim/2] of (p / factor) * theta^(-2i/rotary_dim)."""
    _i32(positions, "positions"); _f32(cos, "cos"); _f32(sin, "sin")
    T = positions.numel()
    assert cos.shape == (T, rotary_dim // 2) and sin.shape == cos.shape
    with _span("rope_table", _nbytes(cos, sin)):
        _check(library().agv_rope_table(_ptr(positions), _ptr(cos), _ptr(sin), T, rotary_dim,
                                        ctypes.c_double(theta), ctypes.c_double(factor), _stream()))


# ---------------------------------------------------------------------- norms
def norm_residual(h: Optional[torch.Tensor], y: Optional[torch.Tensor],
                  w_post: Optional[torch.Tensor], w_next: Optional[torch.Tensor],
                  x: Optional[torch.Tensor], eps_post: float = 0.0, eps_next: float = 0.0,
                  rows: Optional[torch.Tensor] = None, add_residual: bool = True) -> None:
    """The norm family in one launch.

    y None:  x = norm(h[rows]; w_next)               (rows optional)
    else:    b = y (summed over a leading split axis if y is 3-D);
             b = norm(b; w_post) if w_post; h += b if add_residual;
             x = norm(h or b; w_next) if w_next, else x = b if x is given.
    h is the 32-bit residual stream [R, H]; w_* are 32-bit and already hold
    1 + w where the norm is zero-centred.
    """
    _f32(h, "h"); _f32(w_post, "w_post"); _f32(w_next, "w_next"); _i32(rows, "rows")
    n_splits, split_stride, y_code = 1, 0, F32
    if y is not None:
        _dense(y, "y")
        y_code = dtype_code(y.dtype)
        if y.dim() == 3:
            n_splits, R, H = y.shape
            split_stride = R * H
        else:
            R, H = y.shape
    else:
        H = h.shape[-1]
        R = rows.numel() if rows is not None else h.shape[0]
    if h is not None:
        _dense(h, "h")
    x_code = F32
    if x is not None:
        _dense(x, "x")
        x_code = dtype_code(x.dtype)
        assert x.shape == (R, H), (x.shape, R, H)
    with _span("norm", _nbytes(y, x) + (R * H * 4 * (2 if y is not None and add_residual else 1)
                                         if h is not None else 0)):
        _check(library().agv_norm_residual(
            _ptr(h), _ptr(y), y_code, n_splits, ctypes.c_longlong(split_stride), _ptr(w_post),
            _ptr(w_next), _ptr(x), x_code, _ptr(rows), R, H, ctypes.c_float(eps_post),
            ctypes.c_float(eps_next), 1 if (add_residual and y is not None) else 0, _stream()))


# ------------------------------------------------------------ matrix products
def _linear_cost(x, w, w2, out):
    """(bytes, flops) of a projection: weights and operands once, 2 T N K flops."""
    T, K = x.shape
    N = w.shape[0]
    n = 2 if w2 is not None else 1
    return (n * N * K * w.element_size() + T * K * x.element_size() + _nbytes(out),
            2 * n * T * N * K)


def linear_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                w2: Optional[torch.Tensor] = None, activation: str = "gelu_tanh",
                op: str = "linear") -> None:
    """out = x w^T, or act(x w^T) * (x w2^T); FFMA kernel (the 32-bit path)."""
    M, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and out.shape == (M, N)
    assert x.stride(1) == 1 and out.stride(1) == 1
    _dense(w, "w")
    if w2 is not None:
        _dense(w2, "w2")
        assert w2.shape == w.shape and w2.dtype == w.dtype
    if x.dtype != w.dtype:
        raise KernelError(f"linear: input {x.dtype} and weight {w.dtype} differ")
    with _span(op, *_linear_cost(x, w, w2, out)):
        _check(library().agv_linear_simt(
            _ptr(x), _ptr(w), _ptr(w2), _ptr(out), M, N, K, ctypes.c_longlong(x.stride(0)),
            ctypes.c_longlong(out.stride(0)), dtype_code(x.dtype), dtype_code(out.dtype),
            ACT[activation], _stream()))


# ------------------------------------------------------------------ attention
def qk_norm_rope_store(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                       wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                       positions: Optional[torch.Tensor],
                       k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
                       page_table: Optional[torch.Tensor] = None,
                       slots: Optional[torch.Tensor] = None, lens: Optional[torch.Tensor] = None,
                       seq_index: Optional[torch.Tensor] = None, page: int = 0,
                       cap: int = 0, partial: Optional[torch.Tensor] = None,
                       vt: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None,
                       max_len: int = 0) -> None:
    """In place on qkv [T, (nh + 2 nkv) * hd]: per-head norm of q and k, rotation,
    and (if pools are given) the store of k and v rows into the paged cache.
    ``partial`` [S, T, (nh + 2 nkv) * hd] (32-bit partial sums of the projection)
    replaces qkv as the input; qkv then only receives the result.  ``vt`` (from
    ``prefill_values_scratch``) also receives the values transposed, for the prompt
    attention; that needs seq_index, positions, cu_seqlens and the greatest length."""
    T = qkv.shape[0]
    n_splits = 0
    if partial is not None:
        _f32(partial, "partial"); _dense(partial, "partial")
        assert partial.dim() == 3 and partial.shape[1] == T
        assert partial.shape[2] == (n_heads + 2 * n_kv_heads) * head_dim
        n_splits = partial.shape[0]
    assert qkv.stride(1) == 1
    _f32(wq, "wq"); _f32(wk, "wk"); _f32(cos, "cos"); _f32(sin, "sin")
    for t, n in ((positions, "positions"), (page_table, "page_table"), (slots, "slots"),
                 (lens, "lens"), (seq_index, "seq_index")):
        _i32(t, n)
    if k_pool is not None:
        _dense(k_pool, "k_pool"); _dense(v_pool, "v_pool")
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
    max_pages = page_table.shape[1] if page_table is not None else 0
    n_seq = 0
    if vt is not None:
        _dense(vt, "vt"); _i32(cu_seqlens, "cu_seqlens")
        assert vt.dtype == torch.bfloat16 and vt.shape[0] == n_kv_heads * head_dim
        n_seq = cu_seqlens.numel() - 1
    with _span("qk_norm_rope", 2 * _nbytes(qkv) + _nbytes(partial, vt)):
        _check(library().agv_qk_norm_rope_store(
            _ptr(qkv), dtype_code(qkv.dtype), ctypes.c_longlong(qkv.stride(0)), _ptr(partial),
            n_splits, T, n_heads, n_kv_heads, head_dim, _ptr(wq), _ptr(wk), ctypes.c_float(eps),
            _ptr(cos), _ptr(sin), rotary_dim, _ptr(positions), _ptr(k_pool), _ptr(v_pool),
            _ptr(page_table), _ptr(slots), _ptr(lens), _ptr(seq_index), max_pages, page, cap,
            _ptr(vt), ctypes.c_longlong(vt.shape[1] if vt is not None else 0), _ptr(cu_seqlens),
            n_seq, max_len, _stream()))


_FUSED_QKV = os.environ.get("AGAVE_B200_FUSED_QKV_PREFILL", "1") != "0"


def qkv_prefill_supported(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int) -> bool:
    """Whether ``qkv_prefill`` takes a prompt step of these sizes: bfloat16 on the tensor
    cores, head sizes 64, 128 or 256 rotated whole or not at all, and enough tiles (128
    tokens x 256 weight rows) that a CTA works on several: the epilogue of one tile then
    runs under the products of the next.  With about one tile per CTA it is exposed, and
    the plain product followed by the norm / rotation / store kernel, whose thousands of
    warps hide their memory trips, is faster (1B sizes, 2,048 tokens: 149 against 156 us a
    layer; 4B: 441 against 433; 27B: 1,624 against 1,612).  ``AGAVE_B200_FUSED_QKV_PREFILL``
    = 0 turns it off, = 2 takes it whenever the sizes allow."""
    if not _FUSED_QKV or x.shape[0] <= 128 or not linear_tc_supported(x, w):
        return False
    tiles = ((w.shape[0] + 255) // 256) * ((x.shape[0] + 127) // 128)
    if tiles * 2 < 3 * n_sms() and os.environ.get("AGAVE_B200_FUSED_QKV_PREFILL") != "2":
        return False
    return (bool(
        library().agv_qkv_prefill_tc_supported(head_dim, rotary_dim, w.shape[1],
                                               ctypes.c_longlong(x.stride(0)),
                                               ctypes.c_longlong(w.shape[0]))))


def qkv_prefill(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, n_heads: int, n_kv_heads: int,
                head_dim: int, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
                cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                positions: torch.Tensor, seq_index: torch.Tensor,
                k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                lens: Optional[torch.Tensor] = None, page: int = 0, cap: int = 0,
                vt: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None) -> None:
    """qkv [T, (nh + 2 nkv) * hd] = x w^T with the per-head norm of q and k, the rotation, the
    store of k and v into the paged cache (if pools are given) and the transposed copy of
    the values (if ``vt`` is given) all done in the product's epilogue."""
    T, K = x.shape
    N = (n_heads + 2 * n_kv_heads) * head_dim
    assert w.shape == (N, K) and qkv.shape == (T, N) and qkv.dtype == torch.bfloat16
    assert x.stride(1) == 1 and qkv.stride(1) == 1
    _dense(w, "w")
    _f32(wq, "wq"); _f32(wk, "wk"); _f32(cos, "cos"); _f32(sin, "sin")
    for t, n in ((positions, "positions"), (page_table, "page_table"), (slots, "slots"),
                 (lens, "lens"), (seq_index, "seq_index"), (cu_seqlens, "cu_seqlens")):
        _i32(t, n)
    if cos is not None:
        _dense(cos, "cos"); _dense(sin, "sin")
        assert cos.shape == (T, head_dim // 2)
    if k_pool is not None:
        _dense(k_pool, "k_pool"); _dense(v_pool, "v_pool")
        assert k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16
    if vt is not None:
        _dense(vt, "vt")
        assert vt.dtype == torch.bfloat16 and vt.shape[0] == n_kv_heads * head_dim
    max_pages = page_table.shape[1] if page_table is not None else 0
    with _span("qkv", *_linear_cost(x, w, None, qkv)):
        _check(library().agv_qkv_prefill_tc(
            _ptr(x), _ptr(w), T, K, ctypes.c_longlong(x.stride(0)), _ptr(qkv),
            ctypes.c_longlong(qkv.stride(0)), n_heads, n_kv_heads, head_dim, _ptr(wq), _ptr(wk),
            ctypes.c_float(eps), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(k_pool), _ptr(v_pool),
            _ptr(page_table), _ptr(slots), _ptr(lens), _ptr(seq_index), max_pages, page, cap,
            _ptr(vt), ctypes.c_longlong(vt.shape[1] if vt is not None else 0), _ptr(cu_seqlens),
            _stream()))


def attention_prefill_simt(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                           positions: torch.Tensor, seq_index: torch.Tensor,
                           cu_seqlens: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                           scale: float, window: int) -> None:
    """Prompts that start at 0; q [T, nh*hd], k, v [T, nkv*hd] row-strided views."""
    T = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    assert k.stride(0) == v.stride(0)
    _dense(out, "out")
    _i32(positions, "positions"); _i32(seq_index, "seq_index"); _i32(cu_seqlens, "cu_seqlens")
    _check(library().agv_attention_prefill_simt(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(k), _ptr(v),
        ctypes.c_longlong(k.stride(0)), _ptr(out), dtype_code(q.dtype), _ptr(positions),
        _ptr(seq_index), _ptr(cu_seqlens), T, n_heads, n_kv_heads, head_dim,
        ctypes.c_float(scale), window, _stream()))


def attention_paged_simt(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor,
                         v_pool: torch.Tensor, page_table: torch.Tensor, slots: torch.Tensor,
                         positions: torch.Tensor, seq_index: torch.Tensor, page: int, cap: int,
                         n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                         window: int) -> None:
    """Queries against the paged cache; their own keys are already stored."""
    T = q.shape[0]
    assert q.stride(1) == 1
    _dense(out, "out"); _dense(k_pool, "k_pool"); _dense(v_pool, "v_pool")
    for t, n in ((positions, "positions"), (page_table, "page_table"), (slots, "slots"),
                 (seq_index, "seq_index")):
        _i32(t, n)
    assert k_pool.dtype == q.dtype
    _check(library().agv_attention_paged_simt(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(out), dtype_code(q.dtype), _ptr(k_pool),
        _ptr(v_pool), _ptr(page_table), _ptr(slots), _ptr(positions), _ptr(seq_index),
        page_table.shape[1], page, cap, T, n_heads, n_kv_heads, head_dim,
        ctypes.c_float(scale), window, _stream()))


# ------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _f32(logits, "logits"); _i32(out, "out")
    B, V = logits.shape
    assert logits.stride(1) == 1
    with _span("argmax", B * V * 4):
        _check(library().agv_argmax(_ptr(logits), ctypes.c_longlong(logits.stride(0)), B, V,
                                    _ptr(out), _stream()))


def history_append(tokens: torch.Tensor, slots: torch.Tensor, hist: torch.Tensor,
                   hist_len: torch.Tensor) -> None:
    """hist[slot, hist_len[slot]++] = token for every entry with a slot."""
    for t, n in ((tokens, "tokens"), (slots, "slots"), (hist, "hist"), (hist_len, "hist_len")):
        _i32(t, n)
    _dense(hist, "hist")
    _check(library().agv_history_append(_ptr(tokens), _ptr(slots), _ptr(hist), _ptr(hist_len),
                                        hist.shape[1], slots.numel(), _stream()))


def take_tokens(tokens: torch.Tensor, prev: torch.Tensor, take: torch.Tensor,
                vocab_size: int) -> None:
    """tokens[b] = prev[b] for every b if take[0] is set (on the device)."""
    for t, n in ((tokens, "tokens"), (prev, "prev"), (take, "take")):
        _i32(t, n)
    assert prev.numel() >= tokens.numel() and take.numel() >= 1
    _check(library().agv_take_tokens(_ptr(tokens), _ptr(prev), _ptr(take), tokens.numel(),
                                     vocab_size, _stream()))


SAMPLING_WORDS = 8


def sampling_words(temperature: float, top_k: int, top_p: float, seed: int,
                   penalty: float):
    """The sampling options as the int32 words the kernels read from the device
    (``dev_params``): [1 / temperature, top_k, top_p, seed low, seed high, penalty]."""
    import numpy as np
    w = np.zeros(SAMPLING_WORDS, dtype=np.int32)
    f = w.view(np.float32)
    f[0] = 1.0 / temperature if temperature > 0 else 1.0
    w[1] = int(top_k)
    f[2] = top_p
    w[3:5] = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint32).view(np.int32)
    f[5] = penalty
    return w


def repeat_penalty(logits: torch.Tensor, slots: torch.Tensor, hist: torch.Tensor,
                   hist_len: torch.Tensor, penalty: float,
                   dev_params: Optional[torch.Tensor] = None) -> None:
    """Penalise, in place, every id in each row's slot history, once per occurrence.
    ``dev_params`` (``sampling_words`` on the device) replaces ``penalty`` at run time."""
    _f32(logits, "logits"); _i32(dev_params, "dev_params")
    for t, n in ((slots, "slots"), (hist, "hist"), (hist_len, "hist_len")):
        _i32(t, n)
    B, V = logits.shape
    _dense(hist, "hist")
    _check(library().agv_repeat_penalty(_ptr(logits), ctypes.c_longlong(logits.stride(0)), B, V,
                                        _ptr(slots), _ptr(hist), _ptr(hist_len), hist.shape[1],
                                        ctypes.c_float(penalty), _ptr(dev_params), _stream()))


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float, top_k: int, top_p: float,
           seed: int, seq_ids: torch.Tensor, steps: torch.Tensor,
           dev_params: Optional[torch.Tensor] = None) -> None:
    """out[b] drawn from logits[b]; ``dev_params`` (``sampling_words`` on the device)
    replaces temperature, top_k, top_p and seed at run time."""
    _f32(logits, "logits"); _i32(out, "out"); _i32(steps, "steps"); _i32(dev_params, "dev_params")
    if dev_params is not None:
        assert dev_params.numel() >= SAMPLING_WORDS
    if seq_ids.dtype != torch.int64:
        raise KernelError("seq_ids must be int64")
    B, V = logits.shape
    assert logits.stride(1) == 1
    with _span("sample", B * V * 4):
        _check(library().agv_sample(_ptr(logits), ctypes.c_longlong(logits.stride(0)), B, V,
                                    _ptr(out), ctypes.c_float(temperature), int(top_k),
                                    ctypes.c_float(top_p), ctypes.c_ulonglong(seed & (2**64 - 1)),
                                    _ptr(seq_ids), _ptr(steps), _ptr(dev_params), _stream()))


def linear_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
              w2: Optional[torch.Tensor] = None, activation: str = "gelu_tanh",
              splits: int = 1, token_tile: int = 0, cluster: int = 0,
              op: str = "linear") -> None:
    """bfloat16 product on the tensor cores (tcgen05 + TMA).

    out [T, N] in bfloat16 or 32-bit.  With splits > 1, K is cut into ranges that
    run in CTAs of their own.  ``cluster`` = c (2..8, dividing splits): every c CTAs
    of a tile add their partial sums through distributed shared memory and out is
    [splits / c, T, N] (plain [T, N] when splits == c).  ``cluster`` = 0: out is
    [splits, T, N] 32-bit partial sums (use ``linear_tc_splits`` for the real count).
    """
    T, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(1) == 1
    _dense(w, "w")
    if w2 is not None:
        _dense(w2, "w2")
        assert w2.shape == w.shape and w2.dtype == w.dtype
    cluster = int(cluster)
    groups = splits // cluster if cluster else splits
    if groups > 1:
        assert out.dim() == 3 and out.shape == (groups, T, N) and out.is_contiguous()
        ldc = N
    else:
        assert out.shape == (T, N) and out.stride(1) == 1
        ldc = out.stride(0)
    with _span(op, *_linear_cost(x, w, w2, out)):
        _check(library().agv_linear_tc(
            _ptr(x), _ptr(w), _ptr(w2), _ptr(out), T, N, K, ctypes.c_longlong(x.stride(0)),
            ctypes.c_longlong(ldc), dtype_code(out.dtype), ACT[activation], splits, cluster,
            token_tile, _stream()))


ARGMAX_MAX_ROWS = 128


def linear_argmax_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``linear_argmax`` takes these operands (else: the product, then ``argmax``)."""
    return linear_tc_supported(x, w) and x.shape[0] <= ARGMAX_MAX_ROWS


def linear_argmax(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = first index of the greatest element of (x w^T)[t, :], bfloat16 on the
    tensor cores; the [T, N] product is never written.  At most 128 rows of x."""
    T, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(1) == 1 and T <= ARGMAX_MAX_ROWS
    _dense(w, "w"); _i32(out, "out")
    assert out.numel() >= T and out.is_contiguous()
    global _launches
    with _span("lm_head_argmax", N * K * 2 + T * K * 2, 2 * T * N * K):
        _check(library().agv_linear_tc_argmax(_ptr(x), _ptr(w), _ptr(out), T, N, K,
                                              ctypes.c_longlong(x.stride(0)), _stream()))
    _launches += 1            # the product and the kernel that reads its keys out


def linear_tc_splits(K: int, splits: int) -> int:
    return library().agv_linear_tc_splits(K, splits)


def linear_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and
            w.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and
            w.data_ptr() % 16 == 0)


def linear_tc_status() -> int:
    """0, or the code of the first bounded wait of a tensor-core kernel that gave
    up since the last call (this call synchronises the device)."""
    torch.cuda.synchronize()
    return library().agv_linear_tc_status()


def selftest_bounded_wait(limit: int = 2000, ctas: int = 4):
    """Runs the unit kernel whose mbarrier waits all run out after ``limit`` polls;
    returns (status code, clock cycles the first wait took).  The kernel follows the
    tensor-core kernels' give-up protocol: record a code, stop, free tensor memory,
    return."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cycles = torch.zeros(1, dtype=torch.int32, device="cuda")
    _check(library().agv_selftest_bounded_wait(ctypes.c_uint(limit), ctas, _ptr(status),
                                               _ptr(cycles), _stream()))
    torch.cuda.synchronize()
    return int(status.item()), int(cycles.item()) & 0xFFFFFFFF


# ------------------------------------------------------------------ dispatch
_n_sms = None


def n_sms() -> int:
    """Streaming multiprocessors of the current device (read once)."""
    global _n_sms
    if _n_sms is None:
        _n_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _n_sms

_PREFILL_TC = os.environ.get("AGAVE_B200_PREFILL_ATTENTION", "tcgen05") != "mma"

def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
           w2: Optional[torch.Tensor] = None, activation: str = "gelu_tanh",
           op: str = "linear") -> None:
    """out = x w^T (or the gated pair).  Which kernel runs follows from the dtype and the
    weight's shape; how K is cut into ranges (and with it the order of the 32-bit sums)
    also follows from the number of rows of x, so a token's result is the same in any
    company up to that summation order."""
    if linear_tc_supported(x, w) and (w2 is None or out.dtype == torch.bfloat16):
        c = 0
        if w2 is not None and x.shape[0] <= 64:
            # decoding through a gated layer with few 64-feature tiles: two or four
            # CTAs per tile, each on a range of K, joined by a cluster
            tiles = (w.shape[0] + 63) // 64
            kb = (w.shape[1] + 63) // 64
            sms = n_sms()
            c = 4 if tiles * 4 <= sms and kb >= 8 else 2 if tiles * 2 <= 2 * sms and kb >= 4 else 0
        linear_tc(x, w, out, w2, activation, splits=max(c, 1), cluster=c, op=op)
    else:
        linear_simt(x, w, out, w2, activation, op=op)


def plan_splits(T: int, N: int, K: int, cheap_sum: bool = False):
    """(groups, cluster size) of the ranges K is cut into so that about one CTA per
    SM is busy when the weight has few row tiles (decoding through narrow
    layers).  The CTAs of a cluster add their sums in the kernel; the groups are
    left to the consumer.  ``cheap_sum``: the consumer adds partial sums in the
    loads it makes anyway (the q/k norm kernel), so up to eight groups are better
    than a cluster, whose exchange costs about 2 us.  Prompts are not cut."""
    if T > 64:
        tile = 128 if T <= 128 else 256
        ctas = ((N + 127) // 128) * ((T + tile - 1) // tile)
        kb = (K + 63) // 64
        if T <= 512:
            # short prompts have one or two token tiles: without a cut a narrow weight
            # would run on a dozen CTAs; the partial sums (fewer, the more tokens there
            # are to write them for) are left to the consumer
            most = 16 if T <= 128 else 8 if T <= 256 else 4
            want = min(kb // 2, n_sms() // ctas, most)
            return (linear_tc_splits(K, want), 0) if want >= 2 else (1, 0)
        # long prompts: only a long K over few tiles is cut, in two, with the partial
        # sums left to the consumer (a cluster's exchange is slow for wide tiles)
        if ctas <= n_sms() // 2 + 6 and kb >= 32:
            return 2, 0
        return 1, 0
    tile = 16 if T <= 16 else 32 if T <= 32 else 64
    ctas = ((N + 127) // 128) * ((T + tile - 1) // tile)
    kb = (K + 63) // 64
    want = min(kb, (n_sms() + ctas - 1) // ctas)
    if ctas >= 100 or want < 2:
        return 1, 0
    if T > 16:
        # tiles of 32 and 64 tokens: a cluster's exchange grows with the tile, the
        # consumer's extra reads do not matter yet
        return linear_tc_splits(K, min(want, 16)), 0
    if cheap_sum:
        return linear_tc_splits(K, min(want, 8)), 0
    if want <= 8 or kb < 64:
        # a single cluster per tile adds its ranges in the kernel
        c = min(want, 8)
        return 1, c
    # a long K: more ranges than a cluster holds; the consumer adds the partial sums
    return linear_tc_splits(K, min(want, 16)), 0


def linear_partial(x: torch.Tensor, w: torch.Tensor, cheap_sum: bool = False,
                   op: str = "linear") -> torch.Tensor:
    """x w^T in 32-bit for a consumer that adds over a leading axis: [G, T, N] on
    the tensor-core path (G >= 1 groups of ranges of K; the ranges of a group
    are added inside the kernel by a cluster), else [T, N] in x's dtype.
    ``cheap_sum``: see ``plan_splits``."""
    T, K = x.shape
    N = w.shape[0]
    if linear_tc_supported(x, w):
        groups, csize = plan_splits(T, N, K, cheap_sum)
        out = torch.empty((groups, T, N), dtype=torch.float32, device=x.device)
        linear_tc(x, w, out if groups > 1 else out[0], splits=groups * max(csize, 1),
                  cluster=csize, op=op)
        return out
    out = torch.empty((T, N), dtype=x.dtype, device=x.device)
    linear_simt(x, w, out, op=op)
    return out


GEMV_FEW_MAX_ROWS = 4
# Decode steps of at most this many tokens run their projections as dot products with the
# joins in their prologues (five kernels a layer instead of seven); measured at the 1B
# sizes: one token gains 18 %, two gain 3 %, four lose 22 %.
FEW_TOKENS = int(os.environ.get("AGAVE_B200_FEW_TOKENS", "2"))


def gemv_few_supported(T: int, N: int, K: int, ldx: int = 8, join: bool = False) -> bool:
    """Whether ``gemv_few`` takes these sizes (one to four rows; see the kernel)."""
    return bool(library().agv_gemv_few_supported(T, N, K, ctypes.c_longlong(ldx), 1 if join else 0))


def gemv_few(w: torch.Tensor, out: torch.Tensor, x: Optional[torch.Tensor] = None,
             w2: Optional[torch.Tensor] = None, activation: str = "gelu_tanh",
             h_in: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None,
             y: Optional[torch.Tensor] = None, w_post: Optional[torch.Tensor] = None,
             w_next: Optional[torch.Tensor] = None, eps_post: float = 0.0, eps_next: float = 0.0,
             op: str = "linear") -> None:
    """A projection of one to four tokens, one dot product per warp and output row:
    out [T, N] = x w^T in 32-bit, or with w2 the gated pair in bfloat16.  x [T, K]
    bfloat16, or None: then x = bfloat16(norm(h_out; w_next)) with
    h_out = h_in + norm(y; w_post) (or h_in + y, or h_in itself without y) formed in the
    kernel's prologue; h_out (another buffer than h_in) receives the joined stream."""
    N, K = w.shape
    _dense(w, "w")
    assert w.dtype == torch.bfloat16 and out.stride(-1) == 1
    T = out.shape[0]
    if x is not None:
        assert x.shape == (T, K) and x.dtype == torch.bfloat16 and x.stride(1) == 1
    else:
        assert h_in is not None and h_in.shape == (T, K) and w_next is not None
        _f32(h_in, "h_in"); _f32(h_out, "h_out"); _f32(y, "y"); _f32(w_post, "w_post")
        _f32(w_next, "w_next"); _dense(h_in, "h_in")
        for t in (h_out, y):
            if t is not None:
                _dense(t, "join operand")
                assert t.shape == (T, K)
    if w2 is not None:
        _dense(w2, "w2")
        assert w2.shape == w.shape and out.dtype == torch.bfloat16
    else:
        assert out.dtype == torch.float32
    assert out.shape == (T, N)
    nbytes = (2 if w2 is not None else 1) * N * K * 2 + _nbytes(x, h_in, y, out)
    with _span(op, nbytes, 2 * T * N * K * (2 if w2 is not None else 1)):
        _check(library().agv_gemv_few(
            _ptr(w), _ptr(w2), N, K, T, _ptr(x), ctypes.c_longlong(x.stride(0) if x is not None else 0),
            _ptr(h_in), _ptr(h_out), _ptr(y), _ptr(w_post), _ptr(w_next), ctypes.c_float(eps_post),
            ctypes.c_float(eps_next), _ptr(out), ctypes.c_longlong(out.stride(0)), ACT[activation],
            _stream()))


def attention_prefill_mma(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                          cu_seqlens: torch.Tensor, max_len: int, n_heads: int, n_kv_heads: int,
                          head_dim: int, scale: float, window: int) -> None:
    """Prompts that start at 0 on the tensor cores (bfloat16, head sizes in steps
    of 8 up to 256); q, k, v are row-strided views, out is dense."""
    assert q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    assert k.stride(0) == v.stride(0)
    _dense(out, "out"); _i32(cu_seqlens, "cu_seqlens")
    _check(library().agv_attention_prefill_mma(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(k), _ptr(v),
        ctypes.c_longlong(k.stride(0)), _ptr(out), _ptr(cu_seqlens), cu_seqlens.numel() - 1,
        max_len, n_heads, n_kv_heads, head_dim, ctypes.c_float(scale), window, _stream()))


def prefill_values_scratch(T: int, B: int, n_kv_heads: int, head_dim: int,
                           device: torch.device) -> torch.Tensor:
    """The buffer the tcgen05 prompt attention reads the values from, transposed:
    [nkv * hd, columns], every sequence padded to a multiple of 64 columns."""
    cols = library().agv_attention_prefill_tc_vt_cols(T, B)
    return torch.empty((n_kv_heads * head_dim, cols), dtype=torch.bfloat16, device=device)


def transpose_values(v: torch.Tensor, vt: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int,
                     n_kv_heads: int, head_dim: int) -> None:
    """vt (from ``prefill_values_scratch``) = the values v [T, nkv * hd] (row-strided
    view) transposed, every sequence padded with zeros to a multiple of 64 columns."""
    assert v.dtype == torch.bfloat16 and vt.dtype == torch.bfloat16 and v.stride(1) == 1
    _dense(vt, "vt"); _i32(cu_seqlens, "cu_seqlens")
    _check(library().agv_transpose_values(
        _ptr(v), ctypes.c_longlong(v.stride(0)), _ptr(vt), ctypes.c_longlong(vt.shape[1]),
        _ptr(cu_seqlens), cu_seqlens.numel() - 1, max_len, n_kv_heads, head_dim, _stream()))


def attention_prefill_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                         cu_seqlens: torch.Tensor, max_len: int, n_heads: int, n_kv_heads: int,
                         head_dim: int, scale: float, window: int,
                         vt: Optional[torch.Tensor] = None) -> None:
    """Prompts that start at 0 on the tcgen05 tensor cores (bfloat16, head sizes in
    steps of 16 up to 256); q, k, v are row-strided views, out is dense.  ``vt``:
    the values already transposed (by ``qk_norm_rope_store``); else this call
    transposes them."""
    assert q.dtype == torch.bfloat16 and k.dtype == q.dtype and v.dtype == q.dtype
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    assert k.stride(0) == v.stride(0)
    _dense(out, "out"); _i32(cu_seqlens, "cu_seqlens")
    T, B = q.shape[0], cu_seqlens.numel() - 1
    ready = vt is not None
    if vt is None:
        vt = prefill_values_scratch(T, B, n_kv_heads, head_dim, q.device)
    _dense(vt, "vt")
    _check(library().agv_attention_prefill_tc(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(k), _ptr(v),
        ctypes.c_longlong(k.stride(0)), _ptr(out), _ptr(vt), ctypes.c_longlong(vt.shape[1]),
        1 if ready else 0, _ptr(cu_seqlens), B, T, max_len, n_heads, n_kv_heads, head_dim,
        ctypes.c_float(scale), window, _stream()))


def attention_tc_status() -> int:
    """0, or the code of the first bounded wait of the tcgen05 attention kernel that
    gave up since the last call (this call synchronises the device)."""
    torch.cuda.synchronize()
    return library().agv_attention_tc_status()


# A prompt step of at most this many tokens runs the mma.sync attention: the tcgen05
# kernel's CTAs take 128 query rows each, so a short prompt gives it a handful of CTAs with
# a long set-up each (a 128-token step: 586 against 624 us over six layers; from 256 tokens
# on the tcgen05 kernel is ahead).
PREFILL_TC_MIN_TOKENS = 192


def attention_prefill_wants_transposed_values(qkv: torch.Tensor, head_dim: int) -> bool:
    """Whether ``attention_prefill`` on views of this projection output will take the
    tcgen05 kernel, which reads the values transposed."""
    return (_PREFILL_TC and qkv.shape[0] > PREFILL_TC_MIN_TOKENS and qkv.dtype == torch.bfloat16 and
            head_dim % 16 == 0 and head_dim <= 256 and qkv.stride(0) % 8 == 0 and
            qkv.data_ptr() % 16 == 0)


def attention_prefill(q, k, v, out, ctx, n_heads, n_kv_heads, head_dim, scale, window,
                      vt=None) -> None:
    """Prompt attention of one layer in bfloat16: the tcgen05 kernel for head sizes
    in steps of 16 up to 256, the mma.sync kernel for the other multiples of 8; else
    the one-warp-per-(token, head) kernel."""
    aligned = (q.dtype == torch.bfloat16 and head_dim <= 256 and
               q.stride(0) % 8 == 0 and k.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and
               k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0)
    with _span("attention", *_attention_cost(ctx, q, k, v, out, n_heads, head_dim, window)):
        if aligned and head_dim % 16 == 0 and _PREFILL_TC and q.shape[0] > PREFILL_TC_MIN_TOKENS:
            attention_prefill_tc(q, k, v, out, ctx.cu_seqlens, ctx.max_new, n_heads, n_kv_heads,
                                 head_dim, scale, window, vt=vt)
        elif aligned and head_dim % 8 == 0:
            attention_prefill_mma(q, k, v, out, ctx.cu_seqlens, ctx.max_new, n_heads,
                                  n_kv_heads, head_dim, scale, window)
        else:
            attention_prefill_simt(q, k, v, out, ctx.positions, ctx.seq_index, ctx.cu_seqlens,
                                   n_heads, n_kv_heads, head_dim, scale, window)


def _attention_cost(ctx, q, k, v, out, n_heads, head_dim, window, n_kv_heads=0):
    """(bytes, flops) of one layer's attention, from the lengths the host knows
    (``ctx.lens_host``; zeros when a step does not carry them)."""
    if _perf is None:
        return 0, 0
    lens = getattr(ctx, "lens_host", None)
    if lens is None:
        return _nbytes(q, k, v, out), 0
    seen = 0                      # (query, key) pairs
    kv_rows = 0                   # cache rows a decode step reads
    for n in lens:
        n = int(n)
        if n <= 0:
            continue
        if ctx.mode == "decode":
            vis = min(n, window) if window else n
            seen += vis
            kv_rows += vis
        elif window and n > window:
            seen += window * (window + 1) // 2 + (n - window) * window
        else:
            seen += n * (n + 1) // 2
    esz = out.element_size()
    nbytes = _nbytes(q, k, v, out) + 2 * kv_rows * n_kv_heads * head_dim * esz
    return nbytes, 4 * n_heads * head_dim * seen


def attention_decode_plan(head_dim: int, dtype: torch.dtype, max_keys: int):
    """(chunk length, number of chunks) the split decode attention uses."""
    chunk, n = ctypes.c_int(0), ctypes.c_int(0)
    _check(library().agv_attention_decode_plan(head_dim, dtype_code(dtype), max_keys,
                                               ctypes.byref(chunk), ctypes.byref(n)))
    return chunk.value, n.value


_counters = {}


def _decode_counters(device: torch.device, n: int) -> torch.Tensor:
    """Arrival counters of the split decode attention: zero between launches (the
    kernel resets what it counted), so one buffer per device serves every layer."""
    t = _counters.get(device)
    if t is None or t.numel() < n:
        t = _counters[device] = torch.zeros(max(n, 65536), dtype=torch.int32, device=device)
    return t


def attention_decode_status() -> int:
    """0, or 1 + the tile at which a bounded wait of the decode attention for a tile of keys
    and values gave up first since the last call (this call synchronises the device)."""
    return library().agv_attention_decode_status()


DECODE_TILES = {"auto": 0, "copies": 1, "tma": 2}


def attention_decode_tiles(form: str) -> str:
    """How the tensor-core decode attention brings its key / value tiles: "auto" (from the
    sizes), "copies" (16-byte copies by all threads) or "tma" (the cache's pages as TMA
    boxes, wherever the cache's geometry allows).  Returns the setting before."""
    before = library().agv_attention_decode_set_tiles(DECODE_TILES[form])
    if before < 0:
        raise KernelError("attention_decode_set_tiles failed")
    return {v: k for k, v in DECODE_TILES.items()}[before]


def prepare_device(device: torch.device) -> None:
    """Allocate what the kernels share on a device before any graph is recorded."""
    _decode_counters(device, 65536)


def attention_decode_split(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor,
                           v_pool: torch.Tensor, page_table: torch.Tensor, slots: torch.Tensor,
                           positions: torch.Tensor, page: int, cap: int, n_heads: int,
                           n_kv_heads: int, head_dim: int, scale: float, window: int,
                           max_keys: int, part_acc: Optional[torch.Tensor] = None,
                           part_ml: Optional[torch.Tensor] = None) -> None:
    """One query per batch entry against the paged cache, keys split into chunks
    whose partial results go through scratch memory (allocated here if not given)."""
    B = q.shape[0]
    assert q.stride(1) == 1
    _dense(out, "out"); _dense(k_pool, "k_pool"); _dense(v_pool, "v_pool")
    for t, n in ((positions, "positions"), (page_table, "page_table"), (slots, "slots")):
        _i32(t, n)
    assert k_pool.dtype == q.dtype and out.dtype == q.dtype
    _, n_splits = attention_decode_plan(head_dim, q.dtype, max_keys)
    if part_acc is None:
        part_acc = torch.empty((B, n_heads, n_splits, head_dim), dtype=torch.float32,
                               device=q.device)
        part_ml = torch.empty((B, n_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    assert part_acc.numel() >= B * n_heads * n_splits * head_dim
    assert part_ml.numel() >= B * n_heads * n_splits * 2
    _f32(part_acc, "part_acc"); _f32(part_ml, "part_ml")
    counters = _decode_counters(q.device, B * n_heads)
    _check(library().agv_attention_decode(
        _ptr(q), ctypes.c_longlong(q.stride(0)), _ptr(out), dtype_code(q.dtype), _ptr(k_pool),
        _ptr(v_pool), _ptr(page_table), _ptr(slots), _ptr(positions), page_table.shape[1], page,
        cap, B, n_heads, n_kv_heads, head_dim, ctypes.c_float(scale), window, max_keys,
        _ptr(part_acc), _ptr(part_ml), _ptr(counters), _stream()))


_FUSED_DECODE = os.environ.get("AGAVE_B200_FUSED_DECODE_ATTENTION", "1") != "0"


def attention_decode_fused_supported(dtype: torch.dtype, head_dim: int, rotary_dim: int) -> bool:
    """Whether ``attention_decode_fused`` takes a layer of these sizes."""
    return (_FUSED_DECODE and dtype == torch.bfloat16 and bool(
        library().agv_attention_decode_fused_supported(BF16, head_dim, rotary_dim)))


def attention_decode_fused(partial: torch.Tensor, wq: Optional[torch.Tensor],
                           wk: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                           sin: Optional[torch.Tensor], store_kv: bool, out: torch.Tensor, view,
                           ctx, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                           window: int) -> None:
    """Decode attention of one layer with the q/k norm, the rotation and the cache store
    of the new position inside the attention kernel: ``partial`` [G, B, (nh + 2 nkv) *
    hd] are the projection's 32-bit partial sums."""
    _f32(partial, "partial"); _dense(partial, "partial"); _dense(out, "out")
    _f32(wq, "wq"); _f32(wk, "wk"); _f32(cos, "cos"); _f32(sin, "sin")
    G, B, width = partial.shape
    assert width == (n_heads + 2 * n_kv_heads) * head_dim and out.dtype == torch.bfloat16
    assert view.k_pool.dtype == torch.bfloat16
    if cos is not None:
        _dense(cos, "cos"); _dense(sin, "sin")
        assert cos.shape == (B, head_dim // 2) and sin.shape == cos.shape
    max_keys = max(1, min(window, ctx.max_len) if window else ctx.max_len)
    _, n_splits = attention_decode_plan(head_dim, torch.bfloat16, max_keys)
    # the tensor-core form leaves at most one partial result per cluster, and at most 16
    # clusters share a sequence, however long the context may get
    n_splits = min(n_splits, 16)
    part_acc = torch.empty((B, n_heads, n_splits, head_dim), dtype=torch.float32,
                           device=out.device)
    part_ml = torch.empty((B, n_heads, n_splits, 2), dtype=torch.float32, device=out.device)
    counters = _decode_counters(out.device, B * n_heads)
    with _span("attention", *_attention_cost(ctx, partial, None, None, out, n_heads, head_dim,
                                             window, n_kv_heads)):
        _check(library().agv_attention_decode_fused(
            _ptr(partial), G, _ptr(wq), _ptr(wk), ctypes.c_float(eps), _ptr(cos), _ptr(sin),
            1 if store_kv else 0, _ptr(out), _ptr(view.k_pool), _ptr(view.v_pool),
            _ptr(view.page_table), _ptr(ctx.slots), _ptr(ctx.positions),
            view.page_table.shape[1], view.page, view.cap, B, n_heads, n_kv_heads, head_dim,
            ctypes.c_float(scale), window, max_keys, _ptr(part_acc), _ptr(part_ml),
            _ptr(counters), _stream()))


def attention_decode(q, out, view, ctx, n_heads, n_kv_heads, head_dim, scale, window) -> None:
    """Decode attention of one layer: the split kernel for head sizes in steps of
    16 up to 512, else the one-warp-per-head kernel."""
    with _span("attention", *_attention_cost(ctx, q, None, None, out, n_heads, head_dim, window,
                                             n_kv_heads)):
        if head_dim % 16 == 0 and head_dim <= 512:
            max_keys = min(window, ctx.max_len) if window else ctx.max_len
            attention_decode_split(q, out, view.k_pool, view.v_pool, view.page_table, ctx.slots,
                                   ctx.positions, view.page, view.cap, n_heads, n_kv_heads,
                                   head_dim, scale, window, max(1, max_keys))
        else:
            attention_paged_simt(q, out, view.k_pool, view.v_pool, view.page_table, ctx.slots,
                                 ctx.positions, ctx.seq_index, view.page, view.cap, n_heads,
                                 n_kv_heads, head_dim, scale, window)
