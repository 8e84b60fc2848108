"""Small, self-contained workloads of single kernels and of a decode step, for
profilers and timing.

    python -m agave_b200.profiling <case> [--iters N]

Cases (Gemma 3 1B layer sizes, random bfloat16 data):
  gemm_gated_prefill   gate/up product with the activation epilogue, 2,048 tokens
  gemm_down_prefill    down projection, 2,048 tokens
  gemm_gated_decode    gate/up product, 8 tokens
  gemm_down_decode     down projection, 8 tokens (K split over a cluster or partial sums)
  gemm_gated_decode_4b, gemm_gated_decode_27b   gate/up product with the 4B model's sizes
                       (2,560 x 10,240, 8 tokens) and the 27B model's (5,376 x 21,504, 16 tokens)
  gemm_lm_head_decode  the head over a 262,144-row table, 8 tokens
  gemm_lm_head_argmax_decode   the same with the arg max taken in the epilogue (no logits written)
  gemm_qkv_fused_prefill_4b    q/k/v product with norm, rotation, cache store and transposed
                       values in its epilogue, 4B layer sizes (width 2,560, 8 + 4 + 4 heads
                       of 256), 2,048 tokens
  gemm_qkv_prefill     q/k/v projection (32-bit output), 2,048 tokens
  qk_norm_rope_prefill q/k norm + rotation + cache store + transposed values, 2,048 tokens
  norm_prefill         residual sum + two RMS norms over 2,048 rows
  attention_prefill    prompt attention (tcgen05), one sequence of 2,048 tokens, no window
  attention_prefill_window   the same with a window of 512
  attention_prefill_mma      the mma.sync kernel on the first workload
  attention_decode_window   decode attention, 8 sequences of 128..2,048 positions, window 512
  attention_decode_full     the same without a window
  attention_decode_window_27b   16 sequences of 2,048 positions, window 1,024, with the 27B
                       model's heads (32 query, 16 kv, 128 wide: 256 pairs of sequence and kv head)
  attention_decode_window_b64, attention_decode_full_b64   the same for 64 sequences (the
                       second with a grid sized for a context of 8,192)
  norm_decode          residual sum + two RMS norms over 8 rows of 16 partial sums
  gemv_gated_join_one_token, gemv_down_one_token   the gate/up (with the join in its prologue)
                       and down projections of one token as dot products (gemv_few.cu)
  decode_step          whole decode steps of a 6-layer model (vocabulary 32,768), batch 8
  decode_step_b1, decode_step_b64   the same at batch 1 (dot-product projections) and 64
  decode_step_4b, decode_step_27b   the same with the layer sizes of the 4B model (batch 8,
                       256..4,096 positions) and the 27B model (batch 16, 2,048 positions)
  prefill_step         whole prompt steps of the same model, one prompt of 2,048 tokens

Each case prints the mean time per call: the calls run back to back from a CUDA
graph, each on the next of several copies of its operands, the copies together
larger than L2, so operands come from HBM as they do in a model step.  The
working set stays below 2 GB.
"""
from __future__ import annotations

import argparse
import sys

import torch

DEV = "cuda:0"
H, FF, NH, NKV, HD, V = 1152, 6912, 4, 1, 256, 262144


def _rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


L2_BYTES = 126 * 1024 * 1024


def _copies(nbytes: int) -> int:
    """How many copies of an operand set make the ring larger than L2 (twice over)."""
    return max(1, min(64, (2 * L2_BYTES + nbytes - 1) // max(nbytes, 1)))


def _run(fn, copies: int, iters: int) -> float:
    """Mean microseconds per call: the calls run back to back from a CUDA graph,
    each on the next copy of its operands, so that none finds them in L2."""
    n = max(copies, 8)
    for i in range(min(n, 3)):
        fn(i % copies)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(i % copies)
    g.replay()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters / n * 1e3


def case_gemm_gated(T, sizes=None):
    """Gate/up product; ``sizes`` = (hidden, intermediate) of a larger model: then through
    ``kernels.linear``, which picks the tiles and the cut of K as a decode step does."""
    from . import kernels
    h, ff = sizes or (H, FF)
    nbytes = (2 * ff * h + T * h + T * ff) * 2
    c = _copies(2 * ff * h * 2)
    x = _rnd(T, h)
    wg = [_rnd(ff, h, scale=0.02) for _ in range(c)]
    wu = [_rnd(ff, h, scale=0.02) for _ in range(c)]
    out = torch.empty(T, ff, dtype=torch.bfloat16, device=DEV)
    product = kernels.linear if sizes else kernels.linear_tc
    return (lambda i: product(x, wg[i], out, w2=wu[i])), 4 * T * ff * h, nbytes, c


def case_gemv_gated_join():
    """Gate/up of one token as dot products, the join (residual sum, both norms) in the prologue."""
    from . import kernels
    c = _copies(2 * FF * H * 2)
    wg = [_rnd(FF, H, scale=0.02) for _ in range(c)]
    wu = [_rnd(FF, H, scale=0.02) for _ in range(c)]
    h, y = torch.randn(1, H, device=DEV), torch.randn(1, H, device=DEV)
    h2 = torch.empty_like(h)
    w = torch.ones(H, device=DEV)
    out = torch.empty(1, FF, dtype=torch.bfloat16, device=DEV)
    return (lambda i: kernels.gemv_few(wg[i], out, w2=wu[i], h_in=h, h_out=h2, y=y, w_post=w, w_next=w,
                                       eps_post=1e-6, eps_next=1e-6)), 4 * FF * H, \
        2 * FF * H * 2 + FF * 2 + 3 * H * 4, c


def case_gemv_down():
    from . import kernels
    c = _copies(FF * H * 2)
    x = _rnd(1, FF)
    w = [_rnd(H, FF, scale=0.02) for _ in range(c)]
    out = torch.empty(1, H, dtype=torch.float32, device=DEV)
    return (lambda i: kernels.gemv_few(w[i], out, x=x)), 2 * FF * H, FF * H * 2 + FF * 2 + H * 4, c


def case_gemm_down(T):
    from . import kernels
    c = _copies(FF * H * 2)
    x = _rnd(T, FF)
    w = [_rnd(H, FF, scale=0.02) for _ in range(c)]
    return (lambda i: kernels.linear_partial(x, w[i])), 2 * T * FF * H, \
        (FF * H + T * FF) * 2 + T * H * 4, c


def case_gemm_qkv(T):
    from . import kernels
    N = (NH + 2 * NKV) * HD
    c = 8                                  # (the weights are small: they stay in L2, as in a step)
    x = [_rnd(T, H) for _ in range(c)]
    w = _rnd(N, H, scale=0.02)
    return (lambda i: kernels.linear_partial(x[i], w, cheap_sum=True)), 2 * T * N * H, \
        (N * H + T * H) * 2 + T * N * 4, c


def case_qk_norm_rope_prefill(T=2048):
    from . import kernels
    width, PAGE = (NH + 2 * NKV) * HD, 64
    n_pages = T // PAGE
    c = 12
    parts = [torch.randn(1, T, width, device=DEV) for _ in range(c)]
    qkvs = [torch.empty(T, width, dtype=torch.bfloat16, device=DEV) for _ in range(c)]
    kp = [torch.empty(n_pages, PAGE, NKV, HD, dtype=torch.bfloat16, device=DEV) for _ in range(c)]
    vp = [torch.empty(n_pages, PAGE, NKV, HD, dtype=torch.bfloat16, device=DEV) for _ in range(c)]
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).reshape(1, n_pages)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    lens = torch.tensor([T], dtype=torch.int32, device=DEV)
    seq_index = torch.zeros(T, dtype=torch.int32, device=DEV)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    cos = torch.empty(T, HD // 2, device=DEV)
    sin = torch.empty_like(cos)
    kernels.rope_table(positions, HD, 10000.0, 1.0, cos, sin)
    w = torch.ones(HD, device=DEV)
    vt = kernels.prefill_values_scratch(T, 1, NKV, HD, torch.device(DEV))

    def fn(i):
        kernels.qk_norm_rope_store(qkvs[i], NH, NKV, HD, w, w, 1e-6, cos, sin, HD, positions,
                                   kp[i], vp[i], table, slots, lens, seq_index, PAGE, T,
                                   partial=parts[i], vt=vt, cu_seqlens=cu, max_len=T)
    return fn, 0, T * width * (4 + 2) + 3 * T * NKV * HD * 2, c


def case_norm_prefill(T=2048):
    from . import kernels
    c = 12
    hs = [torch.randn(T, H, device=DEV) for _ in range(c)]
    ys = [torch.randn(1, T, H, device=DEV) for _ in range(c)]
    xs = [torch.empty(T, H, dtype=torch.bfloat16, device=DEV) for _ in range(c)]
    w = torch.ones(H, device=DEV)
    return (lambda i: kernels.norm_residual(hs[i], ys[i], w, w, xs[i], 1e-6, 1e-6)), 0, \
        T * H * (4 + 4 + 4 + 2), c


def case_lm_head():
    from . import kernels
    x, w = _rnd(8, H), _rnd(V, H, scale=0.02)
    out = torch.empty(8, V, dtype=torch.float32, device=DEV)
    return (lambda i: kernels.linear_tc(x, w, out)), 2 * 8 * V * H, V * H * 2 + 8 * V * 4, 1


def case_lm_head_argmax():
    from . import kernels
    x, w = _rnd(8, H), _rnd(V, H, scale=0.02)
    out = torch.empty(8, dtype=torch.int32, device=DEV)
    return (lambda i: kernels.linear_argmax(x, w, out)), 2 * 8 * V * H, V * H * 2, 1


def case_qkv_fused_prefill_4b(T=2048):
    from . import kernels
    Hq, nh, nkv, hd, PAGE = 2560, 8, 4, 256, 64
    width = (nh + 2 * nkv) * hd
    c = 6
    xs = [_rnd(T, Hq) for _ in range(c)]
    w = _rnd(width, Hq, scale=0.02)
    qkvs = [torch.empty(T, width, dtype=torch.bfloat16, device=DEV) for _ in range(c)]
    n_pages = T // PAGE
    kp = [torch.empty(n_pages, PAGE, nkv, hd, dtype=torch.bfloat16, device=DEV) for _ in range(c)]
    vp = [torch.empty(n_pages, PAGE, nkv, hd, dtype=torch.bfloat16, device=DEV) for _ in range(c)]
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).reshape(1, n_pages)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    lens = torch.tensor([T], dtype=torch.int32, device=DEV)
    seq_index = torch.zeros(T, dtype=torch.int32, device=DEV)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    cos = torch.empty(T, hd // 2, device=DEV)
    sin = torch.empty_like(cos)
    kernels.rope_table(positions, hd, 10000.0, 1.0, cos, sin)
    wn = torch.ones(hd, device=DEV)
    vt = kernels.prefill_values_scratch(T, 1, nkv, hd, torch.device(DEV))

    def fn(i):
        kernels.qkv_prefill(xs[i], w, qkvs[i], nh, nkv, hd, wn, wn, 1e-6, cos, sin, positions,
                            seq_index, k_pool=kp[i], v_pool=vp[i], page_table=table, slots=slots,
                            lens=lens, page=PAGE, cap=T, vt=vt, cu_seqlens=cu)
    return fn, 2 * T * width * Hq, (width * Hq + T * Hq + 2 * T * width) * 2, c


def case_attention_prefill(window=0, legacy=False):
    from . import kernels
    T = 2048
    c = 8
    qkv = [_rnd(T, (NH + 2 * NKV) * HD, scale=0.5) for _ in range(c)]
    out = torch.empty(T, NH * HD, dtype=torch.bfloat16, device=DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    pairs = T * (T + 1) // 2 if not window else sum(min(p + 1, window) for p in range(T))
    flops = 4 * NH * HD * pairs
    # the values transposed, as the q/k norm launch leaves them in a model step
    vts = []
    for t in qkv:
        vt = kernels.prefill_values_scratch(T, 1, NKV, HD, t.device)
        kernels.transpose_values(t[:, (NH + NKV) * HD:], vt, cu, T, NKV, HD)
        vts.append(vt)

    def fn(i):
        t = qkv[i]
        q, k, v = t[:, :NH * HD], t[:, NH * HD:(NH + NKV) * HD], t[:, (NH + NKV) * HD:]
        if legacy:
            kernels.attention_prefill_mma(q, k, v, out, cu, T, NH, NKV, HD, 0.0625, window)
        else:
            kernels.attention_prefill_tc(q, k, v, out, cu, T, NH, NKV, HD, 0.0625, window,
                                         vt=vts[i])
    return fn, flops, qkv[0].numel() * 2 + out.numel() * 2, c


def case_attention_decode(window, max_keys, B=8, grid_keys=0, heads=None, lo=128, hi=2048):
    from . import kernels
    NH, NKV, HD = heads or (globals()["NH"], globals()["NKV"], globals()["HD"])
    PAGE, max_pages = 64, 40
    c = 16 if B <= 8 else 4
    pools = [(_rnd(B * max_pages, PAGE, NKV, HD), _rnd(B * max_pages, PAGE, NKV, HD))
             for _ in range(c)]
    table = torch.arange(B * max_pages, dtype=torch.int32, device=DEV).reshape(B, max_pages)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    lens = torch.linspace(lo, hi, B).round().int().tolist()
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    q = _rnd(B, NH * HD)
    out = torch.empty_like(q)
    kernels.prepare_device(torch.device(DEV))

    def fn(i):
        kernels.attention_decode_split(q, out, pools[i][0], pools[i][1], table, slots, positions,
                                       PAGE, max_pages * PAGE, NH, NKV, HD, 0.0625, window,
                                       grid_keys or max_keys)
    nbytes = sum(min(n, window) if window else n for n in lens) * NKV * HD * 2 * 2
    return fn, 0, nbytes, c


def case_norm_decode():
    from . import kernels
    h = torch.randn(8, H, device=DEV)
    y = torch.randn(16, 8, H, device=DEV)
    w = torch.ones(H, device=DEV)
    x = torch.empty(8, H, dtype=torch.bfloat16, device=DEV)
    return (lambda i: kernels.norm_residual(h, y, w, w, x, 1e-6, 1e-6)), 0, \
        y.numel() * 4 + 3 * 8 * H * 4, 1


# layer sizes of the larger family members: hidden, heads, kv heads, head_dim, scalar, ff, window
SIZES = {"1b": (H, NH, NKV, HD, HD, FF, 512), "4b": (2560, 8, 4, 256, 256, 10240, 1024),
         "27b": (5376, 32, 16, 128, 168, 21504, 1024)}


def _six_layer_engine(max_batch=16, sizes="1b"):
    from .engine.api import Engine
    h, nh, nkv, hd, scalar, ff, window = SIZES[sizes]
    cfg = {
        "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
        "num_hidden_layers": 6, "hidden_size": h, "num_attention_heads": nh,
        "num_key_value_heads": nkv, "head_dim": hd, "query_pre_attn_scalar": scalar,
        "intermediate_size": ff, "vocab_size": 32768, "sliding_window": window,
        "sliding_window_pattern": 6, "rope_local_base_freq": 10000.0, "rope_theta": 1000000.0,
        "rms_norm_eps": 1e-6, "max_position_embeddings": 8192, "eos_token_id": 1}
    return Engine.from_config(cfg, seed=2, dtype="bfloat16", max_tokens=max_batch * 8192,
                              ctx_size=8192, max_batch=max_batch, use_graphs=False)


def case_prefill_step():
    eng = _six_layer_engine()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(3, 32768, (2048,), generator=g).tolist()

    def fn(i):
        s = eng.acquire()
        eng.step([(s, prompt)], [[2047]])
        eng.release(s)
    return fn, 0, 0, 0


def case_decode_step(batch=8, sizes="1b", lo=128, hi=2048):
    eng = _six_layer_engine(max_batch=max(16, batch), sizes=sizes)
    g = torch.Generator().manual_seed(0)
    lens = torch.linspace(lo, hi, batch).round().int().tolist()
    prompts = [torch.randint(3, 32768, (n,), generator=g).tolist() for n in lens]
    slots = [eng.acquire() for _ in prompts]
    eng.step([(s, p) for s, p in zip(slots, prompts)], [[] for _ in prompts])
    return (lambda i: eng.step([(s, [5]) for s in slots], [[0]] * batch)), 0, 0, 0


CASES = {
    "gemm_gated_prefill": lambda: case_gemm_gated(2048),
    "gemm_down_prefill": lambda: case_gemm_down(2048),
    "gemm_gated_decode": lambda: case_gemm_gated(8),
    "gemm_down_decode": lambda: case_gemm_down(8),
    "gemm_gated_decode_4b": lambda: case_gemm_gated(8, (SIZES["4b"][0], SIZES["4b"][5])),
    "gemm_gated_decode_27b": lambda: case_gemm_gated(16, (SIZES["27b"][0], SIZES["27b"][5])),
    "gemv_gated_join_one_token": case_gemv_gated_join,
    "gemv_down_one_token": case_gemv_down,
    "gemm_lm_head_decode": case_lm_head,
    "gemm_lm_head_argmax_decode": case_lm_head_argmax,
    "gemm_qkv_fused_prefill_4b": case_qkv_fused_prefill_4b,
    "gemm_qkv_prefill": lambda: case_gemm_qkv(2048),
    "qk_norm_rope_prefill": case_qk_norm_rope_prefill,
    "norm_prefill": case_norm_prefill,
    "attention_prefill": case_attention_prefill,
    "attention_prefill_window": lambda: case_attention_prefill(512),
    "attention_prefill_mma": lambda: case_attention_prefill(0, True),
    "attention_decode_window": lambda: case_attention_decode(512, 512),
    "attention_decode_full": lambda: case_attention_decode(0, 2048),
    "attention_decode_window_b64": lambda: case_attention_decode(512, 512, 64),
    "attention_decode_full_b64": lambda: case_attention_decode(0, 2048, 64, 8192),
    "attention_decode_full_b64_tight": lambda: case_attention_decode(0, 2048, 64, 2048),
    "attention_decode_window_27b": lambda: case_attention_decode(1024, 1024, 16, heads=(32, 16, 128),
                                                                lo=2048, hi=2048),
    "norm_decode": case_norm_decode,
    "decode_step": case_decode_step,
    "decode_step_b1": lambda: case_decode_step(1),
    "decode_step_b64": lambda: case_decode_step(64),
    "decode_step_4b": lambda: case_decode_step(8, "4b", 256, 4096),
    "decode_step_27b": lambda: case_decode_step(16, "27b", 2048, 2048),
    "prefill_step": case_prefill_step,
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="agave_b200.profiling", description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    fn, flops, nbytes, copies = CASES[args.case]()
    if copies == 0:                      # a whole step: host work included, no graph
        for _ in range(3):
            fn(0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn(0)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / args.iters * 1e3
    else:
        us = _run(fn, copies, args.iters)
    msg = f"{args.case}: {us:.1f} us per call"
    if flops:
        msg += f", {flops / us / 1e6:.0f} TFLOP/s"
    if nbytes:
        msg += f", {nbytes / us / 1e3:.0f} GB/s of {nbytes / 1e6:.1f} MB"
    print(msg)
    return 0


if __name__ == "__main__":
    sys.exit(main())
