// Softmax attention, one warp per (query token, head), keys visited one by one
// with a running maximum and sum.  It reads keys and values either from the
// step's own projection output (prompts that start at position 0) or from the
// paged cache (decoding), and serves the 32-bit path and small or odd shapes
// of the bfloat16 path.  Scores, softmax and the weighted sum are 32-bit.
//
// Reference: score = (q . k) * scale, head h uses kv head h / (nh / nkv), softmax
// with the maximum subtracted (src/backend/kernels/cpu/sdpa.zig:36-37,58,184-234);
// causal bound src/backend/kernels/cuda/sdpa_prefill.zig:50; window start
// sl - W for sl = p + 1 > W (src/models/gemma4.zig:1153-1155).  No value row is
// skipped for a small weight (the reference skips below 1e-6,
// src/backend/kernels/cuda/sdpa.zig:14,99).
#include "common.cuh"

constexpr int AT_WARPS = 4;
constexpr int AT_MAX_I = 16;          // head_dim <= 32 * AT_MAX_I

struct PagedKV {
    const void* k_pool;        // [n_pages, page, n_kv, hd] of this layer
    const void* v_pool;
    const int* page_table;     // [n_slots, max_pages]
    const int* slots;          // [B]
    int max_pages, page, cap;
};

template <typename T, bool PAGED>
__global__ void __launch_bounds__(AT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k,
                      const T* __restrict__ v, long long kv_stride, T* __restrict__ out,
                      const int* __restrict__ positions, const int* __restrict__ seq_index,
                      const int* __restrict__ cu_seqlens, PagedKV pk, int n_tokens, int nh, int nkv,
                      int hd, float scale, int window) {
    pdl_wait();
    pdl_launch_next();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * AT_WARPS + warp;
    if (item >= (long long)n_tokens * nh) return;
    const int t = (int)(item / nh), h = (int)(item % nh);
    const int g = h / (nh / nkv);
    const int b = seq_index[t];
    T* o = out + ((size_t)t * nh + h) * hd;
    int slot = 0;
    if (PAGED) {
        slot = pk.slots[b];
        if (slot < 0) {
            for (int e = lane; e < hd; e += 32) o[e] = from_f32<T>(0.f);
            return;
        }
    }
    const int p = positions[t];
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const T* qp = q + (size_t)t * q_stride + (size_t)h * hd;
    float qr[AT_MAX_I], acc[AT_MAX_I];
#pragma unroll
    for (int i = 0; i < AT_MAX_I; ++i) {
        const int e = lane + 32 * i;
        qr[i] = e < hd ? to_f32(qp[e]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const size_t base = PAGED ? 0 : (size_t)cu_seqlens[b];
    for (int j = lo; j <= p; ++j) {
        const T *kp, *vp;
        if (PAGED) {
            const int row = j % pk.cap;
            const int page = pk.page_table[(size_t)slot * pk.max_pages + row / pk.page];
            const size_t off = (((size_t)page * pk.page + row % pk.page) * nkv + g) * hd;
            kp = (const T*)pk.k_pool + off;
            vp = (const T*)pk.v_pool + off;
        } else {
            kp = k + (base + j) * kv_stride + (size_t)g * hd;
            vp = v + (base + j) * kv_stride + (size_t)g * hd;
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < AT_MAX_I; ++i) {
            const int e = lane + 32 * i;
            if (e < hd) s = fmaf(qr[i], to_f32(kp[e]), s);
        }
        s = warp_sum(s) * scale;
        const float mn = fmaxf(m, s);
        const float alpha = expf(m - mn);      // exp(-inf) = 0 on the first key
        const float w = expf(s - mn);
        l = l * alpha + w;
#pragma unroll
        for (int i = 0; i < AT_MAX_I; ++i) {
            const int e = lane + 32 * i;
            if (e < hd) acc[i] = acc[i] * alpha + w * to_f32(vp[e]);
        }
        m = mn;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < AT_MAX_I; ++i) {
        const int e = lane + 32 * i;
        if (e < hd) o[e] = from_f32<T>(acc[i] * inv);
    }
}

static int check_attn(int n_tokens, int nh, int nkv, int hd, int window) {
    AGV_REQUIRE(n_tokens >= 0 && nh > 0 && nkv > 0 && hd > 0, "attention: bad sizes");
    AGV_REQUIRE(nh % nkv == 0, "attention: %d heads are not a multiple of %d kv heads", nh, nkv);
    AGV_REQUIRE(hd <= 32 * AT_MAX_I, "attention: head_dim %d exceeds %d", hd, 32 * AT_MAX_I);
    AGV_REQUIRE(window >= 0, "attention: negative window");
    return 0;
}

// Whole prompts that start at position 0.  q: [T, nh, hd] with row stride
// q_stride; k, v: [T, nkv, hd] with row stride kv_stride (both may point into
// the fused projection output); out: [T, nh * hd] dense.  Token t of batch
// entry b = seq_index[t] has position positions[t] and sees the tokens
// cu_seqlens[b] + j for lo <= j <= position.  window 0: no window.
AGV_API int agv_attention_prefill_simt(const void* q, long long q_stride, const void* k,
                                       const void* v, long long kv_stride, void* out, int dtype,
                                       const int* positions, const int* seq_index,
                                       const int* cu_seqlens, int n_tokens, int nh, int nkv, int hd,
                                       float scale, int window, cudaStream_t stream) {
    if (int rc = check_attn(n_tokens, nh, nkv, hd, window)) return rc;
    if (n_tokens == 0) return 0;
    const long long items = (long long)n_tokens * nh;
    const unsigned grid = (unsigned)((items + AT_WARPS - 1) / AT_WARPS);
    PagedKV pk{};
    if (dtype == AGV_F32)
        agv_launch(attention_simt_kernel<float, false>, grid, AT_WARPS * 32, 0, stream, (const float*)q, q_stride, (const float*)k, (const float*)v, kv_stride, (float*)out,
            positions, seq_index, cu_seqlens, pk, n_tokens, nh, nkv, hd, scale, window);
    else if (dtype == AGV_BF16)
        agv_launch(attention_simt_kernel<__nv_bfloat16, false>, grid, AT_WARPS * 32, 0, stream, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
            kv_stride, (__nv_bfloat16*)out, positions, seq_index, cu_seqlens, pk, n_tokens, nh,
            nkv, hd, scale, window);
    else
        return agv_fail(-1, "attention: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("attention_simt_kernel");
    return 0;
}

// Queries against the paged cache (the query's own key is already stored).
// Token t of entry b = seq_index[t] at positions[t] sees cache positions
// lo..positions[t] of slot slots[b]; a negative slot yields zeros.
AGV_API int agv_attention_paged_simt(const void* q, long long q_stride, void* out, int dtype,
                                     const void* k_pool, const void* v_pool, const int* page_table,
                                     const int* slots, const int* positions, const int* seq_index,
                                     int max_pages, int page, int cap, int n_tokens, int nh,
                                     int nkv, int hd, float scale, int window,
                                     cudaStream_t stream) {
    if (int rc = check_attn(n_tokens, nh, nkv, hd, window)) return rc;
    AGV_REQUIRE(page > 0 && cap > 0 && max_pages > 0, "attention: bad cache geometry");
    AGV_REQUIRE(window == 0 || window <= cap, "attention: window %d exceeds the ring of %d rows",
                window, cap);
    if (n_tokens == 0) return 0;
    const long long items = (long long)n_tokens * nh;
    const unsigned grid = (unsigned)((items + AT_WARPS - 1) / AT_WARPS);
    PagedKV pk{k_pool, v_pool, page_table, slots, max_pages, page, cap};
    if (dtype == AGV_F32)
        agv_launch(attention_simt_kernel<float, true>, grid, AT_WARPS * 32, 0, stream, (const float*)q, q_stride, nullptr, nullptr, 0, (float*)out, positions, seq_index,
            nullptr, pk, n_tokens, nh, nkv, hd, scale, window);
    else if (dtype == AGV_BF16)
        agv_launch(attention_simt_kernel<__nv_bfloat16, true>, grid, AT_WARPS * 32, 0, stream, (const __nv_bfloat16*)q, q_stride, nullptr, nullptr, 0, (__nv_bfloat16*)out, positions,
            seq_index, nullptr, pk, n_tokens, nh, nkv, hd, scale, window);
    else
        return agv_fail(-1, "attention: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("attention_simt_kernel");
    return 0;
}
