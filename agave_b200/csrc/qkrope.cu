// Per-head RMS norm of q and k, rotation, and the write of k and v into the
// paged cache, in one pass over the fused projection output.
//
// One warp per (token, head).  Reference order: norm before rotation
// (src/models/gemma3.zig:724-748), split-half pairs (i, i + rotary_dim/2)
// (src/backend/kernels/cuda/rope.zig:9-37), k stored after norm and rotation,
// v as projected (src/backend/kernels/cpu/sdpa.zig:18-21).
//
// Cache addressing: position p of a sequence lives in ring row p % cap of its
// slot; the row's page comes from the slot's page table.  A token whose row a
// later token of the same step overwrites (p < len_after - cap) is not stored.
#include "common.cuh"
#include "cache_write.cuh"
#include <type_traits>

constexpr int QK_WARPS = 4;
constexpr int QK_MAX_HD = 1024;

extern "C" int agv_transpose_values(const void* v, long long kv_stride, void* vt, long long vt_ld,
                                    const int* cu_seqlens, int B, int max_len, int nkv, int hd,
                                    cudaStream_t stream);

template <typename T>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_norm_rope_store_kernel(T* __restrict__ qkv, long long row_stride,
                          const float* __restrict__ part, int n_splits, long long split_stride,
                          int n_tokens, int nh, int nkv,
                          int hd, const float* __restrict__ wq, const float* __restrict__ wk,
                          float eps, const float* __restrict__ cosv,
                          const float* __restrict__ sinv, int rotary_half,
                          const int* __restrict__ positions, CacheWrite cw) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = nh + 2 * nkv;
    const long long item = (long long)blockIdx.x * QK_WARPS + warp;
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads), head = (int)(item % heads);
    float* buf = smem + warp * hd;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    const float* w = is_q ? wq : (is_k ? wk : nullptr);
    // where the row goes in the cache: these loads depend on one another, so they
    // start now and overlap the arithmetic below
    const bool stores = !is_q && cw.k_pool;
    int c_pos = 0, c_slot = -1, c_len = 0, c_page = 0;
    if (stores) {
        const int cb = cw.seq_index[t];
        c_pos = positions[t];
        c_slot = cw.slots[cb];
        c_len = cw.lens[cb];
        if (c_slot >= 0)
            c_page = cw.page_table[(size_t)c_slot * cw.max_pages + (c_pos % cw.cap) / cw.page];
    }

    float ss = 0.f;
    if (part) {
        // the projection arrives as 32-bit partial sums over ranges of K
        const float* ps = part + (size_t)t * (size_t)(heads * hd) + (size_t)head * hd;
        // eight elements per lane at a time, all their loads independent; the
        // ranges of K are added in order
        for (int e0 = 0; e0 < hd; e0 += 256) {
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
            for (int sp = 0; sp < n_splits; ++sp) {
                const float* row = ps + (size_t)sp * split_stride;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int e = e0 + lane + 32 * i;
                    if (e < hd) v[i] += row[e];
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = e0 + lane + 32 * i;
                if (e < hd) {
                    buf[e] = v[i];
                    ss += v[i] * v[i];
                }
            }
        }
    } else {
        for (int e = lane; e < hd; e += 32) {
            const float v = to_f32(src[e]);
            buf[e] = v;
            ss += v * v;
        }
    }
    if (!is_q && !is_k) {
        // v head: stored as projected
        if (part) {
            __syncwarp();
            for (int e = lane; e < hd; e += 32) src[e] = from_f32<T>(buf[e]);
        }
    } else {
        if (w) {
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)hd + eps);
            for (int e = lane; e < hd; e += 32) buf[e] = buf[e] * r * w[e];
        }
        __syncwarp();
        if (cosv) {
            const float* c = cosv + (size_t)t * rotary_half;
            const float* s = sinv + (size_t)t * rotary_half;
            for (int e = lane; e < rotary_half; e += 32) {
                const float re = buf[e], im = buf[e + rotary_half];
                buf[e] = re * c[e] - im * s[e];
                buf[e + rotary_half] = re * s[e] + im * c[e];
            }
        }
        __syncwarp();
        for (int e = lane; e < hd; e += 32) src[e] = from_f32<T>(buf[e]);
    }
    if (!stores || c_slot < 0) return;
    const int p = c_pos;
    if (p < c_len - cw.cap) return;
    const int row = p % cw.cap;
    const int page = c_page;
    const int g = is_k ? head - nh : head - nh - nkv;
    T* pool = (T*)(is_k ? cw.k_pool : cw.v_pool);
    T* dst = pool + (((size_t)page * cw.page + row % cw.page) * nkv + g) * hd;
    for (int e = lane; e < hd; e += 32) dst[e] = from_f32<T>(buf[e]);
}

// The same for head sizes that are multiples of 64 up to 256 with the whole head
// in registers.  A lane keeps two runs of HALF = hd / 64 consecutive elements: one
// in the first half of the head (from lane * HALF) and its partners in the rotation
// (the same offsets in the second half).  Runs of 2 or 4 elements move as one
// 8- or 16-byte access.  Every load the row needs (partial sums, weights, cos / sin,
// the chain that finds the cache row) is issued before the first use, so their
// latencies overlap.
template <int N>
__device__ __forceinline__ void ld_run(const float* __restrict__ p, float* o) {
    if constexpr (N == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        o[0] = t.x, o[1] = t.y, o[2] = t.z, o[3] = t.w;
    } else if constexpr (N == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        o[0] = t.x, o[1] = t.y;
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) o[i] = p[i];
    }
}
template <int N>
__device__ __forceinline__ void ld_run(const __nv_bfloat16* __restrict__ p, float* o) {
    if constexpr (N == 4) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        o[0] = __low2float(a), o[1] = __high2float(a), o[2] = __low2float(b), o[3] = __high2float(b);
    } else if constexpr (N == 2) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(p);
        o[0] = __low2float(a), o[1] = __high2float(a);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) o[i] = __bfloat162float(p[i]);
    }
}
template <int N>
__device__ __forceinline__ void st_run(float* p, const float* v) {
    if constexpr (N == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else if constexpr (N == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    else {
#pragma unroll
        for (int i = 0; i < N; ++i) p[i] = v[i];
    }
}
template <int N>
__device__ __forceinline__ void st_run(__nv_bfloat16* p, const float* v) {
    if constexpr (N == 4) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
        const __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<const uint32_t*>(&a);
        t.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    } else if constexpr (N == 2) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) p[i] = __float2bfloat16(v[i]);
    }
}

template <typename T, int NE, bool MULTI>
__global__ void __launch_bounds__(QK_WARPS * 32, MULTI ? 1 : 8)
qk_norm_rope_store_reg_kernel(T* __restrict__ qkv, long long row_stride,
                              const float* __restrict__ part, int n_splits,
                              long long split_stride, int n_tokens, int nh, int nkv,
                              const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                              const float* __restrict__ cosv, const float* __restrict__ sinv,
                              const int* __restrict__ positions, CacheWrite cw, VtWrite vw,
                              int vt_blocks) {
    // What the host copied in at the start of the step (positions, sequence index, slots,
    // lengths, page table) and the norm weights are read before the wait for the
    // predecessor, which only produces the projection (and, early in a step, cos / sin).
    pdl_launch_next();
    constexpr int hd = NE * 32, HALF = NE / 2, H2 = hd / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = nh + 2 * nkv;
    if ((int)blockIdx.x < vt_blocks) {
        // ---- the first blocks write the values transposed (they take longest, so they
        // start first): one tile of 64 tokens x 64 of the nkv * hd value columns each
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
            __shared__ __align__(16) __nv_bfloat16 tile[64][72];    // rows of 9 x 16 bytes
            __shared__ int cols[64], pads[64], pad_at[64], n_pads;
            const int vb = blockIdx.x, ncb = nkv * hd / 64;
            const int t0 = (vb / ncb) * 64, c0 = (vb % ncb) * 64;
            if (threadIdx.x == 0) n_pads = 0;
            __syncthreads();
            if (threadIdx.x < 64) {
                const int t = t0 + threadIdx.x;
                int col = -1, pad = 0;
                if (t < n_tokens) {
                    const int b = vw.seq_index[t], p = positions[t];
                    int start = 0;
                    for (int i = 0; i < b; ++i) start += (vw.cu[i + 1] - vw.cu[i] + 63) & ~63;
                    col = start + p;
                    const int len = vw.cu[b + 1] - vw.cu[b];
                    if (p == len - 1) pad = ((len + 63) & ~63) - len;
                }
                cols[threadIdx.x] = col;
                pads[threadIdx.x] = pad;
                if (pad) pad_at[atomicAdd(&n_pads, 1)] = threadIdx.x;   // (ends of sequences)
            }
            pdl_wait();
            // 16 threads per token row (4 columns each), 8 rows per pass
            const int tr = threadIdx.x >> 4, tc = (threadIdx.x & 15) * 4;
            const size_t vcol = (size_t)(nh + nkv) * hd + c0 + tc;
            float val[8][4];
#pragma unroll
            for (int ps = 0; ps < 8; ++ps) {
                const int t = t0 + ps * 8 + tr;
                val[ps][0] = val[ps][1] = val[ps][2] = val[ps][3] = 0.f;
                if (t < n_tokens) {
                    if (part) {
                        for (int sp = 0; sp < (MULTI ? n_splits : 1); ++sp) {
                            float x[4];
                            ld_run<4>(part + (size_t)sp * split_stride +
                                          (size_t)t * (size_t)(heads * hd) + vcol, x);
                            val[ps][0] += x[0], val[ps][1] += x[1], val[ps][2] += x[2],
                                val[ps][3] += x[3];
                        }
                    } else {
                        ld_run<4>(qkv + (size_t)t * row_stride + vcol, val[ps]);
                    }
                }
            }
#pragma unroll
            for (int ps = 0; ps < 8; ++ps)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    tile[tc + e][ps * 8 + tr] = __float2bfloat16(val[ps][e]);
            __syncthreads();
            const int g = c0 / hd, d0 = c0 % hd;
            if (cols[0] >= 0 && (cols[0] & 7) == 0 && cols[63] == cols[0] + 63) {
                // 64 tokens of one sequence at an aligned column: 16 bytes (8 tokens) a store
                for (int i = threadIdx.x; i < 64 * 8; i += QK_WARPS * 32) {
                    const int d = i >> 3, ch = i & 7;
                    *reinterpret_cast<uint4*>(vw.vt + (size_t)(g * hd + d0 + d) * vw.ld + cols[0] +
                                              ch * 8) =
                        *reinterpret_cast<const uint4*>(&tile[d][ch * 8]);
                }
            } else {
                for (int d = warp; d < 64; d += QK_WARPS) {
                    __nv_bfloat16* dst = vw.vt + (size_t)(g * hd + d0 + d) * vw.ld;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int tl = h * 32 + lane, col = cols[tl];
                        if (col >= 0) dst[col] = tile[d][tl];
                    }
                }
            }
            for (int k = 0; k < n_pads; ++k) {
                const int tl = pad_at[k], pad = pads[tl];
                for (int i = threadIdx.x; i < 64 * pad; i += QK_WARPS * 32) {
                    const int d = i / pad, pc = i % pad;
                    vw.vt[(size_t)(g * hd + d0 + d) * vw.ld + cols[tl] + 1 + pc] =
                        __float2bfloat16(0.f);
                }
            }
        } else {
            pdl_wait();
        }
        return;
    }
    const long long item = (long long)(blockIdx.x - vt_blocks) * QK_WARPS + warp;
    if (item >= (long long)n_tokens * heads) {
        pdl_wait();
        return;
    }
    const int t = (int)(item / heads), head = (int)(item % heads);
    const int e0 = lane * HALF;                       // first run; the second is at e0 + H2
    T* src = qkv + (size_t)t * row_stride + (size_t)head * hd + e0;
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv, is_v = !is_q && !is_k;
    const float* w = is_q ? wq : (is_k ? wk : nullptr);
    const bool stores = !is_q && cw.k_pool;
    // the chain to the cache row
    int c_pos = 0, c_slot = -1, c_len = 0, c_page = 0;
    if (stores) {
        const int cb = cw.seq_index[t];
        c_pos = positions[t];
        c_slot = cw.slots[cb];
        c_len = cw.lens[cb];
        if (c_slot >= 0)
            c_page = cw.page_table[(size_t)c_slot * cw.max_pages + (c_pos % cw.cap) / cw.page];
    }
    // operands of the arithmetic: v[0..HALF) first run, v[HALF..NE) second run
    float wv[NE], cs[HALF], sn[HALF], v[NE];
    if (w) {
        ld_run<HALF>(w + e0, wv);
        ld_run<HALF>(w + H2 + e0, wv + HALF);
    } else {
#pragma unroll
        for (int i = 0; i < NE; ++i) wv[i] = 1.f;
    }
    pdl_wait();
    const bool rotate = cosv && !is_v;
    if (rotate) {
        ld_run<HALF>(cosv + (size_t)t * H2 + e0, cs);
        ld_run<HALF>(sinv + (size_t)t * H2 + e0, sn);
    } else {
#pragma unroll
        for (int i = 0; i < HALF; ++i) cs[i] = 1.f, sn[i] = 0.f;
    }
    if (part) {
        const float* ps = part + (size_t)t * (size_t)(heads * hd) + (size_t)head * hd + e0;
        if (!MULTI) {
            // (one range of K: prompts, whose many warps need their registers few)
            ld_run<HALF>(ps, v);
            ld_run<HALF>(ps + H2, v + HALF);
        } else {
            constexpr int U = 8;                      // ranges of K loaded together
#pragma unroll
            for (int i = 0; i < NE; ++i) v[i] = 0.f;
            for (int s0 = 0; s0 < n_splits; s0 += U) {
                float tv[U][NE];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float* row = ps + (size_t)min(s0 + u, n_splits - 1) * split_stride;
                    ld_run<HALF>(row, tv[u]);
                    ld_run<HALF>(row + H2, tv[u] + HALF);
                }
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int i = 0; i < NE; ++i) v[i] += s0 + u < n_splits ? tv[u][i] : 0.f;
            }
        }
    } else {
        ld_run<HALF>(src, v);
        ld_run<HALF>(src + H2, v + HALF);
    }
    if (!is_v) {
        if (w) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < NE; ++i) ss += v[i] * v[i];
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
            for (int i = 0; i < NE; ++i) v[i] = v[i] * r * wv[i];
        }
        if (rotate) {
#pragma unroll
            for (int i = 0; i < HALF; ++i) {
                const float re = v[i], im = v[i + HALF];
                v[i] = re * cs[i] - im * sn[i];
                v[i + HALF] = re * sn[i] + im * cs[i];
            }
        }
    }
    if (!is_v || part) {
        st_run<HALF>(src, v);
        st_run<HALF>(src + H2, v + HALF);
    }
    if (!stores || c_slot < 0) return;
    if (c_pos < c_len - cw.cap) return;
    const int row = c_pos % cw.cap;
    const int g = is_k ? head - nh : head - nh - nkv;
    T* pool = (T*)(is_k ? cw.k_pool : cw.v_pool);
    T* dst = pool + (((size_t)c_page * cw.page + row % cw.page) * nkv + g) * hd + e0;
    st_run<HALF>(dst, v);
    st_run<HALF>(dst + H2, v + HALF);
}

template <typename T>
static bool launch_qk_reg(T* qkv, long long row_stride, const float* part, int n_splits,
                          long long split_stride, int n_tokens, int nh, int nkv, int hd,
                          const float* wq, const float* wk, float eps, const float* cosv,
                          const float* sinv, int rotary_dim, const int* positions,
                          const CacheWrite& cw, const VtWrite& vw, unsigned main_blocks,
                          cudaStream_t stream) {
    if (hd % 64 != 0 || hd > 256 || (cosv && rotary_dim != hd)) return false;
    if (vw.vt && !std::is_same<T, __nv_bfloat16>::value) return false;
    const unsigned vt_blocks =
        vw.vt ? (unsigned)((n_tokens + 63) / 64) * (unsigned)(nkv * hd / 64) : 0u;
    const unsigned grid = main_blocks + vt_blocks;
    // runs of hd / 64 elements move as single accesses: everything must sit on 16 bytes
    if (row_stride % 8 || !agv_aligned(qkv, 16) || !agv_aligned(part, 16) ||
        !agv_aligned(wq, 16) || !agv_aligned(wk, 16) || !agv_aligned(cosv, 16) ||
        !agv_aligned(sinv, 16) || !agv_aligned(cw.k_pool, 16) || !agv_aligned(cw.v_pool, 16))
        return false;
#define AGV_QK_REG(NE)                                                                          \
    if (part && n_splits > 1)                                                                   \
        agv_launch(qk_norm_rope_store_reg_kernel<T, NE, true>, grid, QK_WARPS * 32, 0, stream,  \
                   qkv, row_stride, part, n_splits, split_stride, n_tokens, nh, nkv, wq, wk,    \
                   eps, cosv, sinv, positions, cw, vw, (int)vt_blocks);                         \
    else                                                                                        \
        agv_launch(qk_norm_rope_store_reg_kernel<T, NE, false>, grid, QK_WARPS * 32, 0, stream, \
                   qkv, row_stride, part, n_splits, split_stride, n_tokens, nh, nkv, wq, wk,    \
                   eps, cosv, sinv, positions, cw, vw, (int)vt_blocks)
    if (hd == 64) { AGV_QK_REG(2); }
    else if (hd == 128) { AGV_QK_REG(4); }
    else if (hd == 192) { AGV_QK_REG(6); }
    else { AGV_QK_REG(8); }
#undef AGV_QK_REG
    return true;
}

// qkv: [T, nh + 2 nkv, hd] (row stride in elements), rewritten in place: q and k
// heads normed (if wq / wk given) and rotated (if cos / sin given).  k and v
// are also written to the layer's cache pools unless k_pool is null.  With
// part != null the input is read from part [n_splits, T, (nh + 2 nkv) * hd]
// (32-bit partial sums, dense) instead, and qkv only receives the result.
// With vt != null (bfloat16 only) the values are also written transposed into
// vt [nkv * hd, vt_ld] (see VtWrite); that needs seq_index, positions, cu_seqlens
// [n_seq + 1] and the greatest sequence length.
AGV_API int agv_qk_norm_rope_store(void* qkv, int dtype, long long row_stride, const float* part,
                                   int n_splits, int n_tokens, int nh,
                                   int nkv, int hd, const float* wq, const float* wk, float eps,
                                   const float* cosv, const float* sinv, int rotary_dim,
                                   const int* positions, void* k_pool, void* v_pool,
                                   const int* page_table, const int* slots, const int* lens,
                                   const int* seq_index, int max_pages, int page, int cap,
                                   void* vt, long long vt_ld, const int* cu_seqlens, int n_seq,
                                   int max_len, cudaStream_t stream) {
    AGV_REQUIRE(n_tokens >= 0 && nh > 0 && nkv > 0 && hd > 0, "qk_norm_rope: bad sizes");
    AGV_REQUIRE(hd <= QK_MAX_HD, "qk_norm_rope: head_dim %d exceeds %d", hd, QK_MAX_HD);
    AGV_REQUIRE(rotary_dim % 2 == 0 && rotary_dim <= hd, "qk_norm_rope: rotary_dim %d must be even "
                "and at most head_dim %d", rotary_dim, hd);
    AGV_REQUIRE(row_stride >= (long long)(nh + 2 * nkv) * hd, "qk_norm_rope: row stride too short");
    AGV_REQUIRE(!k_pool || (v_pool && page_table && slots && lens && seq_index && page > 0 &&
                            cap > 0 && max_pages > 0), "qk_norm_rope: incomplete cache arguments");
    AGV_REQUIRE(!cosv || (sinv && positions), "qk_norm_rope: cos without sin or positions");
    AGV_REQUIRE(!k_pool || positions, "qk_norm_rope: the cache store needs positions");
    AGV_REQUIRE(!part || n_splits >= 1, "qk_norm_rope: partial sums need n_splits >= 1");
    AGV_REQUIRE(!vt || (dtype == AGV_BF16 && seq_index && positions && cu_seqlens && n_seq > 0 &&
                        vt_ld % 64 == 0 && agv_aligned(vt, 16)),
                "qk_norm_rope: the transposed values need bfloat16, seq_index, positions and "
                "cu_seqlens");
    if (n_tokens == 0) return 0;
    VtWrite vw{(__nv_bfloat16*)vt, vt_ld, cu_seqlens, seq_index};
    const long long split_stride = (long long)n_tokens * (nh + 2 * nkv) * hd;
    CacheWrite cw{k_pool, v_pool, page_table, slots, lens, seq_index, max_pages, page, cap};
    const long long items = (long long)n_tokens * (nh + 2 * nkv);
    const unsigned grid = (unsigned)((items + QK_WARPS - 1) / QK_WARPS);
    const size_t smem = (size_t)QK_WARPS * hd * sizeof(float);
    const int half = cosv ? rotary_dim / 2 : 0;
    if (dtype == AGV_F32 &&
        launch_qk_reg<float>((float*)qkv, row_stride, part, n_splits, split_stride, n_tokens, nh,
                             nkv, hd, wq, wk, eps, cosv, sinv, rotary_dim, positions, cw, vw, grid,
                             stream)) {
        AGV_LAUNCH_OK("qk_norm_rope_store_reg_kernel");
        return 0;
    }
    if (dtype == AGV_BF16 &&
        launch_qk_reg<__nv_bfloat16>((__nv_bfloat16*)qkv, row_stride, part, n_splits, split_stride,
                                     n_tokens, nh, nkv, hd, wq, wk, eps, cosv, sinv, rotary_dim,
                                     positions, cw, vw, grid, stream)) {
        AGV_LAUNCH_OK("qk_norm_rope_store_reg_kernel");
        return 0;
    }
    if (dtype == AGV_F32)
        agv_launch(qk_norm_rope_store_kernel<float>, grid, QK_WARPS * 32, smem, stream, (float*)qkv, row_stride, part, n_splits, split_stride, n_tokens, nh, nkv, hd, wq, wk,
            eps, cosv, sinv, half, positions, cw);
    else if (dtype == AGV_BF16)
        agv_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, grid, QK_WARPS * 32, smem, stream, (__nv_bfloat16*)qkv, row_stride, part, n_splits, split_stride, n_tokens, nh, nkv, hd,
            wq, wk, eps, cosv, sinv, half, positions, cw);
    else
        return agv_fail(-1, "qk_norm_rope: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("qk_norm_rope_store_kernel");
    if (vt) {
        // the general kernel does not transpose: a kernel of its own reads the values
        // that the launch above wrote
        const __nv_bfloat16* v = (const __nv_bfloat16*)qkv + (size_t)(nh + nkv) * hd;
        return agv_transpose_values(v, row_stride, vt, vt_ld, cu_seqlens, n_seq, max_len, nkv, hd,
                                    stream);
    }
    return 0;
}
