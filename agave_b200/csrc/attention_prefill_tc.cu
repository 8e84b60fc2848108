// Prompt attention on the fifth-generation tensor cores (bfloat16): a flash-style
// kernel over the step's own keys and values, causal with an optional window,
// ragged over the sequences of a batch.
//
// One CTA owns 128 query rows of one sequence: the G query heads that share a
// key/value head times 128 / G consecutive tokens (G = heads per kv head when that
// divides 128 and is at most 16, else one head and 128 tokens), so a key/value tile
// is loaded once for all heads that read it.  Keys come in tiles of 64 positions.
//
//   S = Q K^T     tcgen05.mma M 128, N 64, K 16 over head_dim; Q [128 x hd] and
//                 K [64 x hd] are K-major tiles that TMA brings (128-byte swizzle);
//                 S is a 32-bit accumulator in tensor memory, two buffers.
//   softmax       four warps, one query row per thread (its TMEM lane): scores read
//                 with tcgen05.ld, bounds applied, running maximum and sum in
//                 32-bit, P rounded to bfloat16 and written to shared memory as a
//                 K-major tile.  O is only rescaled when the maximum grows by more
//                 than 2^8 (the sum carries the same stale maximum, so the result
//                 is the same up to rounding).
//   O += P V      tcgen05.mma M 128, N hd, K 16 over the 64 keys; the V operand must
//                 be K-major too, i.e. [hd x keys]: a small kernel first writes the
//                 step's values transposed, each sequence padded to a multiple of
//                 64 columns (zeros), so every tile starts on a 128-byte boundary.
//
// Warp roles: warp 0 loads (TMA), warp 1 allocates tensor memory, warps 1 and 7
// issue S = Q K^T (even and odd tiles), warps 2-5 are the softmax and the epilogue,
// warp 6 issues O += P V.
// S of tile j + 1 is computed while the softmax of tile j runs.  Every wait on an mbarrier is bounded; when one gives up the kernel
// records a code, stops, frees its tensor memory and returns.
//
// Reference: online softmax per (token, head) over KV tiles
// (src/backend/kernels/cuda/sdpa_prefill.zig:26-216); score = (q . k) * scale,
// kv head = h / (nh / nkv) (src/backend/kernels/cpu/sdpa.zig:36-37,58); window
// start sl - W (src/models/gemma4.zig:1153-1155).
#include "common.cuh"
#include "tcgen05.cuh"
#include <map>
#include <tuple>

using namespace tc5;

namespace {

constexpr int AT_M = 128;          // query rows per CTA
constexpr int AT_N = 64;           // keys per tile
constexpr int AT_THREADS = 256;     // loader, QK issuer, four softmax warps, PV issuer, QK issuer
constexpr int AT_S_COLS = 64;      // one S buffer
constexpr int AT_O_COL = 2 * AT_S_COLS;
constexpr float AT_LAZY = 8.0f;    // log2 units the maximum may lag before O is rescaled

__device__ int g_attn_status = 0;  // 0 ok; else (role << 8) | detail of the first wait that gave up

struct AtArgs {
    __nv_bfloat16* out;            // [T, nh * hd]
    const int* cu;                 // [B + 1]
    int nh, nkv, hd, G, QT;        // G heads packed per CTA, QT = 128 / G tokens
    int window;
    float scale_log2e;
    int kb;                        // 64-element blocks of head_dim
    int tmem_cols;
};

// 2^x by the hardware approximation (relative error about 2^-22; -inf gives 0).
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Sum of the lengths before sequence b, each rounded up to a multiple of 64.
__device__ __forceinline__ int padded_start(const int* cu, int b) {
    int s = 0;
    for (int i = 0; i < b; ++i) s += (cu[i + 1] - cu[i] + 63) & ~63;
    return s;
}

// ------------------------------------------------------------ V transposed
// vt[(g * hd + d), padded_start(b) + t] = v[cu[b] + t, g, d]; columns between a
// sequence's length and its padded length are zero.
__global__ void __launch_bounds__(256)
transpose_values_kernel(const __nv_bfloat16* __restrict__ v, long long kv_stride,
                        __nv_bfloat16* __restrict__ vt, long long vt_ld,
                        const int* __restrict__ cu, int hd) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ __nv_bfloat16 tile[];            // [64][hd + 2]
    const int b = blockIdx.z, g = blockIdx.y, t0 = blockIdx.x * 64;
    const int seq0 = cu[b], len = cu[b + 1] - seq0;
    if (t0 >= len) return;
    const int col0 = padded_start(cu, b) + t0;
    const int ld = hd + 2;
    const int pairs = hd / 2;
    for (int i = threadIdx.x; i < 64 * pairs; i += blockDim.x) {
        const int r = i / pairs, c = i % pairs;
        __nv_bfloat162 val = __floats2bfloat162_rn(0.f, 0.f);
        if (t0 + r < len)
            val = *reinterpret_cast<const __nv_bfloat162*>(v + (size_t)(seq0 + t0 + r) * kv_stride +
                                                           (size_t)g * hd + 2 * c);
        *reinterpret_cast<__nv_bfloat162*>(tile + r * ld + 2 * c) = val;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < hd * 32; i += blockDim.x) {
        const int d = i / 32, c = i % 32;               // two tokens per thread
        __nv_bfloat162 val;
        val.x = tile[(2 * c) * ld + d];
        val.y = tile[(2 * c + 1) * ld + d];
        *reinterpret_cast<__nv_bfloat162*>(vt + (size_t)(g * hd + d) * vt_ld + col0 + 2 * c) = val;
    }
}

// ------------------------------------------------------------------ attention
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                            const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_vt, AtArgs a) {
    // barriers, tensor memory and the sequence bounds (copied in at the start of the
    // step) are set up while the predecessor still runs; the loader and the softmax
    // warps wait for it before they touch q, k, v or out
    pdl_launch_next();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int q_bytes = a.kb * AT_M * 128;              // [kb][128 rows][128 B]
    const int k_bytes = a.kb * AT_N * 128;              // [kb][64 keys][128 B]
    const int v_bytes = a.hd * 128;                     // [hd rows][64 keys]
    constexpr int p_bytes = AT_M * 128;                 // [128 rows][64 keys]
    uint8_t* Qs = smem;
    uint8_t* Ks = Qs + q_bytes;                         // two stages
    uint8_t* Vs = Ks + 2 * k_bytes;                     // two stages (rounded to 1024 below)
    const int v_stage = (v_bytes + 1023) & ~1023;
    uint8_t* Ps = Vs + 2 * v_stage;                     // two buffers
    uint64_t* bars = (uint64_t*)(Ps + 2 * p_bytes);
    uint64_t* q_full = bars;            // [1]
    uint64_t* k_full = bars + 1;        // [2]
    uint64_t* k_empty = bars + 3;       // [2]
    uint64_t* v_full = bars + 5;        // [2]
    uint64_t* v_empty = bars + 7;       // [2]
    uint64_t* s_full = bars + 9;        // [2]
    uint64_t* s_free = bars + 11;       // [2]
    uint64_t* p_full = bars + 13;       // [2]
    uint64_t* o_done = bars + 15;       // [1]
    uint32_t* tmem_slot = (uint32_t*)(bars + 16);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z;
    const int seq0 = a.cu[b], len = a.cu[b + 1] - seq0;
    // tiles at the end of a sequence walk the most key tiles: they are scheduled first
    const int q0 = (gridDim.x - 1 - blockIdx.x) * a.QT;
    if (q0 >= len) {
        pdl_wait();
        return;
    }
    const int heads_per_kv = a.nh / a.nkv;
    const int head0 = a.G > 1 ? blockIdx.y * a.G : blockIdx.y;   // first query head of this CTA
    const int kvh = head0 / heads_per_kv;

    // visible key range of this query tile: causal end, window start
    const int j_hi = min(q0 + a.QT - 1, len - 1);
    const int j_lo = a.window > 0 ? max(0, q0 - a.window + 1) : 0;
    const int t_lo = j_lo / AT_N, n_tiles = j_hi / AT_N - t_lo + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&s_free[s], 4);               // one arrival per softmax warp
            mbar_init(&p_full[s], 4);
        }
        mbar_init(o_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"((uint32_t)a.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto give_up = [&](int role, int detail) {
        atomicCAS(&g_attn_status, 0, (role << 8) | detail);
        *abort_flag = 1;
    };

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ loader
        const int vt0 = padded_start(a.cu, b);
        pdl_wait();
        mbar_expect_tx(q_full, (uint32_t)q_bytes);
        for (int hl = 0; hl < a.G; ++hl)
            for (int kb = 0; kb < a.kb; ++kb)
                tma_load_3d(Qs + kb * (AT_M * 128) + hl * a.QT * 128, &map_q, kb * 64, head0 + hl,
                            seq0 + q0, q_full);
        auto load_k = [&](int j) -> bool {
            const int s = j & 1;
            if (!mbar_wait(&k_empty[s], ((j >> 1) & 1) ^ 1)) {
                give_up(1, s);
                return false;
            }
            mbar_expect_tx(&k_full[s], (uint32_t)k_bytes);
            for (int kb = 0; kb < a.kb; ++kb)
                tma_load_3d(Ks + s * k_bytes + kb * (AT_N * 128), &map_k, kb * 64, kvh,
                            seq0 + (t_lo + j) * AT_N, &k_full[s]);
            return true;
        };
        auto load_v = [&](int j) -> bool {
            const int s = j & 1;
            if (!mbar_wait(&v_empty[s], ((j >> 1) & 1) ^ 1)) {
                give_up(1, 2 + s);
                return false;
            }
            mbar_expect_tx(&v_full[s], (uint32_t)v_bytes);
            tma_load_2d(Vs + s * v_stage, &map_vt, vt0 + (t_lo + j) * AT_N, kvh * a.hd, &v_full[s]);
            return true;
        };
        // keys run one tile ahead of values: K of tile j + 1 is wanted before V of tile j
        int issued_k = 0, issued_v = 0;
        bool ok = load_k(0);
        if (ok) issued_k = 1;
        for (int j = 0; ok && j < n_tiles && !*abort_flag; ++j) {
            if (j + 1 < n_tiles) {
                ok = load_k(j + 1);
                if (!ok) break;
                issued_k = j + 2;
            }
            ok = load_v(j);
            if (ok) issued_v = j + 1;
        }
        if (*abort_flag) {
            // wait (bounded) for the copies in flight before the CTA ends
            mbar_wait(q_full, 0);
            for (int j = max(0, issued_k - 2); j < issued_k; ++j) mbar_wait(&k_full[j & 1], (j >> 1) & 1);
            for (int j = max(0, issued_v - 2); j < issued_v; ++j) mbar_wait(&v_full[j & 1], (j >> 1) & 1);
        }
    } else if ((warp == 1 || warp == 7) && lane == 0) {
        // ------------------------------------------------------------ S = Q K^T
        // two issuers, one for the even tiles and one for the odd ones (each S buffer
        // and each K stage has its own), so that one's waits hide behind the other's work
        const uint32_t idesc_s = umma_idesc(AT_M, AT_N);
        // a descriptor is linear in the address: the steps add constants to it
        const uint64_t q_desc0 = umma_desc(smem_u32(Qs)), k_desc0 = umma_desc(smem_u32(Ks));
        const int full_kb = a.hd / 64, tail_steps = (a.hd % 64) / 16;
        bool ok = mbar_wait(q_full, 0);
        if (!ok) give_up(2, 0);
        for (int j = warp == 1 ? 0 : 1; ok && j < n_tiles && !*abort_flag; j += 2) {
            const int s = j & 1;
            const uint32_t ph = (j >> 1) & 1;
            if (!mbar_wait(&k_full[s], ph)) {
                give_up(2, 2 + s);
                break;
            }
            if (j >= 2 && !mbar_wait(&s_free[s], ph ^ 1)) {
                give_up(2, 8 + s);
                break;
            }
            tc_fence_after();
            const uint32_t d = tmem_base + s * AT_S_COLS;
            uint64_t qd = q_desc0, kd = k_desc0 + (uint64_t)((s * k_bytes) >> 4);
            for (int kb = 0; kb < full_kb; ++kb) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma_bf16(d, qd + 2 * k, kd + 2 * k, idesc_s, (kb > 0 || k > 0) ? 1u : 0u);
                qd += (AT_M * 128) >> 4;
                kd += (AT_N * 128) >> 4;
            }
            for (int k = 0; k < tail_steps; ++k)
                tc_mma_bf16(d, qd + 2 * k, kd + 2 * k, idesc_s, (full_kb > 0 || k > 0) ? 1u : 0u);
            tc_commit(&k_empty[s]);
            tc_commit(&s_full[s]);
        }
    } else if (warp == 6 && lane == 0) {
        // ------------------------------------------------------------ O += P V
        const uint32_t idesc_o = umma_idesc(AT_M, a.hd);
        const uint64_t v_desc0 = umma_desc(smem_u32(Vs)), p_desc0 = umma_desc(smem_u32(Ps));
        for (int i = 0; i < n_tiles && !*abort_flag; ++i) {
            const int s = i & 1;
            const uint32_t ph = (i >> 1) & 1;
            if (!mbar_wait(&v_full[s], ph)) {
                give_up(4, s);
                break;
            }
            if (!mbar_wait(&p_full[s], ph)) {
                give_up(4, 2 + s);
                break;
            }
            tc_fence_after();
            const uint64_t pd = p_desc0 + (uint64_t)((s * p_bytes) >> 4);
            const uint64_t vd = v_desc0 + (uint64_t)((s * v_stage) >> 4);
#pragma unroll
            for (int k = 0; k < AT_N / 16; ++k)
                tc_mma_bf16(tmem_base + AT_O_COL, pd + 2 * k, vd + 2 * k, idesc_o,
                            (i > 0 || k > 0) ? 1u : 0u);
            tc_commit(&v_empty[s]);
            tc_commit(o_done);
        }
    } else if (warp >= 2 && warp < 6) {
        // ------------------------------------------------------------ softmax, epilogue
        const int row = (warp & 3) * 32 + lane;                      // TMEM lane = query row
        const int hl = row / a.QT, tl = row % a.QT;
        const int qp = q0 + tl;                                       // position in the sequence
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const int q_min = q0, q_max = q0 + a.QT - 1;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        pdl_wait();
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            const uint32_t ph = (j >> 1) & 1;
            if (*abort_flag || !mbar_wait(&s_full[s], ph)) {
                if (!*abort_flag) give_up(3, s);
                ok = false;
                break;
            }
            tc_fence_after();
            uint32_t sr[4][16];
#pragma unroll
            for (int c = 0; c < 4; ++c) tc_ld16(lane_addr + s * AT_S_COLS + c * 16, sr[c]);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[s]);
            const int j0 = (t_lo + j) * AT_N;
            // a tile every row of the CTA sees whole needs no bounds
            const bool whole = j0 + AT_N - 1 <= q_min && (a.window <= 0 || j0 > q_max - a.window);
            float sv[64];
            if (whole) {
#pragma unroll
                for (int c = 0; c < 64; ++c) sv[c] = __uint_as_float(sr[c >> 4][c & 15]);
            } else {
                const int lo = a.window > 0 ? qp - a.window : -1;     // visible: lo < key <= qp
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int key = j0 + c;
                    sv[c] = (key <= qp && key > lo) ? __uint_as_float(sr[c >> 4][c & 15]) : -INFINITY;
                }
            }
            // the maximum of the raw scores, four chains side by side (the scale is positive)
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
                mx[0] = fmaxf(mx[0], sv[c]);
                mx[1] = fmaxf(mx[1], sv[c + 1]);
                mx[2] = fmaxf(mx[2], sv[c + 2]);
                mx[3] = fmaxf(mx[3], sv[c + 3]);
            }
            const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * a.scale_log2e;
            // the maximum in use may lag the true one by up to AT_LAZY
            float factor = 1.f;
            bool rescale = false;
            if (m_used == -INFINITY) {
                m_used = tmax;
            } else if (tmax > m_used + AT_LAZY) {
                factor = exp2f(m_used - tmax);
                m_used = tmax;
                l *= factor;
                rescale = true;
            }
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            float ps[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
                const float p0 = ex2_fast(fmaf(sv[c], a.scale_log2e, neg_m));
                const float p1 = ex2_fast(fmaf(sv[c + 1], a.scale_log2e, neg_m));
                const float p2 = ex2_fast(fmaf(sv[c + 2], a.scale_log2e, neg_m));
                const float p3 = ex2_fast(fmaf(sv[c + 3], a.scale_log2e, neg_m));
                ps[0] += p0, ps[1] += p1, ps[2] += p2, ps[3] += p3;
                const __nv_bfloat162 t0 = __floats2bfloat162_rn(p0, p1);
                const __nv_bfloat162 t1 = __floats2bfloat162_rn(p2, p3);
                pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&t0);
                pk[(c >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&t1);
            }
            l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
            // O and the P buffer of two tiles ago are free once the product of the last tile ended
            if (j > 0) {
                if (!mbar_wait(o_done, (j - 1) & 1)) {
                    give_up(3, 2);
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (__any_sync(0xffffffffu, rescale)) {
                    for (int c = 0; c < a.hd; c += 16) {
                        uint32_t o[16];
                        tc_ld16(lane_addr + AT_O_COL + c, o);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                        tc_st16(lane_addr + AT_O_COL + c, o);
                    }
                    tc_wait_st();
                }
            }
            uint8_t* prow = Ps + s * p_bytes + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) =
                    make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            fence_async_shared();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[s]);
        }
        if (ok && !*abort_flag) {
            if (!mbar_wait(o_done, (n_tiles - 1) & 1)) {
                give_up(3, 3);
            } else {
                tc_fence_after();
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                __nv_bfloat16* dst = a.out + (size_t)(seq0 + qp) * ((size_t)a.nh * a.hd) +
                                     (size_t)(head0 + hl) * a.hd;
                const bool valid = qp < len;
                // 64 columns per wait: four loads in flight, then their stores
                for (int c0 = 0; c0 < a.hd; c0 += 64) {
                    uint32_t o[4][16];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (c0 + q * 16 < a.hd) tc_ld16(lane_addr + AT_O_COL + c0 + q * 16, o[q]);
                    tc_wait_ld();
                    if (valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int c = c0 + q * 16;
                            if (c < a.hd) {
                                uint32_t w[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const __nv_bfloat162 t = __floats2bfloat162_rn(
                                        __uint_as_float(o[q][2 * i]) * inv,
                                        __uint_as_float(o[q][2 * i + 1]) * inv);
                                    w[i] = *reinterpret_cast<const uint32_t*>(&t);
                                }
                                *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
                                *reinterpret_cast<uint4*>(dst + c + 8) =
                                    make_uint4(w[4], w[5], w[6], w[7]);
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)a.tmem_cols)
                     : "memory");
    }
}

// A bf16 tensor of up to three dimensions (innermost first), read in boxes with the
// 128-byte swizzle; cached by its geometry.
int make_map_nd(CUtensorMap* out, const void* ptr, int rank, const cuuint64_t* dims,
                const cuuint64_t* strides_bytes, const cuuint32_t* box) {
    typedef std::tuple<const void*, int, unsigned long long, unsigned long long, unsigned long long,
                       unsigned long long, unsigned long long, unsigned, unsigned, unsigned> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key(ptr, rank, dims[0], dims[1], rank > 2 ? dims[2] : 0, strides_bytes[0],
            rank > 2 ? strides_bytes[1] : 0, box[0], box[1], rank > 2 ? box[2] : 0);
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *out = it->second;
            return 0;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return agv_fail(-4, "attention: the driver does not export cuTensorMapEncodeTiled");
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr),
                    dims, strides_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return agv_fail(-4, "attention: cuTensorMapEncodeTiled failed with code %d", (int)r);
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

int packed_heads(int nh, int nkv) {
    const int g = nh / nkv;
    return (g > 1 && g <= 16 && 128 % g == 0) ? g : 1;
}

}  // namespace

AGV_API int agv_attention_prefill_tc_supported(int hd, long long q_stride, long long kv_stride) {
    return (hd >= 16 && hd % 16 == 0 && hd <= 256 && q_stride % 8 == 0 && kv_stride % 8 == 0) ? 1 : 0;
}

// Columns the transposed-values scratch needs for B sequences of T tokens in all.
AGV_API long long agv_attention_prefill_tc_vt_cols(int T, int B) {
    return ((long long)T + 63LL * B + 63) / 64 * 64;
}


AGV_API int agv_attention_tc_status() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int));
    if (v) {
        int zero = 0;
        cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
    }
    return v;
}

// vt[(g * hd + d), start(b) + t] = v[cu[b] + t, g, d] for all sequences (start(b):
// the earlier lengths, each rounded up to 64), zeros up to the next multiple of 64.
AGV_API int agv_transpose_values(const void* v, long long kv_stride, void* vt, long long vt_ld,
                                 const int* cu_seqlens, int B, int max_len, int nkv, int hd,
                                 cudaStream_t stream) {
    AGV_REQUIRE(hd % 2 == 0 && kv_stride % 2 == 0 && vt_ld % 2 == 0 && agv_aligned(v, 4) &&
                agv_aligned(vt, 4), "transpose_values: sizes must be even");
    if (B <= 0 || max_len <= 0) return 0;
    dim3 grid((max_len + 63) / 64, nkv, B);
    const size_t smem = (size_t)64 * (hd + 2) * sizeof(__nv_bfloat16);
    agv_launch(transpose_values_kernel, grid, 256, smem, stream, (const __nv_bfloat16*)v, kv_stride,
               (__nv_bfloat16*)vt, vt_ld, cu_seqlens, hd);
    AGV_LAUNCH_OK("transpose_values_kernel");
    return 0;
}

// Whole prompts that start at position 0, bfloat16.  q: [T, nh, hd] rows of
// stride q_stride; k, v: [T, nkv, hd] rows of stride kv_stride; out: [T, nh * hd]
// dense; vt: scratch [nkv * hd, vt_cols] (see agv_attention_prefill_tc_vt_cols);
// cu_seqlens: [B + 1] first token of each sequence; T: rows of q, k and v;
// max_len: the greatest sequence length (sizes the grid).  window 0: no window.
// vt_ready != 0: vt already holds the transposed values (agv_qk_norm_rope_store
// wrote them); else they are transposed here first.
AGV_API int agv_attention_prefill_tc(const void* q, long long q_stride, const void* k,
                                     const void* v, long long kv_stride, void* out, void* vt,
                                     long long vt_cols, int vt_ready, const int* cu_seqlens, int B,
                                     int T, int max_len, int nh, int nkv, int hd, float scale,
                                     int window, cudaStream_t stream) {
    AGV_REQUIRE(B >= 0 && T >= 0 && nh > 0 && nkv > 0 && hd > 0 && max_len >= 0,
                "attention: bad sizes");
    AGV_REQUIRE(nh % nkv == 0, "attention: %d heads are not a multiple of %d kv heads", nh, nkv);
    AGV_REQUIRE(agv_attention_prefill_tc_supported(hd, q_stride, kv_stride),
                "attention: the tcgen05 kernel needs head_dim (%d) a multiple of 16 up to 256 and "
                "row strides that are multiples of 8", hd);
    AGV_REQUIRE(agv_aligned(q, 16) && agv_aligned(k, 16) && agv_aligned(v, 16) &&
                agv_aligned(out, 16) && agv_aligned(vt, 128),
                "attention: operands must be 16-byte aligned (the scratch 128-byte)");
    AGV_REQUIRE(vt_cols >= agv_attention_prefill_tc_vt_cols(T, B) && vt_cols % 64 == 0,
                "attention: the transposed-values scratch has %lld columns, %lld are needed",
                vt_cols, agv_attention_prefill_tc_vt_cols(T, B));
    AGV_REQUIRE(window >= 0, "attention: negative window");
    AGV_REQUIRE(B <= 65535 && nh <= 65535, "attention: batch or head count exceeds the grid limit");
    if (B == 0 || max_len == 0 || T == 0) return 0;

    AtArgs a;
    a.out = (__nv_bfloat16*)out;
    a.cu = cu_seqlens;
    a.nh = nh, a.nkv = nkv, a.hd = hd;
    a.G = packed_heads(nh, nkv);
    a.QT = AT_M / a.G;
    a.window = window;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.kb = (hd + 63) / 64;
    a.tmem_cols = AT_O_COL + hd <= 256 ? 256 : 512;

    CUtensorMap mq, mk, mvt;
    {
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nh, (cuuint64_t)T};
        cuuint64_t str[2] = {(cuuint64_t)hd * 2, (cuuint64_t)q_stride * 2};
        cuuint32_t box[3] = {64, 1, (cuuint32_t)a.QT};
        if (int rc = make_map_nd(&mq, q, 3, dims, str, box)) return rc;
    }
    {
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nkv, (cuuint64_t)T};
        cuuint64_t str[2] = {(cuuint64_t)hd * 2, (cuuint64_t)kv_stride * 2};
        cuuint32_t box[3] = {64, 1, (cuuint32_t)AT_N};
        if (int rc = make_map_nd(&mk, k, 3, dims, str, box)) return rc;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)vt_cols, (cuuint64_t)nkv * hd};
        cuuint64_t str[1] = {(cuuint64_t)vt_cols * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)hd};
        if (int rc = make_map_nd(&mvt, vt, 2, dims, str, box)) return rc;
    }

    if (!vt_ready)
        if (int rc = agv_transpose_values(v, kv_stride, vt, vt_cols, cu_seqlens, B, max_len, nkv, hd,
                                          stream))
            return rc;
    const int v_stage = (hd * 128 + 1023) & ~1023;
    const size_t smem = 1024 + (size_t)a.kb * AT_M * 128 + 2 * (size_t)a.kb * AT_N * 128 +
                        2 * (size_t)v_stage + 2 * (size_t)AT_M * 128 + 256;
    static size_t configured = 0;
    if (smem > configured) {
        AGV_CUDA_OK(cudaFuncSetAttribute(attention_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    dim3 grid((max_len + a.QT - 1) / a.QT, a.G > 1 ? nkv : nh, B);
    agv_launch(attention_prefill_tc_kernel, grid, AT_THREADS, smem, stream, mq, mk, mvt, a);
    AGV_LAUNCH_OK("attention_prefill_tc_kernel");
    return 0;
}
