// bfloat16 matrix products on the fifth-generation tensor cores:
//     out[T, N] = x[T, K] * w[N, K]^T          (plain, or K split into partial sums)
//     out[T, N] = act(x wg^T) * (x wu^T)       (gated)
//
// The weight is the M operand: one CTA owns 128 weight rows and a tile of BN
// tokens (BN = 16 ... 256), so the same kernel serves decoding (a few tokens,
// the weight streamed once from HBM) and prompts (256 tokens per tile).  TMA
// brings [128 x 64] weight boxes and [BN x 64] activation boxes into a ring of
// shared-memory stages (128-byte swizzle, K-major); one thread issues
// tcgen05.mma (M 128, N BN, K 16) into a 32-bit accumulator in tensor memory;
// four warps read the accumulator back with tcgen05.ld and write the result,
// applying the gate's activation in the gated form (two accumulators side by
// side).  Every output element is one dot product accumulated over K in
// ascending order, so a token's result does not depend on its tile mates.
//
// Warp roles: warp 0 loads, warp 1 allocates tensor memory and issues the
// products, warps 2-5 are the epilogue (warp w reads TMEM lanes 32 (w % 4) ...).
// Every wait on an mbarrier is bounded; when a wait gives up the kernel records
// a code in a status word, stops issuing work, drains what it started, frees
// its tensor memory and returns.
//
// Reference: the engine this replaces computes the same products as one dot
// product per output row with f32 accumulation, bf16 weights converted in the
// loop (src/backend/kernels/cuda/gemv_bf16.zig:6-24), once per token for
// prompts (src/backend/cuda.zig:1569-1570).
#include "common.cuh"
#include "tcgen05.cuh"
#include "cache_write.cuh"
#include <stdlib.h>
#include <map>
#include <mutex>
#include <tuple>

using namespace tc5;

namespace {

constexpr int TILE_M = 128;        // weight rows per CTA
constexpr int TILE_K = 64;         // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int RED_LD = TILE_M + 4;     // row length of a partial tile in shared memory

__device__ int g_gemm_status = 0;   // 0 ok; else (role << 8) | stage of the first wait that gave up

// The arg max of a product's rows, taken in its epilogue (the head over the vocabulary
// when the next token is the greatest logit: the logits themselves are never written).
// Every CTA reduces its 128 features to one (value, index) per token and folds it into
// the token's key with a 64-bit atomic maximum; the key orders by value first and by
// lower index second, so ties go to the first index whatever the order of arrival.  A
// one-CTA kernel launched behind the product turns the keys into indices and puts them
// back to zero for the next launch (a CTA of the product that waited to learn whether it
// is the last would hold its shared memory a memory round trip longer, which costs more
// than that launch).  Launches that use this must not overlap on the device.
constexpr int ARGMAX_MAX_TOKENS = 128;
__device__ unsigned long long g_argmax_keys[ARGMAX_MAX_TOKENS];

__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
    const unsigned u = __float_as_uint(v);
    const unsigned ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // orders like the floats
    return ((unsigned long long)ord << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)idx);
}

// The activation of the gated epilogue.  Its result is rounded to bfloat16
// (relative step 2^-8), so the hardware tanh (relative error about 2^-11) serves.
__device__ __forceinline__ float gelu_tanh_fast(float t) {
    const float u = 0.7978845608028654f * (t + 0.044715f * t * t * t);
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(u));
    return 0.5f * t * (1.0f + th);
}
__device__ __forceinline__ float silu_fast(float t) { return __fdividef(t, 1.0f + __expf(-t)); }

// MODE 0: plain.  MODE 1: gated, gate and up tiles of 128 rows each with an
// accumulator of their own (prompts).  MODE 2: gated, 64 gate rows and the 64 up
// rows of the same features share one 128-row tile and one accumulator, and the
// epilogue warps exchange the halves through shared memory (decoding: twice as
// many CTAs stream the weights).
template <int BN, int MODE, int SLIM = 0>
struct Tile {
    static constexpr bool DUAL = MODE == 1;
    static constexpr bool HALF = MODE == 2;
    static constexpr int A_BYTES = TILE_M * TILE_K * 2;                 // 16 KB
    static constexpr int B_BYTES = BN * TILE_K * 2;
    static constexpr int STAGE_BYTES = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
    static constexpr int XCHG_BYTES = HALF ? 64 * BN * 4 : 0;
    // token tiles of 128 and more run one CTA per SM with a deep ring; smaller ones
    // (decoding) leave room for a second CTA that hides this one's start and end
    // A cluster of token tiles of 16 adds its partial sums by pushing them into the shared
    // memory of the CTA that owns the features (PUSH); the inbox must not overlap the
    // stages, which a slower CTA still reads while faster peers already push.
    static constexpr bool PUSH = BN == 16 && !DUAL;
    static constexpr int INBOX_BYTES = PUSH ? BN * 144 * 4 : 0;
    // SLIM: a ring of three stages, so that three CTAs share an SM: for a weight whose
    // tiles number between two and three times the SMs, which would otherwise run as one
    // full round and a second, nearly empty one
    static constexpr int BUDGET =
        SLIM ? 56 * 1024
             : (DUAL ? 196 * 1024 : (BN >= 128 ? 196 * 1024 : (PUSH ? 96 * 1024 : 108 * 1024)));
    static constexpr int STAGES_RAW = (BUDGET - XCHG_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : (STAGES_RAW < 2 ? 2 : STAGES_RAW);
    static constexpr int TMEM_COLS_RAW = DUAL ? 2 * BN : BN;
    static constexpr int TMEM_COLS = TMEM_COLS_RAW < 32 ? 32 : TMEM_COLS_RAW;
    static constexpr int SMEM =
        STAGES * STAGE_BYTES + XCHG_BYTES + 1024 /*align*/ + 256 + (PUSH ? 1024 + INBOX_BYTES : 0);
};

__device__ __forceinline__ void st_peer_f32(float* local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)),
                 "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// out element types
template <typename TO> __device__ __forceinline__ void store_out(TO* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

template <int BN, int MODE, typename TO, int SLIM = 0>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_w2,
                    const __grid_constant__ CUtensorMap map_x, TO* __restrict__ out, int T, int N,
                    int K, long long ldc, long long split_stride, int kb_per_split, int act,
                    int cluster_reduce, int* __restrict__ argmax_out) {
    pdl_launch_next();
    using TL = Tile<BN, MODE, SLIM>;
    constexpr bool GATED = MODE == 1;          // two accumulators
    constexpr bool HALF = MODE == 2;           // gate and up rows in one tile
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* xchg = (float*)(smem + TL::STAGES * TL::STAGE_BYTES);
    uint64_t* full = (uint64_t*)(smem + TL::STAGES * TL::STAGE_BYTES + TL::XCHG_BYTES);
    uint64_t* empty = full + TL::STAGES;
    uint64_t* acc_full = empty + TL::STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    // [rank][token][row of this CTA's slice]: what the cluster's CTAs push here
    float* inbox = (float*)(smem + TL::STAGES * TL::STAGE_BYTES + TL::XCHG_BYTES + 1024);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * (HALF ? TILE_M / 2 : TILE_M);   // first output feature
    const int n0 = blockIdx.y * BN;              // first token
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    const int kb_begin = blockIdx.z * kb_per_split;
    const int kb_end = min(kb_total, kb_begin + kb_per_split);
    const int n_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TL::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"((uint32_t)TL::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // A cluster of token tiles of 16 writes into its peers' shared memory: every CTA of the
    // cluster must have started by then.  All arrive here without waiting (the loader goes
    // on to request weights) and wait just before the first such write, or, the two warps
    // that write nothing, before the cluster's second barrier.
    if (TL::PUSH && cluster_reduce)
        asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ loader
        // The weights never change, so the first ring of weight boxes is requested
        // before this kernel waits for its predecessor (which produces x): the
        // stream from HBM starts while the predecessor is still running.
        const int early = min(n_kb, TL::STAGES);
        for (int i = 0; i < early; ++i) {
            uint8_t* st = smem + i * TL::STAGE_BYTES;
            mbar_expect_tx(&full[i], TL::STAGE_BYTES);
            const int kx = (kb_begin + i) * TILE_K;
            tma_load_2d(st, &map_w, kx, m0, &full[i]);
            if (GATED) tma_load_2d(st + TL::A_BYTES, &map_w2, kx, m0, &full[i]);
            if (HALF) tma_load_2d(st + TL::A_BYTES / 2, &map_w2, kx, m0, &full[i]);
        }
        pdl_wait();
        for (int i = 0; i < early; ++i)
            tma_load_2d(smem + i * TL::STAGE_BYTES + TL::A_BYTES * (GATED ? 2 : 1), &map_x,
                        (kb_begin + i) * TILE_K, n0, &full[i]);
        int issued = early;
        for (int i = early; i < n_kb; ++i) {
            const int s = i % TL::STAGES;
            const uint32_t ph = (i / TL::STAGES) & 1;
            if (*abort_flag) break;
            if (!mbar_wait(&empty[s], ph ^ 1)) {
                atomicCAS(&g_gemm_status, 0, (1 << 8) | s);
                *abort_flag = 1;
                break;
            }
            uint8_t* st = smem + s * TL::STAGE_BYTES;
            mbar_expect_tx(&full[s], TL::STAGE_BYTES);
            const int kx = (kb_begin + i) * TILE_K;
            tma_load_2d(st, &map_w, kx, m0, &full[s]);
            if (GATED) tma_load_2d(st + TL::A_BYTES, &map_w2, kx, m0, &full[s]);
            if (HALF) tma_load_2d(st + TL::A_BYTES / 2, &map_w2, kx, m0, &full[s]);
            tma_load_2d(st + TL::A_BYTES * (GATED ? 2 : 1), &map_x, kx, n0, &full[s]);
            ++issued;
        }
        if (*abort_flag) {
            // let the copies already issued land before the shared memory is given up
            const int first = issued > TL::STAGES ? issued - TL::STAGES : 0;
            for (int i = first; i < issued; ++i)
                mbar_wait(&full[i % TL::STAGES], (i / TL::STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ products
        constexpr uint32_t idesc = umma_idesc(TILE_M, BN);
        bool ok = true;
        for (int i = 0; i < n_kb && ok; ++i) {
            const int s = i % TL::STAGES;
            const uint32_t ph = (i / TL::STAGES) & 1;
            if (*abort_flag) { ok = false; break; }
            if (!mbar_wait(&full[s], ph)) {
                atomicCAS(&g_gemm_status, 0, (2 << 8) | s);
                *abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(smem + s * TL::STAGE_BYTES);
            const uint32_t b_addr = a_addr + TL::A_BYTES * (GATED ? 2 : 1);
#pragma unroll
            for (int k = 0; k < TILE_K / UMMA_K; ++k) {
                const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                const uint64_t bd = umma_desc(b_addr + k * UMMA_K * 2);
                tc_mma_bf16(tmem_base, umma_desc(a_addr + k * UMMA_K * 2), bd, idesc, acc);
                if (GATED)
                    tc_mma_bf16(tmem_base + BN, umma_desc(a_addr + TL::A_BYTES + k * UMMA_K * 2),
                                bd, idesc, acc);
            }
            tc_commit(&empty[s]);          // the stage is free once these products have read it
        }
        tc_commit(acc_full);               // arrives when every product above is done
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;
        // this thread's output feature (in the shared-tile form lanes 64-127 hold the
        // up rows of the features whose gate rows lanes 0-63 hold)
        const int f = HALF ? m0 + (quarter & 1) * 32 + lane : m0 + quarter * 32 + lane;
        pdl_wait();          // this warp writes global memory: not before the predecessor is done
        // (the peers run: asked here, where the answer comes while the products are under way)
        if (TL::PUSH && cluster_reduce) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
        bool ok = mbar_wait(acc_full, 0);
        if (!ok) {
            atomicCAS(&g_gemm_status, 0, (3 << 8));
            *abort_flag = 1;
        }
        tc_fence_after();
        const bool run = ok && !*abort_flag && n_kb > 0;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        TO* obase = out + (size_t)blockIdx.z * split_stride;
        if (TL::PUSH && cluster_reduce) {
            // token tiles of 16: every value goes straight into the inbox of the CTA that
            // adds this feature (a rank without a range of K, or one that gave up, sends
            // zeros), so that after one cluster barrier everybody adds from its own
            // shared memory and may leave
            constexpr int FEATS_T = HALF ? TILE_M / 2 : TILE_M;
            const int S = cluster_reduce, rank = blockIdx.z % S;
            const int per = (FEATS_T + S - 1) / S, rows = HALF ? 2 * per : per;
            const int fl = quarter * 32 + lane;                       // row of the tile
            const int feat = HALF ? fl % FEATS_T : fl, part = HALF ? fl / FEATS_T : 0;
            const int dest = feat / per, j = part * per + feat % per;
            uint32_t r[16];
            if (run) {
                tc_ld16(lane_base, r);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int n = 0; n < 16; ++n) r[n] = 0u;
            }
#pragma unroll
            for (int n = 0; n < 16; ++n)
                st_peer_f32(inbox + ((size_t)rank * BN + n) * rows + j, (uint32_t)dest,
                            __uint_as_float(r[n]));
        } else if (cluster_reduce && ok && !*abort_flag && n_kb <= 0) {
            // a rank without a range of K contributes zeros
            float* red = (float*)smem;
            const int fl = quarter * 32 + lane;
            for (int c = 0; c < BN; ++c) red[c * RED_LD + fl] = 0.f;
        }
        if (TL::PUSH && cluster_reduce) {
        } else if (run && cluster_reduce) {
            // this CTA's partial sums -> shared memory [token][tile row], for the cluster
            float* red = (float*)smem;
            const int fl = quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t r[16];
                tc_ld16(lane_base + c, r);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) red[(c + j) * RED_LD + fl] = __uint_as_float(r[j]);
            }
        } else if (HALF) {
            // up half -> shared memory, then the gate half combines and stores
            if (run && quarter >= 2) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t u[16];
                    tc_ld16(lane_base + c, u);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        xchg[(c + j) * 64 + (quarter & 1) * 32 + lane] = __uint_as_float(u[j]);
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps
            if (run && quarter < 2) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t r[16];
                    tc_ld16(lane_base + c, r);
                    tc_wait_ld();
                    if (f < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int n = n0 + c + j;
                            if (n < T) {
                                const float gv = __uint_as_float(r[j]);
                                const float uv = xchg[(c + j) * 64 + quarter * 32 + lane];
                                store_out<TO>(obase + (size_t)n * ldc + f,
                                              (act == 1 ? silu_fast(gv) : gelu_tanh_fast(gv)) * uv);
                            }
                        }
                    }
                }
            }
        } else {
            // plain and two-accumulator forms: the tile goes through shared memory
            // (the ring of stages is free by now) so that rows leave in 16-byte pieces
            static_assert(BN * TILE_M * (int)sizeof(TO) <= TL::STAGES * TL::STAGE_BYTES,
                          "the output tile must fit the ring of stages");
            TO* ctile = (TO*)smem;                       // [BN][TILE_M]
            const int fl = quarter * 32 + lane;
            if (run) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t r[16], u[16];
                    tc_ld16(lane_base + c, r);
                    if (GATED) tc_ld16(lane_base + BN + c, u);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float v = __uint_as_float(r[j]);
                        if (GATED)
                            v = (act == 1 ? silu_fast(v) : gelu_tanh_fast(v)) * __uint_as_float(u[j]);
                        store_out<TO>(ctile + (c + j) * TILE_M + fl, v);
                    }
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps
            if (MODE == 0 && sizeof(TO) == 4 && argmax_out != nullptr) {
                // no logits leave the chip: each warp reduces tokens quarter, quarter + 4,
                // ... of the tile to (greatest value, first index) over the tile's features
                if (run) {
                    const float* ft = reinterpret_cast<const float*>(ctile);
                    const int rows = min(BN, T - n0);
                    for (int n = quarter; n < rows; n += 4) {
                        unsigned long long best = 0ull;
#pragma unroll
                        for (int i = 0; i < TILE_M / 32; ++i) {
                            const int f2 = lane + 32 * i;
                            if (m0 + f2 < N) {
                                const unsigned long long k2 = argmax_key(ft[n * TILE_M + f2], m0 + f2);
                                best = k2 > best ? k2 : best;
                            }
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
                            best = other > best ? other : best;
                        }
                        if (lane == 0) atomicMax(&g_argmax_keys[n0 + n], best);
                    }
                }
            } else if (run) {
                constexpr int EPV = 16 / (int)sizeof(TO);          // elements per 16 bytes
                constexpr int VPR = TILE_M / EPV;                  // 16-byte pieces per row
                const int et = (warp - 2) * 32 + lane;
                const int rows = min(BN, T - n0);
                TO* gbase = obase + (size_t)n0 * ldc + m0;
                const bool fast = m0 + TILE_M <= N && ldc % EPV == 0 &&
                                  ((uintptr_t)gbase & 15) == 0;
                if (fast) {
                    for (int i = et; i < rows * VPR; i += 128) {
                        const int n = i / VPR, vi = i % VPR;
                        const uint4 val = reinterpret_cast<const uint4*>(ctile)[i];
                        *reinterpret_cast<uint4*>(gbase + (size_t)n * ldc + vi * EPV) = val;
                    }
                } else {
                    for (int i = et; i < rows * TILE_M; i += 128) {
                        const int n = i / TILE_M, f2 = i % TILE_M;
                        if (m0 + f2 < N) gbase[(size_t)n * ldc + f2] = ctile[i];
                    }
                }
            }
        }
    }
    __syncwarp();
    if (cluster_reduce) {
        if (TL::PUSH && warp < 2) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
        pdl_wait();
        // The gridDim.z CTAs of a cluster hold partial sums of one tile over
        // consecutive ranges of K.  Each adds, in rank order, a slice of the tile's
        // features and writes the result.  Token tiles of 16: the values were pushed
        // into the adder's inbox, one barrier and everybody adds locally.  Wider tiles:
        // the adder reads every peer's shared memory, and nobody leaves before all
        // have read.
        cluster_sync_all();
        const int S = cluster_reduce, rank = blockIdx.z % S, group = blockIdx.z / S;
        constexpr int FEATS = HALF ? TILE_M / 2 : TILE_M;      // output features of the tile
        const int per = (FEATS + S - 1) / S;
        const int f_lo = rank * per, f_hi = min(FEATS, f_lo + per);
        const float* red = (const float*)smem;
        TO* gout = out + (size_t)group * split_stride;
        if (TL::PUSH) {
            // the peers' values for this CTA's features lie in its own inbox
            const int rows = HALF ? 2 * per : per;
            const int width = f_hi - f_lo;
            if (!*abort_flag && width > 0)
            for (int i = threadIdx.x; i < BN * width; i += GEMM_THREADS) {
                const int n = i / width, jl = i % width, fl = f_lo + jl;
                if (n0 + n < T && m0 + fl < N) {
                    float acc = 0.f, up = 0.f;
                    for (int q = 0; q < S; ++q) {                      // in rank order
                        acc += inbox[((size_t)q * BN + n) * rows + jl];
                        if (HALF) up += inbox[((size_t)q * BN + n) * rows + per + jl];
                    }
                    if (HALF) acc = (act == 1 ? silu_fast(acc) : gelu_tanh_fast(acc)) * up;
                    store_out<TO>(gout + (size_t)(n0 + n) * ldc + m0 + fl, acc);
                }
            }
        } else {
        if (!*abort_flag && f_hi > f_lo) {
            const int width = f_hi - f_lo;
            for (int i = threadIdx.x; i < BN * width; i += GEMM_THREADS) {
                const int n = i / width, fl = f_lo + i % width;
                if (n0 + n < T && m0 + fl < N) {
                    // every peer's value is requested before the first is used: a load
                    // from a peer's shared memory takes hundreds of cycles
                    float pv[8], pu[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        pv[q] = q < S ? ld_peer_f32(red + n * RED_LD + fl, q) : 0.f;
                        // rows 64..127 of the tile are the up rows of the same features
                        if (HALF) pu[q] = q < S ? ld_peer_f32(red + n * RED_LD + TILE_M / 2 + fl, q) : 0.f;
                    }
                    float acc = 0.f;
#pragma unroll
                    for (int q = 0; q < 8; ++q) acc += pv[q];          // in rank order
                    if (HALF) {
                        float up = 0.f;
#pragma unroll
                        for (int q = 0; q < 8; ++q) up += pu[q];
                        acc = (act == 1 ? silu_fast(acc) : gelu_tanh_fast(acc)) * up;
                    }
                    store_out<TO>(gout + (size_t)(n0 + n) * ldc + m0 + fl, acc);
                }
            }
        }
        cluster_sync_all();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)TL::TMEM_COLS)
                     : "memory");
    }
}

// Keys of the arg max epilogue -> indices; the keys go back to zero.
__global__ void __launch_bounds__(ARGMAX_MAX_TOKENS)
argmax_finish_kernel(int* __restrict__ out, int T) {
    pdl_wait();
    pdl_launch_next();
    const int t = threadIdx.x;
    if (t >= T) return;
    const unsigned long long key = g_argmax_keys[t];
    g_argmax_keys[t] = 0ull;
    out[t] = key ? (int)(0xFFFFFFFFu - (unsigned)(key & 0xFFFFFFFFull)) : 0;
}

// ------------------------------------------------------------ persistent form
// Prompts: one CTA per SM walks over output tiles.  The accumulator in tensor
// memory is double-buffered, so the products of a tile run while the epilogue
// warps still read and store the tile before it; the ring of operand stages runs
// on across tile boundaries.  Plain (MODE 0): weight rows on M, BN tokens on N.
// Gated (MODE 1): the 128-token tile is the M operand and the gate and up weight
// tiles together are one N operand of 256 rows, because a product of N 256 keeps
// the tensor pipe busy where two of N 128 do not; the accumulator's lanes are
// tokens, columns 0..127 gate and 128..255 up values of the same features, and
// each epilogue thread writes 16 consecutive features of its token.  K may be cut
// into `splits` ranges whose partial sums go to out + split * split_stride
// (MODE 0, 32-bit out).  q/k/v (MODE 3): tokens on M as in the gated form and 256
// consecutive rows of the fused q | k | v weight as the N operand, so that an epilogue
// thread holds whole heads of its token; it norms q and k heads, rotates them, writes q, k
// and v in bfloat16, stores k and v into the paged cache and writes the values transposed
// for the prompt attention: what a separate kernel would otherwise do on 32-bit sums that
// go through global memory in between (see QkvEpilogue).
constexpr int PERSISTENT_EPI_WARPS = 8;
constexpr int PERSISTENT_THREADS = 64 + 32 * PERSISTENT_EPI_WARPS;

template <int BN, int MODE>
struct PTile {
    static constexpr bool DUAL = MODE == 1 || MODE == 3;     // two weight boxes per stage
    static constexpr int A_BYTES = TILE_M * TILE_K * 2;
    static constexpr int B_BYTES = BN * TILE_K * 2;
    static constexpr int STAGE_BYTES = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
    static constexpr int ACC_COLS = DUAL ? 2 * BN : BN;
    static constexpr int TMEM_USED = 2 * ACC_COLS;              // two accumulator stages
    // (an allocation is a power of two)
    static constexpr int TMEM_COLS = TMEM_USED <= 32 ? 32 : TMEM_USED <= 64 ? 64 :
                                     TMEM_USED <= 128 ? 128 : TMEM_USED <= 256 ? 256 : 512;
    static constexpr int STAGES_RAW = (200 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int EPI_BYTES = PERSISTENT_EPI_WARPS * 16 * 32 * 4;   // per-warp staging, f32
    static constexpr int SMEM = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
    static_assert(TMEM_USED <= 512, "accumulators must fit tensor memory");
};


// What the q/k/v form's epilogue does with a token's heads (the order of
// src/models/gemma3.zig:724-748: norm, then rotation; k stored after both, v as projected,
// src/backend/kernels/cpu/sdpa.zig:18-21).  Head sizes 64, 128 and 256 (a chunk of 256
// columns then holds whole heads); the whole head is rotated, or none of it.
struct QkvEpilogue {
    __nv_bfloat16* qkv;        // [T, (nh + 2 nkv) * hd], row stride in elements
    long long row_stride;
    int nh, nkv, hd;
    const float* wq;           // [hd] or null: no norm
    const float* wk;
    float eps;
    const float* cosv;         // [T, hd / 2] or null: no rotation
    const float* sinv;
    const int* positions;      // [T]
    CacheWrite cw;
    VtWrite vw;
};

__device__ __forceinline__ void st_bf16x16(__nv_bfloat16* dst, const float (&v)[16]) {
    __nv_bfloat16 tmp[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) tmp[j] = __float2bfloat16_rn(v[j]);
    reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(tmp)[0];
    reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(tmp)[1];
}

// One epilogue warp's share of one accumulator [128 tokens x 256 columns]: lanes are tokens
// (tok), the columns are rows m0 .. m0 + 255 of the fused weight.  The two warps that share
// the lanes (half 0 and 1) each take half of every head's rotation pairs (i, i + hd / 2);
// both add up the whole head's squares, which costs a few tensor-memory loads and saves an
// exchange.
__device__ __forceinline__ void qkv_epilogue(uint32_t lane_base, int m0, int tok, int half, int T,
                                             const QkvEpilogue& qe) {
    const int hd = qe.hd, H2 = hd / 2, heads = qe.nh + 2 * qe.nkv;
    const bool live = tok < T;
    const int share = H2 / 2;                       // pairs per warp and head: 16, 32 or 64
    // where this token's key and value go: looked up when the first k or v head comes
    bool looked = false;
    int c_page = -1, c_row = 0;
    long long vt_col = -1;
    int vt_pad = 0;
    for (int hh = 0; hh * hd < 2 * TILE_M; ++hh) {
        const int head = m0 / hd + hh;
        if (head >= heads) break;
        const uint32_t base = lane_base + hh * hd;
        const bool is_q = head < qe.nh, is_k = !is_q && head < qe.nh + qe.nkv;
        const bool is_v = !is_q && !is_k;
        const float* w = is_q ? qe.wq : (is_k ? qe.wk : nullptr);
        float rs = 1.f;
        if (w) {
            float ss = 0.f;
#pragma unroll 1
            for (int c = 0; c < hd; c += 32) {
                uint32_t a[16], b[16];
                tc_ld16(base + c, a);
                tc_ld16(base + c + 16, b);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float x = __uint_as_float(a[j]), y = __uint_as_float(b[j]);
                    ss = fmaf(x, x, ss);
                    ss = fmaf(y, y, ss);
                }
            }
            rs = 1.0f / sqrtf(ss / (float)hd + qe.eps);
        }
        if (!is_q && !looked && live) {
            looked = true;
            const int b = qe.cw.seq_index ? qe.cw.seq_index[tok] : qe.vw.seq_index[tok];
            const int p = qe.positions[tok];
            if (qe.cw.k_pool) {
                const int slot = qe.cw.slots[b], len = qe.cw.lens[b];
                if (slot >= 0 && p >= len - qe.cw.cap) {
                    c_row = p % qe.cw.cap;
                    c_page = qe.cw.page_table[(size_t)slot * qe.cw.max_pages + c_row / qe.cw.page];
                }
            }
            if (qe.vw.vt) {
                int start = 0;
                for (int i = 0; i < b; ++i) start += (qe.vw.cu[i + 1] - qe.vw.cu[i] + 63) & ~63;
                vt_col = start + p;
                const int len = qe.vw.cu[b + 1] - qe.vw.cu[b];
                if (p == len - 1) vt_pad = ((len + 63) & ~63) - len;
            }
        }
        const int g = is_k ? head - qe.nh : head - qe.nh - qe.nkv;
        __nv_bfloat16* row_dst = qe.qkv + (size_t)tok * qe.row_stride + (size_t)head * hd;
        __nv_bfloat16* pool_dst = nullptr;
        if (!is_q && c_page >= 0)
            pool_dst = (__nv_bfloat16*)(is_k ? qe.cw.k_pool : qe.cw.v_pool) +
                       (((size_t)c_page * qe.cw.page + c_row % qe.cw.page) * qe.nkv + g) * hd;
        const bool rotate = qe.cosv && !is_v;
#pragma unroll 1
        for (int i = half * share; i < (half + 1) * share; i += 16) {
            uint32_t a[16], b[16];
            tc_ld16(base + i, a);
            tc_ld16(base + H2 + i, b);
            tc_wait_ld();
            if (!live) continue;
            float x[16], y[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                x[j] = __uint_as_float(a[j]);
                y[j] = __uint_as_float(b[j]);
            }
            if (w) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 wa = *reinterpret_cast<const float4*>(w + i + 4 * q);
                    const float4 wb = *reinterpret_cast<const float4*>(w + H2 + i + 4 * q);
                    x[4 * q] *= rs * wa.x, x[4 * q + 1] *= rs * wa.y;
                    x[4 * q + 2] *= rs * wa.z, x[4 * q + 3] *= rs * wa.w;
                    y[4 * q] *= rs * wb.x, y[4 * q + 1] *= rs * wb.y;
                    y[4 * q + 2] *= rs * wb.z, y[4 * q + 3] *= rs * wb.w;
                }
            }
            if (rotate) {
                const float* cs = qe.cosv + (size_t)tok * H2 + i;
                const float* sn = qe.sinv + (size_t)tok * H2 + i;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 c4 = *reinterpret_cast<const float4*>(cs + 4 * q);
                    const float4 s4 = *reinterpret_cast<const float4*>(sn + 4 * q);
                    const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float re = x[4 * q + e], im = y[4 * q + e];
                        x[4 * q + e] = re * cc[e] - im * sv[e];
                        y[4 * q + e] = re * sv[e] + im * cc[e];
                    }
                }
            }
            st_bf16x16(row_dst + i, x);
            st_bf16x16(row_dst + H2 + i, y);
            if (pool_dst) {
                st_bf16x16(pool_dst + i, x);
                st_bf16x16(pool_dst + H2 + i, y);
            }
            if (is_v && vt_col >= 0) {
                __nv_bfloat16* v0 = qe.vw.vt + (size_t)(g * hd + i) * qe.vw.ld + vt_col;
                __nv_bfloat16* v1 = qe.vw.vt + (size_t)(g * hd + H2 + i) * qe.vw.ld + vt_col;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    v0[(size_t)j * qe.vw.ld] = __float2bfloat16_rn(x[j]);
                    v1[(size_t)j * qe.vw.ld] = __float2bfloat16_rn(y[j]);
                }
                for (int pc = 1; pc <= vt_pad; ++pc)        // the sequence's last token: zero padding
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        v0[(size_t)j * qe.vw.ld + pc] = __float2bfloat16_rn(0.f);
                        v1[(size_t)j * qe.vw.ld + pc] = __float2bfloat16_rn(0.f);
                    }
            }
        }
    }
}

template <int BN, int MODE, typename TO>
__global__ void __launch_bounds__(PERSISTENT_THREADS, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_w,
                               const __grid_constant__ CUtensorMap map_w2,
                               const __grid_constant__ CUtensorMap map_x, TO* __restrict__ out,
                               int T, int N, int K, long long ldc, long long split_stride,
                               int splits, int kb_per_split, int act,
                               const __grid_constant__ QkvEpilogue qe) {
    pdl_launch_next();
    using TL = PTile<BN, MODE>;
    constexpr bool GATED = MODE == 1;
    constexpr bool QKV = MODE == 3;
    constexpr bool TOKM = GATED || QKV;                    // the token tile is the M operand
    constexpr int M_STEP = QKV ? 2 * TILE_M : TILE_M;      // weight rows per item
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* epi = smem + TL::STAGES * TL::STAGE_BYTES;
    uint64_t* full = (uint64_t*)(epi + TL::EPI_BYTES);
    uint64_t* empty = full + TL::STAGES;
    uint64_t* acc_full = empty + TL::STAGES;        // [2]
    uint64_t* acc_empty = acc_full + 2;             // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (N + M_STEP - 1) / M_STEP, n_tiles = (T + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles, items = tiles * splits;
    const int kb_total = (K + TILE_K - 1) / TILE_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TL::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], PERSISTENT_EPI_WARPS);     // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"((uint32_t)TL::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // item -> (split, weight tile, token tile); token tiles vary fastest so that the
    // CTAs of a wave share weight tiles in L2
    auto decode_item = [&](int item, int& m0, int& n0, int& kb_begin, int& n_kb, int& split) {
        split = item / tiles;
        const int t = item % tiles;
        m0 = (t / n_tiles) * M_STEP;
        n0 = (t % n_tiles) * BN;
        kb_begin = split * kb_per_split;
        n_kb = min(kb_total, kb_begin + kb_per_split) - kb_begin;
    };

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ loader
        int it = 0;                       // k-blocks issued so far, over all tiles
        bool waited = false;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x) {
            int m0, n0, kb_begin, n_kb, split;
            decode_item(item, m0, n0, kb_begin, n_kb, split);
            for (int i = 0; i < n_kb; ++i, ++it) {
                const int s = it % TL::STAGES;
                const uint32_t ph = (it / TL::STAGES) & 1;
                if (!mbar_wait(&empty[s], ph ^ 1)) {
                    atomicCAS(&g_gemm_status, 0, (1 << 8) | s);
                    *abort_flag = 1;
                    break;
                }
                uint8_t* st = smem + s * TL::STAGE_BYTES;
                mbar_expect_tx(&full[s], TL::STAGE_BYTES);
                const int kx = (kb_begin + i) * TILE_K;
                tma_load_2d(st, &map_w, kx, m0, &full[s]);
                if (GATED) tma_load_2d(st + TL::A_BYTES, &map_w2, kx, m0, &full[s]);
                if (QKV) tma_load_2d(st + TL::A_BYTES, &map_w, kx, m0 + TILE_M, &full[s]);
                if (!waited) {
                    // the weights never change: the first box is requested before the
                    // predecessor (which produces x) is known to have finished
                    pdl_wait();
                    waited = true;
                }
                tma_load_2d(st + TL::A_BYTES * (TOKM ? 2 : 1), &map_x, kx, n0, &full[s]);
            }
        }
        if (*abort_flag) {
            const int first = it > TL::STAGES ? it - TL::STAGES : 0;
            for (int i = first; i < it; ++i) mbar_wait(&full[i % TL::STAGES], (i / TL::STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ products
        constexpr uint32_t idesc = TOKM ? umma_idesc(BN, 2 * TILE_M) : umma_idesc(TILE_M, BN);
        int it = 0, li = 0;
        for (int item = blockIdx.x; item < items && !*abort_flag; item += gridDim.x, ++li) {
            int m0, n0, kb_begin, n_kb, split;
            decode_item(item, m0, n0, kb_begin, n_kb, split);
            const int as = li & 1;
            if (!mbar_wait(&acc_empty[as], ((li >> 1) & 1) ^ 1)) {
                atomicCAS(&g_gemm_status, 0, (4 << 8) | as);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + as * TL::ACC_COLS;
            for (int i = 0; i < n_kb; ++i, ++it) {
                const int s = it % TL::STAGES;
                const uint32_t ph = (it / TL::STAGES) & 1;
                if (!mbar_wait(&full[s], ph)) {
                    atomicCAS(&g_gemm_status, 0, (2 << 8) | s);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * TL::STAGE_BYTES);
                const uint32_t b_addr = a_addr + TL::A_BYTES * (TOKM ? 2 : 1);
#pragma unroll
                for (int k = 0; k < TILE_K / UMMA_K; ++k) {
                    const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    if (TOKM)
                        // the token tile is the M operand; the two weight tiles (gate and up,
                        // or 256 consecutive rows of q | k | v), one after the other in the
                        // stage, are one N operand of 256 rows
                        tc_mma_bf16(d_tmem, umma_desc(b_addr + k * UMMA_K * 2),
                                    umma_desc(a_addr + k * UMMA_K * 2), idesc, acc);
                    else
                        tc_mma_bf16(d_tmem, umma_desc(a_addr + k * UMMA_K * 2),
                                    umma_desc(b_addr + k * UMMA_K * 2), idesc, acc);
                }
                tc_commit(&empty[s]);
            }
            tc_commit(&acc_full[as]);
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue
        // Eight warps: a warp may read only the TMEM lanes of its quarter (warp % 4), so
        // two warps share each quarter and take half of the token columns each.  The
        // load of the next 16 columns is in flight while the current ones are worked.
        pdl_wait();
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        TO* wst = (TO*)(epi + (warp - 2) * (TL::EPI_BYTES / PERSISTENT_EPI_WARPS));
        constexpr int EPV = 16 / (int)sizeof(TO);                    // elements per 16 bytes
        constexpr int VPR = 32 / EPV;                                // 16-byte pieces per staged row
        // plain: BN token columns; gated: 128 feature columns (gate), the up values 128 further
        constexpr int HALF_COLS = (GATED ? TILE_M : BN) / 2;
        constexpr int UP_COL = GATED ? TILE_M : BN;
        static_assert(HALF_COLS % 32 == 0, "the column loop works in pairs of 16");
        static_assert(!TOKM || BN == 128, "these forms put a tile of 128 tokens on M");
        int li = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++li) {
            int m0, n0, kb_begin, n_kb, split;
            decode_item(item, m0, n0, kb_begin, n_kb, split);
            const int as = li & 1;
            bool ok = !*abort_flag && mbar_wait(&acc_full[as], (li >> 1) & 1);
            if (!ok) {
                if (!*abort_flag) atomicCAS(&g_gemm_status, 0, (3 << 8) | as);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const uint32_t lane_base =
                tmem_base + as * TL::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            const int f0 = m0 + quarter * 32;                        // this warp's first feature
            TO* gbase = out + (size_t)split * split_stride + (size_t)n0 * ldc + f0;
            const bool fast = f0 + 32 <= N && ldc % EPV == 0 && ((uintptr_t)gbase & 15) == 0;
            const int c_begin = half * HALF_COLS, c_end = c_begin + HALF_COLS;
            // gated: lanes are tokens, columns 0..127 gate features, 128..255 up features
            const int tok = n0 + quarter * 32 + lane;
            TO* grow = out + (size_t)tok * ldc + m0;
            const bool gfast = m0 + TILE_M <= N && ldc % EPV == 0 && ((uintptr_t)out & 15) == 0;

            auto release = [&]() {
                // every value of this accumulator that the warp needs is in registers
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[as]);
            };
            auto work = [&](const uint32_t (&r)[16], const uint32_t (&u)[16], int c) {
                if constexpr (GATED) {
                    float v[16];
                    if (act == 1) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            v[j] = silu_fast(__uint_as_float(r[j])) * __uint_as_float(u[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            v[j] = gelu_tanh_fast(__uint_as_float(r[j])) * __uint_as_float(u[j]);
                    }
                    if (tok < T) {
                        if (gfast) {
                            TO tmp[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) store_out<TO>(tmp + j, v[j]);
                            constexpr int NV = 16 * (int)sizeof(TO) / 16;
#pragma unroll
                            for (int q = 0; q < NV; ++q)
                                reinterpret_cast<uint4*>(grow + c)[q] =
                                    reinterpret_cast<const uint4*>(tmp)[q];
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (m0 + c + j < N) store_out<TO>(grow + c + j, v[j]);
                        }
                    }
                    return;
                }
                if (GATED) {
                    if (act == 1) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            store_out<TO>(wst + j * 32 + lane, silu_fast(__uint_as_float(r[j])) *
                                                                   __uint_as_float(u[j]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            store_out<TO>(wst + j * 32 + lane,
                                          gelu_tanh_fast(__uint_as_float(r[j])) *
                                              __uint_as_float(u[j]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        store_out<TO>(wst + j * 32 + lane, __uint_as_float(r[j]));
                }
                __syncwarp();
                const int rows = min(16, T - n0 - c);
                if (fast) {
#pragma unroll
                    for (int i = 0; i < 16 * VPR / 32; ++i) {
                        const int vi = lane + 32 * i, row = vi / VPR, part = vi % VPR;
                        if (row < rows)
                            *reinterpret_cast<uint4*>(gbase + (size_t)(c + row) * ldc + part * EPV) =
                                reinterpret_cast<const uint4*>(wst)[vi];
                    }
                } else {
                    for (int i = lane; i < 16 * 32; i += 32) {
                        const int row = i / 32, fl = i % 32;
                        if (row < rows && f0 + fl < N) gbase[(size_t)(c + row) * ldc + fl] = wst[i];
                    }
                }
                __syncwarp();
            };

            if (n_kb <= 0) {
                release();
                continue;
            }
            if constexpr (QKV) {
                qkv_epilogue(lane_base, m0, tok, half, T, qe);
                release();
                continue;
            }
            uint32_t ra[16], ua[16], rb[16], ub[16];
            tc_ld16(lane_base + c_begin, ra);
            if (GATED) tc_ld16(lane_base + UP_COL + c_begin, ua);
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 32) {
                tc_wait_ld();
                tc_ld16(lane_base + c + 16, rb);
                if (GATED) tc_ld16(lane_base + UP_COL + c + 16, ub);
                work(ra, ua, c);
                tc_wait_ld();
                if (c + 32 < c_end) {
                    tc_ld16(lane_base + c + 32, ra);
                    if (GATED) tc_ld16(lane_base + UP_COL + c + 32, ua);
                } else {
                    release();
                }
                work(rb, ub, c + 16);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)TL::TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------------------- CTA-pair form
// The gated product for prompts on two SMs per tile (tcgen05 cta_group::2).  The CTAs of
// a cluster of two share one product of M 256 x N 256 per k-step: each holds 128 of the
// 256 token rows (the M operand) and half of the N operand in its own shared memory, the
// even CTA the gate tile's 128 weight rows, the odd CTA the up tile's; each gets the
// accumulator of its own 128 tokens, columns 0..127 gate and 128..255 up, in its own
// tensor memory.  A CTA therefore takes 32 KB from L2 per k-block where the one-CTA form
// takes 48 KB for the same arithmetic, and the L2 feed (about 69 B/clk per SM while all
// SMs ask) no longer limits the mainloop.
//
// One thread of the even CTA issues the products for both.  Both CTAs load their own
// operands with TMA; all of a stage's bytes are counted on the even CTA's barrier.  The
// commit that follows a stage's products arrives on the "stage free" barrier of both
// CTAs, the commit after a tile's last product on both "accumulator full" barriers, and
// the epilogue warps of both CTAs arrive on the even CTA's "accumulator free" barrier.
// No load is multicast.  Every wait is bounded as in the other forms; nobody leaves
// before its partner has passed the final cluster barrier.
constexpr int PAIR_STAGE_BYTES = 2 * TILE_M * TILE_K * 2;             // 128 token rows + 128 weight rows
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_ACC_COLS = 2 * TILE_M;
constexpr int PAIR_EPI_BYTES = PERSISTENT_EPI_WARPS * 16 * 32 * 4;
constexpr int PAIR_SMEM = PAIR_STAGES * PAIR_STAGE_BYTES + PAIR_EPI_BYTES + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
// TMA tile load of a CTA pair: the bytes are counted on a barrier that may lie in the
// partner CTA (a shared::cluster address).  Not a multicast: one destination.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives, once the products issued so far are done, on the barrier at this shared-memory
// offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(smem_u32(bar)),
        "h"((uint16_t)3)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

__global__ void __launch_bounds__(PERSISTENT_THREADS, 1)
gemm_tcgen05_pair_gated_kernel(const __grid_constant__ CUtensorMap map_w,
                               const __grid_constant__ CUtensorMap map_w2,
                               const __grid_constant__ CUtensorMap map_x,
                               __nv_bfloat16* __restrict__ out, int T, int N, int K, long long ldc,
                               int act) {
    pdl_launch_next();
    typedef __nv_bfloat16 TO;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* epi = smem + PAIR_STAGES * PAIR_STAGE_BYTES;
    uint64_t* full = (uint64_t*)(epi + PAIR_EPI_BYTES);     // used in the even CTA
    uint64_t* empty = full + PAIR_STAGES;                   // one set per CTA
    uint64_t* acc_full = empty + PAIR_STAGES;               // [2], one set per CTA
    uint64_t* acc_empty = acc_full + 2;                     // [2], used in the even CTA
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                // 0: issues the products
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int f_tiles = (N + TILE_M - 1) / TILE_M;          // tiles of 128 features
    const int t_tiles = (T + 2 * TILE_M - 1) / (2 * TILE_M); // tiles of 256 tokens
    const int items = f_tiles * t_tiles;
    const int n_kb = (K + TILE_K - 1) / TILE_K;
    constexpr uint32_t STAGE_TX = 2 * PAIR_STAGE_BYTES;     // both CTAs' bytes of a stage

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 2 * PERSISTENT_EPI_WARPS);   // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the partner's barriers exist before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // item -> (feature tile, token tile); token tiles vary fastest so that the pairs of a
    // wave share weight tiles in L2
    auto decode_item = [&](int item, int& m0, int& n0) {
        m0 = (item / t_tiles) * TILE_M;
        n0 = (item % t_tiles) * 2 * TILE_M + (int)rank * TILE_M;     // this CTA's first token
    };

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ loader (both CTAs)
        int it = 0;
        bool waited = false;
        for (int item = pair; item < items && !*abort_flag; item += n_pairs) {
            int m0, n0;
            decode_item(item, m0, n0);
            for (int i = 0; i < n_kb; ++i, ++it) {
                const int s = it % PAIR_STAGES;
                const uint32_t ph = (it / PAIR_STAGES) & 1;
                if (!mbar_wait(&empty[s], ph ^ 1)) {
                    atomicCAS(&g_gemm_status, 0, (5 << 8) | s);
                    *abort_flag = 1;
                    break;
                }
                uint8_t* st = smem + s * PAIR_STAGE_BYTES;
                const uint32_t bar = mapa_u32(smem_u32(&full[s]), 0);
                if (rank == 0) mbar_expect_tx(&full[s], STAGE_TX);
                const int kx = i * TILE_K;
                // the weights never change: their box is requested before the predecessor
                // (which produces x) is known to have finished
                tma_load_2d_pair(st + TILE_M * TILE_K * 2, rank == 0 ? &map_w : &map_w2, kx, m0, bar);
                if (!waited) {
                    pdl_wait();
                    waited = true;
                }
                tma_load_2d_pair(st, &map_x, kx, n0, bar);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ------------------------------------------------------------ products (even CTA)
        constexpr uint32_t idesc = umma_idesc(2 * TILE_M, 2 * TILE_M);
        int it = 0, li = 0;
        for (int item = pair; item < items && !*abort_flag; item += n_pairs, ++li) {
            const int as = li & 1;
            if (!mbar_wait(&acc_empty[as], ((li >> 1) & 1) ^ 1)) {
                atomicCAS(&g_gemm_status, 0, (6 << 8) | as);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + as * PAIR_ACC_COLS;
            for (int i = 0; i < n_kb; ++i, ++it) {
                const int s = it % PAIR_STAGES;
                const uint32_t ph = (it / PAIR_STAGES) & 1;
                if (!mbar_wait(&full[s], ph)) {
                    atomicCAS(&g_gemm_status, 0, (7 << 8) | s);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * PAIR_STAGE_BYTES);      // tokens
                const uint32_t b_addr = a_addr + TILE_M * TILE_K * 2;               // weight rows
#pragma unroll
                for (int k = 0; k < TILE_K / UMMA_K; ++k)
                    tc_mma_bf16_pair(d_tmem, umma_desc(a_addr + k * UMMA_K * 2),
                                     umma_desc(b_addr + k * UMMA_K * 2), idesc,
                                     (i > 0 || k > 0) ? 1u : 0u);
                tc_commit_pair(&empty[s]);
            }
            if (*abort_flag) break;
            tc_commit_pair(&acc_full[as]);
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue (both CTAs)
        // lanes are this CTA's tokens, columns 0..127 gate and 128..255 up values of the
        // tile's features; two warps share each quarter of the lanes, 64 features each
        pdl_wait();
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        constexpr int EPV = 16 / (int)sizeof(TO);
        const uint32_t acc_empty_leader0 = mapa_u32(smem_u32(&acc_empty[0]), 0);
        const uint32_t acc_empty_leader1 = mapa_u32(smem_u32(&acc_empty[1]), 0);
        int li = 0;
        for (int item = pair; item < items; item += n_pairs, ++li) {
            int m0, n0;
            decode_item(item, m0, n0);
            const int as = li & 1;
            bool ok = !*abort_flag && mbar_wait(&acc_full[as], (li >> 1) & 1);
            if (!ok) {
                if (!*abort_flag) atomicCAS(&g_gemm_status, 0, (8 << 8) | as);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const uint32_t lane_base =
                tmem_base + as * PAIR_ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            const int tok = n0 + quarter * 32 + lane;
            TO* grow = out + (size_t)tok * ldc + m0;
            const bool gfast = m0 + TILE_M <= N && ldc % EPV == 0 && ((uintptr_t)out & 15) == 0;
            const int c_begin = half * (TILE_M / 2), c_end = c_begin + TILE_M / 2;

            auto release = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(as ? acc_empty_leader1 : acc_empty_leader0);
            };
            auto work = [&](const uint32_t (&r)[16], const uint32_t (&u)[16], int c) {
                float v[16];
                if (act == 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        v[j] = silu_fast(__uint_as_float(r[j])) * __uint_as_float(u[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        v[j] = gelu_tanh_fast(__uint_as_float(r[j])) * __uint_as_float(u[j]);
                }
                if (tok < T) {
                    if (gfast) {
                        TO tmp[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) tmp[j] = __float2bfloat16_rn(v[j]);
#pragma unroll
                        for (int q = 0; q < 2; ++q)
                            reinterpret_cast<uint4*>(grow + c)[q] =
                                reinterpret_cast<const uint4*>(tmp)[q];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (m0 + c + j < N) grow[c + j] = __float2bfloat16_rn(v[j]);
                    }
                }
            };
            uint32_t ra[16], ua[16], rb[16], ub[16];
            tc_ld16(lane_base + c_begin, ra);
            tc_ld16(lane_base + TILE_M + c_begin, ua);
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 32) {
                tc_wait_ld();
                tc_ld16(lane_base + c + 16, rb);
                tc_ld16(lane_base + TILE_M + c + 16, ub);
                work(ra, ua, c);
                tc_wait_ld();
                if (c + 32 < c_end) {
                    tc_ld16(lane_base + c + 32, ra);
                    tc_ld16(lane_base + TILE_M + c + 32, ua);
                } else {
                    release();
                }
                work(rb, ub, c + 16);
            }
        }
    }
    // An abort in one CTA leaves the partner to run into its own bounded waits.  Copies
    // still in flight into this CTA's shared memory land before the cluster barrier below
    // lets anybody leave only in a run without an abort; after an abort the result is
    // void anyway and the status word says so.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the partner has no product, commit or arrival left for us
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(512u)
                     : "memory");
    }
}

// ---------------------------------------------------------------- tensor maps
// A [rows, K] bf16 matrix with row stride ld (elements), read in boxes of
// [box_rows x 64]; cached by its geometry (weights are asked for every step).
int make_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld,
             int box_rows) {
    typedef std::tuple<const void*, long long, long long, long long, int> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key(ptr, rows, K, ld, box_rows);
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *out = it->second;
            return 0;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return agv_fail(-4, "linear: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return agv_fail(-4, "linear: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %lld, "
                        "ld %lld)", (int)r, rows, K, ld);
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 8192) cache.clear();
    cache[key] = *out;
    return 0;
}

template <int BN, int MODE, typename TO, int SLIM = 0>
int launch(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, void* out, int T,
           int N, int K, long long ldc, long long split_stride, int splits, int kb_per_split,
           int act, int cluster_reduce, cudaStream_t stream, int* argmax_out = nullptr) {
    using TL = Tile<BN, MODE, SLIM>;
    static_assert(MODE != 0 || BN * RED_LD * 4 <= TL::STAGES * TL::STAGE_BYTES,
                  "a partial tile must fit the ring of stages");
    AGV_REQUIRE(!cluster_reduce || BN * RED_LD * 4 <= TL::STAGES * TL::STAGE_BYTES,
                "linear: a partial tile of %d tokens does not fit the ring of stages", BN);
    auto kern = gemm_tcgen05_kernel<BN, MODE, TO, SLIM>;
    static bool configured = false;
    if (!configured) {
        AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TL::SMEM));
        configured = true;
    }
    constexpr int rows_per_cta = MODE == 2 ? TILE_M / 2 : TILE_M;
    dim3 grid((N + rows_per_cta - 1) / rows_per_cta, (T + BN - 1) / BN, splits);
    AGV_REQUIRE(grid.y <= 65535, "linear: %d tokens exceed the grid limit", T);
    if (cluster_reduce)
        agv_launch_cluster(kern, grid, GEMM_THREADS, TL::SMEM, stream,
                           dim3(1, 1, (unsigned)cluster_reduce), mw,
                           mw2, mx, (TO*)out, T, N, K, ldc, split_stride, kb_per_split, act,
                           cluster_reduce, (int*)nullptr);
    else
        agv_launch(kern, grid, GEMM_THREADS, TL::SMEM, stream, mw, mw2, mx, (TO*)out, T, N, K, ldc,
                   split_stride, kb_per_split, act, 0, argmax_out);
    AGV_LAUNCH_OK("gemm_tcgen05_kernel");
    return 0;
}

template <int BN, int MODE, typename TO>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx,
                      void* out, int T, int N, int K, long long ldc, long long split_stride,
                      int splits, int kb_per_split, int act, cudaStream_t stream,
                      const QkvEpilogue& qe = QkvEpilogue{}) {
    using TL = PTile<BN, MODE>;
    auto kern = gemm_tcgen05_persistent_kernel<BN, MODE, TO>;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TL::SMEM));
        int dev = 0;
        AGV_CUDA_OK(cudaGetDevice(&dev));
        AGV_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        configured = true;
    }
    constexpr int m_step = MODE == 3 ? 2 * TILE_M : TILE_M;
    const long long items =
        (long long)((N + m_step - 1) / m_step) * ((T + BN - 1) / BN) * splits;
    const int grid = (int)(items < sms ? items : sms);
    agv_launch(kern, grid, PERSISTENT_THREADS, TL::SMEM, stream, mw, mw2, mx, (TO*)out, T, N, K,
               ldc, split_stride, splits, kb_per_split, act, qe);
    AGV_LAUNCH_OK("gemm_tcgen05_persistent_kernel");
    return 0;
}

int launch_pair_gated(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx,
                      void* out, int T, int N, int K, long long ldc, int act, cudaStream_t stream) {
    auto kern = gemm_tcgen05_pair_gated_kernel;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         PAIR_SMEM));
        int dev = 0;
        AGV_CUDA_OK(cudaGetDevice(&dev));
        AGV_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        configured = true;
    }
    const long long items =
        (long long)((N + TILE_M - 1) / TILE_M) * ((T + 2 * TILE_M - 1) / (2 * TILE_M));
    long long pairs = sms / 2;
    if (items < pairs) pairs = items;
    agv_launch_cluster(kern, dim3((unsigned)(2 * pairs)), PERSISTENT_THREADS, PAIR_SMEM, stream,
                       dim3(2, 1, 1), mw, mw2, mx, (__nv_bfloat16*)out, T, N, K, ldc, act);
    AGV_LAUNCH_OK("gemm_tcgen05_pair_gated_kernel");
    return 0;
}

template <int MODE, typename TO>
int launch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx,
              void* out, int T, int N, int K, long long ldc, long long split_stride, int splits,
              int kb_per_split, int act, int cluster_reduce, cudaStream_t stream) {
#define AGV_BN_CASE(B)                                                                          \
    case B:                                                                                      \
        return launch<B, MODE, TO>(mw, mw2, mx, out, T, N, K, ldc, split_stride, splits,         \
                                   kb_per_split, act, cluster_reduce, stream)
    switch (bn) {
        AGV_BN_CASE(16);
        AGV_BN_CASE(32);
        AGV_BN_CASE(64);
        AGV_BN_CASE(128);
        case 256:
            if constexpr (MODE != 2)
                return launch<256, MODE, TO>(mw, mw2, mx, out, T, N, K, ldc, split_stride, splits,
                                             kb_per_split, act, cluster_reduce, stream);
    }
#undef AGV_BN_CASE
    return agv_fail(-1, "linear: no kernel for a token tile of %d", bn);
}

}  // namespace

// Whether the tensor-core kernel takes this shape: K and the row strides must
// be multiples of 8 elements (a TMA row stride is a multiple of 16 bytes) and
// the pointers 16-byte aligned.
AGV_API int agv_linear_tc_supported(int N, int K, long long lda) {
    return (N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0) ? 1 : 0;
}

// x: [T, K] bf16, row stride lda; w (and w2 for the gated form): [N, K] bf16
// dense; out: [T, N] (bf16 or f32, row stride ldc).  splits > 1 (plain form)
// cuts K into ranges that run in CTAs of their own.  With cluster 0 (f32 out
// only) out is [splits, T, N] partial sums, to be added by the consumer.  With
// cluster c in 2..8 (splits a multiple of c) every c CTAs of a tile form a
// thread-block cluster, add their partial sums through distributed shared
// memory in rank order, and out is [splits / c, T, N] (a plain [T, N] when
// splits == c; bf16 allowed then).  token_tile 0 lets the launcher choose.
AGV_API int agv_linear_tc(const void* x, const void* w, const void* w2, void* out, int T, int N,
                          int K, long long lda, long long ldc, int out_dtype, int act, int splits,
                          int cluster, int token_tile, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && N > 0 && K > 0, "linear: bad sizes T=%d N=%d K=%d", T, N, K);
    AGV_REQUIRE(K % 8 == 0 && lda % 8 == 0, "linear: the tensor-core kernel needs K (%d) and the "
                "row stride (%lld) to be multiples of 8", K, lda);
    AGV_REQUIRE(agv_aligned(x, 16) && agv_aligned(w, 16) && (!w2 || agv_aligned(w2, 16)),
                "linear: operands must be 16-byte aligned");
    AGV_REQUIRE(lda >= K && ldc >= N, "linear: row strides shorter than rows");
    AGV_REQUIRE(splits >= 1, "linear: splits must be >= 1");
    AGV_REQUIRE(splits == 1 || !w2 || (cluster == splits && T <= 64),
                "linear: the gated form splits K only over one cluster and for at most 64 tokens");
    AGV_REQUIRE(cluster == 0 || (cluster >= 2 && cluster <= 8 && splits % cluster == 0),
                "linear: a cluster holds 2 to 8 ranges of K and must divide the splits (%d, %d)",
                cluster, splits);
    AGV_REQUIRE(splits == 1 || splits == cluster || out_dtype == AGV_F32,
                "linear: partial sums in global memory need a 32-bit output");
    if (T == 0) return 0;
    int bn = token_tile;
    if (bn == 0) {
        bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
    }
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    int kb_per;
    if (cluster) {
        kb_per = (kb_total + splits - 1) / splits;   // trailing ranks may get no range of K
    } else {
        if (splits > kb_total) splits = kb_total;
        kb_per = (kb_total + splits - 1) / splits;
        splits = (kb_total + kb_per - 1) / kb_per;   // no empty split
    }
    // decoding through a gated layer: gate and up rows share a tile (see Tile)
    const bool half = w2 && T <= 64;
    CUtensorMap mw, mw2, mx;
    if (int rc = make_map(&mw, w, N, K, K, half ? TILE_M / 2 : TILE_M)) return rc;
    if (w2) {
        if (int rc = make_map(&mw2, w2, N, K, K, half ? TILE_M / 2 : TILE_M)) return rc;
    } else {
        mw2 = mw;
    }
    const bool persistent = T > 128 && !cluster && token_tile == 0 && getenv("AGV_GEMM_ONESHOT") == nullptr;
    if (persistent) {
        bn = w2 ? 128 : 256;
        if (!w2 && out_dtype == AGV_F32) {
            // the token tile that needs the least time: rounds of the SMs times the time
            // of a k-block, which is the slower of its four products (2 cycles per token
            // column, at least 256) and its bytes from L2 at the 69 B/clk an SM gets
            // while all SMs ask (measured)
            int sms = 148;
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
            const long long m_tiles = (N + TILE_M - 1) / TILE_M;
            long long best = -1;
            for (int cand : {256, 192, 128}) {
                const long long items = m_tiles * ((T + cand - 1) / cand) * splits;
                const long long products = cand * 2 < 256 ? 256 : cand * 2;
                const long long feed = (long long)(TILE_M + cand) * TILE_K * 2 / 69;
                const long long cost = ((items + sms - 1) / sms) * (products > feed ? products : feed);
                if (best < 0 || cost < best) {
                    best = cost;
                    bn = cand;
                }
            }
        }
    }
    if (int rc = make_map(&mx, x, T, K, lda, bn)) return rc;
    const long long split_stride = (long long)T * ldc;
    const int creduce = splits > 1 ? cluster : 0;
    if (persistent) {
        if (w2) {
            AGV_REQUIRE(out_dtype == AGV_BF16, "linear: the gated form writes bfloat16");
            static const bool pairs = getenv("AGAVE_B200_CTA_PAIRS") == nullptr ||
                                      getenv("AGAVE_B200_CTA_PAIRS")[0] != '0';
            if (pairs && T >= 2 * TILE_M)
                return launch_pair_gated(mw, mw2, mx, out, T, N, K, ldc, act, stream);
            return launch_persistent<128, 1, __nv_bfloat16>(mw, mw2, mx, out, T, N, K, ldc, 0, 1,
                                                            kb_total, act, stream);
        }
        if (out_dtype == AGV_BF16)
            return launch_persistent<256, 0, __nv_bfloat16>(mw, mw2, mx, out, T, N, K, ldc, 0, 1,
                                                            kb_total, act, stream);
        if (bn == 128)
            return launch_persistent<128, 0, float>(mw, mw2, mx, out, T, N, K, ldc, split_stride,
                                                    splits, kb_per, act, stream);
        if (bn == 192)
            return launch_persistent<192, 0, float>(mw, mw2, mx, out, T, N, K, ldc, split_stride,
                                                    splits, kb_per, act, stream);
        return launch_persistent<256, 0, float>(mw, mw2, mx, out, T, N, K, ldc, split_stride,
                                                splits, kb_per, act, stream);
    }
    if (w2) {
        AGV_REQUIRE(out_dtype == AGV_BF16, "linear: the gated form writes bfloat16");
        if (half && bn == 16) {
            // between two and three CTAs per SM: the form of which three fit (see Tile)
            int sms = 148;
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
            const long long ctas =
                (long long)((N + TILE_M / 2 - 1) / (TILE_M / 2)) * (creduce ? splits : 1);
            if (ctas > 2LL * sms && ctas <= 3LL * sms)
                return launch<16, 2, __nv_bfloat16, 1>(mw, mw2, mx, out, T, N, K, ldc, 0,
                                                       creduce ? splits : 1,
                                                       creduce ? kb_per : kb_total, act, creduce,
                                                       stream);
        }
        if (half)
            return launch_bn<2, __nv_bfloat16>(bn, mw, mw2, mx, out, T, N, K, ldc, 0,
                                               creduce ? splits : 1, creduce ? kb_per : kb_total,
                                               act, creduce, stream);
        return launch_bn<1, __nv_bfloat16>(bn, mw, mw2, mx, out, T, N, K, ldc, 0, 1, kb_total,
                                           act, 0, stream);
    }
    if (out_dtype == AGV_BF16)
        return launch_bn<0, __nv_bfloat16>(bn, mw, mw2, mx, out, T, N, K, ldc, 0,
                                           creduce ? splits : 1, creduce ? kb_per : kb_total, act,
                                           creduce, stream);
    if (out_dtype == AGV_F32)
        return launch_bn<0, float>(bn, mw, mw2, mx, out, T, N, K, ldc, split_stride, splits,
                                   kb_per, act, creduce, stream);
    return agv_fail(-1, "linear: unknown output dtype %d", out_dtype);
}

// out_idx[t] = first index of the greatest element of (x w^T)[t, :], for up to 128 rows
// of x: the product above (plain form, one range of K) with the arg max taken in its
// epilogue, so that the [T, N] result is never written (the head over the vocabulary
// when the next token is the greatest logit).  x: [T, K] bf16 with row stride lda;
// w: [N, K] bf16 dense.  Ties go to the lowest index.  Two such calls must not overlap
// on the device (they share a table of keys); calls on one stream do not.
AGV_API int agv_linear_tc_argmax(const void* x, const void* w, int* out_idx, int T, int N, int K,
                                 long long lda, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && T <= ARGMAX_MAX_TOKENS && N > 0 && K > 0,
                "linear_argmax: bad sizes T=%d (at most %d) N=%d K=%d", T, ARGMAX_MAX_TOKENS, N, K);
    AGV_REQUIRE(K % 8 == 0 && lda % 8 == 0 && lda >= K, "linear_argmax: K (%d) and the row stride "
                "(%lld) must be multiples of 8", K, lda);
    AGV_REQUIRE(agv_aligned(x, 16) && agv_aligned(w, 16) && out_idx,
                "linear_argmax: operands must be 16-byte aligned");
    if (T == 0) return 0;
    const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128;
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    CUtensorMap mw, mx;
    if (int rc = make_map(&mw, w, N, K, K, TILE_M)) return rc;
    if (int rc = make_map(&mx, x, T, K, lda, bn)) return rc;
#define AGV_ARGMAX_CASE(B)                                                                      \
    case B:                                                                                      \
        rc = launch<B, 0, float>(mw, mw, mx, nullptr, T, N, K, N, 0, 1, kb_total, 0, 0, stream,  \
                                 out_idx);                                                       \
        break
    int rc = -1;
    switch (bn) {
        AGV_ARGMAX_CASE(16);
        AGV_ARGMAX_CASE(32);
        AGV_ARGMAX_CASE(64);
        AGV_ARGMAX_CASE(128);
    }
#undef AGV_ARGMAX_CASE
    if (rc) return rc;
    agv_launch(argmax_finish_kernel, dim3(1), dim3(ARGMAX_MAX_TOKENS), 0, stream, out_idx, T);
    AGV_LAUNCH_OK("argmax_finish_kernel");
    return 0;
}

// Whether agv_qkv_prefill_tc takes a layer of these sizes.
AGV_API int agv_qkv_prefill_tc_supported(int hd, int rotary_dim, int K, long long lda,
                                         long long row_stride) {
    return ((hd == 64 || hd == 128 || hd == 256) && (rotary_dim == 0 || rotary_dim == hd) &&
            K % 8 == 0 && lda % 8 == 0 && row_stride % 8 == 0) ? 1 : 0;
}

// The q | k | v projection of a prompt step with everything that follows it up to the
// attention in its epilogue: qkv [T, (nh + 2 nkv) * hd] (bfloat16, row stride in elements)
// receives q and k normed (wq / wk, [hd], or null) and rotated (cos / sin, [T, hd / 2], or
// null) and v as projected; k and v also go to the layer's cache pools (unless k_pool is
// null) and the values, transposed, to vt (unless null; see VtWrite).  x: [T, K] bf16 with
// row stride lda; w: [(nh + 2 nkv) * hd, K] bf16 dense, rows q | k | v.
AGV_API int agv_qkv_prefill_tc(const void* x, const void* w, int T, int K, long long lda, void* qkv,
                               long long row_stride, int nh, int nkv, int hd, const float* wq,
                               const float* wk, float eps, const float* cosv, const float* sinv,
                               const int* positions, void* k_pool, void* v_pool,
                               const int* page_table, const int* slots, const int* lens,
                               const int* seq_index, int max_pages, int page, int cap, void* vt,
                               long long vt_ld, const int* cu_seqlens, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && K > 0 && nh > 0 && nkv > 0, "qkv_prefill: bad sizes");
    AGV_REQUIRE(agv_qkv_prefill_tc_supported(hd, cosv ? hd : 0, K, lda, row_stride),
                "qkv_prefill: head_dim %d, K %d or a row stride is not supported", hd, K);
    const int N = (nh + 2 * nkv) * hd;
    AGV_REQUIRE(row_stride >= N && lda >= K, "qkv_prefill: row strides shorter than rows");
    AGV_REQUIRE(agv_aligned(x, 16) && agv_aligned(w, 16) && agv_aligned(qkv, 16) &&
                agv_aligned(wq, 16) && agv_aligned(wk, 16) && agv_aligned(cosv, 16) &&
                agv_aligned(sinv, 16) && agv_aligned(k_pool, 16) && agv_aligned(v_pool, 16),
                "qkv_prefill: operands must be 16-byte aligned");
    AGV_REQUIRE(!cosv || sinv, "qkv_prefill: cos without sin");
    AGV_REQUIRE(!k_pool || (v_pool && page_table && slots && lens && seq_index && positions &&
                            page > 0 && cap > 0 && max_pages > 0),
                "qkv_prefill: incomplete cache arguments");
    AGV_REQUIRE(!vt || (seq_index && positions && cu_seqlens && vt_ld % 64 == 0),
                "qkv_prefill: the transposed values need seq_index, positions and cu_seqlens");
    if (T == 0) return 0;
    CUtensorMap mw, mx;
    if (int rc = make_map(&mw, w, N, K, K, TILE_M)) return rc;
    if (int rc = make_map(&mx, x, T, K, lda, TILE_M)) return rc;
    QkvEpilogue qe{(__nv_bfloat16*)qkv, row_stride, nh, nkv, hd, wq, wk, eps, cosv, sinv, positions,
                   CacheWrite{k_pool, v_pool, page_table, slots, lens, seq_index, max_pages, page, cap},
                   VtWrite{(__nv_bfloat16*)vt, vt_ld, cu_seqlens, seq_index}};
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    return launch_persistent<128, 3, __nv_bfloat16>(mw, mw, mx, nullptr, T, N, K, 0, 0, 1, kb_total,
                                                    0, stream, qe);
}

// The number of partial sums agv_linear_tc will really write for these sizes.
AGV_API int agv_linear_tc_splits(int K, int splits) {
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    if (splits > kb_total) splits = kb_total;
    if (splits < 1) splits = 1;
    const int kb_per = (kb_total + splits - 1) / splits;
    return (kb_total + kb_per - 1) / kb_per;
}

// Reads and clears the status word of the tensor-core kernels: 0, or
// (role << 8 | stage) of the first bounded wait that gave up.
AGV_API int agv_linear_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
    return v;
}
