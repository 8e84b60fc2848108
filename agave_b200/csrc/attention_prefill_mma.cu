// Prompt attention on the tensor cores (bfloat16): a flash-style kernel over the
// step's own keys and values, causal with an optional window, ragged over the
// sequences of a batch.
//
// One CTA of four warps owns 64 consecutive query tokens of one sequence and
// one query head; each warp owns 16 of them.  Keys and values come in tiles of
// 64 positions through cp.async into swizzled shared memory; S = Q K^T and
// O += P V are mma.sync m16n8k16 products with 32-bit accumulators; the running
// maximum, the running sum and the rescaling of O are 32-bit.  Only the tiles a
// query tile can see (causal bound, window start) are visited, and the bounds
// are applied per element inside them.
//
// Reference: online softmax per (token, head) over KV tiles of 32
// (src/backend/kernels/cuda/sdpa_prefill.zig:26-216); score = (q . k) * scale,
// kv head = h / (nh / nkv) (src/backend/kernels/cpu/sdpa.zig:36-37,58); window
// start sl - W (src/models/gemma4.zig:1153-1155).
#include "common.cuh"

namespace {

constexpr int FA_N = 64;      // keys per tile; a CTA of NW warps owns NW * 16 query rows

__device__ __forceinline__ unsigned smem_addr(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm4(unsigned addr, unsigned (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(unsigned addr, unsigned (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const unsigned (&a)[4], unsigned b0,
                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Tiles are [rows][HDP] bf16; the 16-byte chunk c of row r sits at chunk
// (c & ~7) | ((c ^ r) & 7), so eight rows read at one column hit eight banks.
template <int HDP>
__device__ __forceinline__ int swz(int row, int chunk) {
    return row * HDP + (((chunk & ~7) | ((chunk ^ row) & 7)) << 3);
}

// Copies rows [row0, row0 + ROWS) x dims [0, hd) of a [*, stride] matrix into a
// swizzled tile; rows at or beyond row_end and dims at or beyond hd become zero.
template <int HDP, int ROWS, int THREADS>
__device__ __forceinline__ void load_tile(__nv_bfloat16* tile, const __nv_bfloat16* src,
                                          long long stride, int row0, int row_end, int hd) {
    constexpr int CPR = HDP / 8;                       // chunks per row
    for (int i = threadIdx.x; i < ROWS * CPR; i += THREADS) {
        const int r = i / CPR, c = i % CPR;
        __nv_bfloat16* dst = tile + swz<HDP>(r, c);
        if (row0 + r < row_end && c * 8 < hd)
            cp16(dst, src + (size_t)(row0 + r) * stride + c * 8);
        else
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
}

template <int HDP, int NW>
__global__ void __launch_bounds__(NW * 32)
attention_prefill_mma_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride,
                             const __nv_bfloat16* __restrict__ k,
                             const __nv_bfloat16* __restrict__ v, long long kv_stride,
                             __nv_bfloat16* __restrict__ out, const int* __restrict__ cu_seqlens,
                             int nh, int nkv, int hd, float scale_log2e, int window) {
    pdl_wait();
    pdl_launch_next();
    constexpr int FA_M = NW * 16, FA_THREADS = NW * 32;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* Ks = Qs + FA_M * HDP;
    __nv_bfloat16* Vs = Ks + FA_N * HDP;

    const int b = blockIdx.z, h = blockIdx.y;
    const int seq0 = cu_seqlens[b], len = cu_seqlens[b + 1] - seq0;
    // tiles at the end of a sequence walk the most key tiles: they are scheduled first
    const int m0 = (gridDim.x - 1 - blockIdx.x) * FA_M;
    if (m0 >= len) return;
    const int g = h / (nh / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;

    const __nv_bfloat16* qb = q + (size_t)seq0 * q_stride + (size_t)h * hd;
    const __nv_bfloat16* kb = k + (size_t)seq0 * kv_stride + (size_t)g * hd;
    const __nv_bfloat16* vb = v + (size_t)seq0 * kv_stride + (size_t)g * hd;

    // visible key range of this query tile: causal end, window start
    const int j_hi = min(m0 + FA_M - 1, len - 1);
    const int j_lo = window > 0 ? max(0, m0 - window + 1) : 0;
    const int t_lo = j_lo / FA_N, t_hi = j_hi / FA_N;

    load_tile<HDP, FA_M, FA_THREADS>(Qs, qb, q_stride, m0, len, hd);
    load_tile<HDP, FA_N, FA_THREADS>(Ks, kb, kv_stride, t_lo * FA_N, len, hd);
    cp_commit();
    load_tile<HDP, FA_N, FA_THREADS>(Vs, vb, kv_stride, t_lo * FA_N, len, hd);
    cp_commit();

    float o[HDP / 8][4];
#pragma unroll
    for (int i = 0; i < HDP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float row_m[2] = {-INFINITY, -INFINITY}, row_l[2] = {0.f, 0.f};
    const int qrow = m0 + warp * 16 + gid;             // this thread's rows: qrow, qrow + 8

    for (int t = t_lo; t <= t_hi; ++t) {
        cp_wait<1>();                                   // K (and Q) of this tile have landed
        __syncthreads();
        // ---- S = Q K^T for 16 rows x 64 keys
        float s[FA_N / 8][4];
#pragma unroll
        for (int i = 0; i < FA_N / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HDP / 16; ++kk) {
            unsigned a[4];
            ldsm4(smem_addr(Qs + swz<HDP>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4))), a);
#pragma unroll
            for (int nn = 0; nn < FA_N / 16; ++nn) {
                unsigned bfr[4];
                const int mat = lane >> 3, r = lane & 7;
                ldsm4(smem_addr(Ks + swz<HDP>(nn * 16 + r + (mat >> 1) * 8, kk * 2 + (mat & 1))),
                      bfr);
                mma16816(s[nn * 2], a, bfr[0], bfr[1]);
                mma16816(s[nn * 2 + 1], a, bfr[2], bfr[3]);
            }
        }
        __syncthreads();                                // every warp is done with this K tile
        if (t < t_hi) load_tile<HDP, FA_N, FA_THREADS>(Ks, kb, kv_stride, (t + 1) * FA_N, len, hd);
        cp_commit();
        // ---- bounds, running maximum and sum
        const int j0 = t * FA_N;
        float mx[2] = {row_m[0], row_m[1]};
#pragma unroll
        for (int i = 0; i < FA_N / 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + i * 8 + tig * 2 + (e & 1);
                const int p = qrow + (e >> 1) * 8;
                const bool ok = j <= p && j < len && (window <= 0 || j > p - window);
                const float val = ok ? s[i][e] * scale_log2e : -INFINITY;
                s[i][e] = val;
                mx[e >> 1] = fmaxf(mx[e >> 1], val);
            }
        }
        float alpha[2], base[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            base[rr] = mx[rr] == -INFINITY ? 0.f : mx[rr];       // a row that sees nothing yet
            alpha[rr] = exp2f(row_m[rr] - base[rr]);
            row_m[rr] = mx[rr];
            row_l[rr] *= alpha[rr];
        }
        unsigned pa[FA_N / 16][4];
#pragma unroll
        for (int i = 0; i < FA_N / 8; ++i) {
            const float p0 = exp2f(s[i][0] - base[0]), p1 = exp2f(s[i][1] - base[0]);
            const float p2 = exp2f(s[i][2] - base[1]), p3 = exp2f(s[i][3] - base[1]);
            row_l[0] += p0 + p1;
            row_l[1] += p2 + p3;
            pa[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
            pa[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int i = 0; i < HDP / 8; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        cp_wait<1>();                                   // V of this tile has landed
        __syncthreads();
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < FA_N / 16; ++kk) {
#pragma unroll
            for (int nn = 0; nn < HDP / 16; ++nn) {
                unsigned bfr[4];
                const int mat = lane >> 3, r = lane & 7;
                ldsm4t(smem_addr(Vs + swz<HDP>(kk * 16 + r + (mat & 1) * 8, nn * 2 + (mat >> 1))),
                       bfr);
                mma16816(o[nn * 2], pa[kk], bfr[0], bfr[1]);
                mma16816(o[nn * 2 + 1], pa[kk], bfr[2], bfr[3]);
            }
        }
        __syncthreads();                                // every warp is done with this V tile
        if (t < t_hi) load_tile<HDP, FA_N, FA_THREADS>(Vs, vb, kv_stride, (t + 1) * FA_N, len, hd);
        cp_commit();
    }
    // ---- normalise and store
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        row_l[rr] += __shfl_xor_sync(0xffffffffu, row_l[rr], 1);
        row_l[rr] += __shfl_xor_sync(0xffffffffu, row_l[rr], 2);
    }
    const float inv0 = row_l[0] > 0.f ? 1.0f / row_l[0] : 0.f;
    const float inv1 = row_l[1] > 0.f ? 1.0f / row_l[1] : 0.f;
    __nv_bfloat16* ob = out + (size_t)seq0 * (size_t)(nh * hd) + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < HDP / 8; ++i) {
        const int d = i * 8 + tig * 2;
        if (d < hd) {
            if (qrow < len)
                *reinterpret_cast<unsigned*>(ob + (size_t)qrow * (nh * hd) + d) =
                    pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
            if (qrow + 8 < len)
                *reinterpret_cast<unsigned*>(ob + (size_t)(qrow + 8) * (nh * hd) + d) =
                    pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
        }
    }
}

template <int HDP, int NW>
int launch_fa(const void* q, long long q_stride, const void* k, const void* v, long long kv_stride,
              void* out, const int* cu_seqlens, int B, int max_len, int nh, int nkv, int hd,
              float scale, int window, cudaStream_t stream) {
    auto kern = attention_prefill_mma_kernel<HDP, NW>;
    constexpr int FA_M = NW * 16, FA_THREADS = NW * 32;
    constexpr int smem = (FA_M + 2 * FA_N) * HDP * 2;
    static bool configured = false;
    if (!configured) {
        AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    dim3 grid((max_len + FA_M - 1) / FA_M, nh, B);
    agv_launch(kern, grid, FA_THREADS, smem, stream, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
        kv_stride, (__nv_bfloat16*)out, cu_seqlens, nh, nkv, hd,
        scale * 1.4426950408889634f, window);
    AGV_LAUNCH_OK("attention_prefill_mma_kernel");
    return 0;
}

}  // namespace

// Whether the tensor-core prompt attention takes this head size: a multiple of
// 8 up to 256 with 16-byte aligned rows.
AGV_API int agv_attention_prefill_mma_supported(int hd, long long q_stride, long long kv_stride) {
    return (hd > 0 && hd % 8 == 0 && hd <= 256 && q_stride % 8 == 0 && kv_stride % 8 == 0) ? 1 : 0;
}

// Whole prompts that start at position 0, bfloat16.  q: [T, nh, hd] rows of
// stride q_stride; k, v: [T, nkv, hd] rows of stride kv_stride; out: [T, nh * hd]
// dense; cu_seqlens: [B + 1] first token of each sequence; max_len: the
// greatest sequence length (sizes the grid).  window 0: no window.
AGV_API int agv_attention_prefill_mma(const void* q, long long q_stride, const void* k,
                                      const void* v, long long kv_stride, void* out,
                                      const int* cu_seqlens, int B, int max_len, int nh, int nkv,
                                      int hd, float scale, int window, cudaStream_t stream) {
    AGV_REQUIRE(B >= 0 && nh > 0 && nkv > 0 && hd > 0 && max_len >= 0, "attention: bad sizes");
    AGV_REQUIRE(nh % nkv == 0, "attention: %d heads are not a multiple of %d kv heads", nh, nkv);
    AGV_REQUIRE(agv_attention_prefill_mma_supported(hd, q_stride, kv_stride),
                "attention: the tensor-core kernel needs head_dim (%d) a multiple of 8 up to 256 "
                "and row strides that are multiples of 8", hd);
    AGV_REQUIRE(agv_aligned(q, 16) && agv_aligned(k, 16) && agv_aligned(v, 16) &&
                agv_aligned(out, 4), "attention: operands must be 16-byte aligned");
    AGV_REQUIRE(window >= 0, "attention: negative window");
    AGV_REQUIRE(B <= 65535 && nh <= 65535, "attention: batch or head count exceeds the grid limit");
    if (B == 0 || max_len == 0) return 0;
    // Four warps (64 query rows) per CTA.  The eight-warp form is kept for
    // comparison: on a 2,048-token sequence it took 146 us where this takes 101.
    const bool wide = false;
#define AGV_FA(HDP)                                                                             \
    return wide ? launch_fa<HDP, 8>(q, q_stride, k, v, kv_stride, out, cu_seqlens, B, max_len,  \
                                    nh, nkv, hd, scale, window, stream)                          \
                : launch_fa<HDP, 4>(q, q_stride, k, v, kv_stride, out, cu_seqlens, B, max_len,  \
                                    nh, nkv, hd, scale, window, stream)
    if (hd <= 64) AGV_FA(64);
    if (hd <= 128) AGV_FA(128);
    AGV_FA(256);
#undef AGV_FA
}
