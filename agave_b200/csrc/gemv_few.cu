// Projections of a decode step with one to four tokens: out[T, N] = x[T, K] w[N, K]^T
// (or the gated pair act(x wg^T) * (x wu^T)), one dot product per warp and output row,
// bfloat16 operands, 32-bit sums.
//
// With so few tokens the tensor cores have nothing to gain: the weight is streamed once
// whatever multiplies it, and what a step costs is the number of kernels in its chain
// and the trips to memory inside each.  So this kernel also takes the join that
// precedes a projection into its own prologue,
//     h_out = h_in + norm(y; w_post)   (or h_in + y; or h_in itself without y),
//     x     = bfloat16(norm(h_out; w_next)),
// computed by every CTA for itself from the [T, K] rows (a few KB for these T), with CTA
// 0 writing h_out; h_in and h_out are different buffers, because the other CTAs still
// read h_in.  A layer then is five kernels instead of seven: q/k/v (join of the layer
// before), attention, output, gate/up (join), down.
//
// Before the dependency wait a warp loads its first two batches of weight rows and the CTA
// copies the two norm weights into shared memory; after it the token rows come in as one
// group of copies.  (Asking the L2 cache for all of a CTA's rows up front as well,
// prefetch.global.L2, made the stream slower: 100 against 72 us for the 27B gate/up.)
// x is rounded to bfloat16 before it is multiplied, as the tensor-core products round it,
// so a token decoded alone and one decoded in a larger batch see the same operands.
//
// Reference: one dot product per output row with 32-bit accumulation, bfloat16 weights
// converted in the loop (src/backend/kernels/cuda/gemv_bf16.zig:6-24); the norms as
// src/backend/kernels/cpu/norm.zig:29-39 with the (1 + w) of src/models/gemma3.zig:908-954
// formed at load time.
#include "common.cuh"

namespace {

constexpr int GF_THREADS = 256;
constexpr int GF_WARPS = GF_THREADS / 32;
constexpr int GF_MAX_SMEM = 200 * 1024;

struct FewJoin {
    const float* h_in;       // [T, K] residual stream as the step left it
    float* h_out;            // [T, K] the stream after the join (written by CTA 0), or null
    const float* y;          // [T, K] branch output to add, or null
    const float* w_post;     // [K] norm of the branch before it is added, or null
    const float* w_next;     // [K] norm that forms x
    float eps_post, eps_next;
};

__device__ __forceinline__ void gf_copy16(void* smem_dst, const void* gmem_src) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void gf_copies_done() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// Block-wide sums of T values per thread; every thread gets all T results.  scratch:
// GF_WARPS * T floats that nobody writes again in this launch (one barrier suffices then).
template <int T>
__device__ __forceinline__ void gf_block_sums(float (&v)[T], float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int t = 0; t < T; ++t) {
        v[t] = warp_sum(v[t]);
        if (lane == 0) scratch[warp * T + t] = v[t];
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < T; ++t) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GF_WARPS; ++w) s += scratch[w * T + t];      // in warp order
        v[t] = s;
    }
}

// eight bfloat16 times eight bfloat16, added to acc in 32-bit
__device__ __forceinline__ float gf_dot8(const uint4& w, const uint4& x, float acc) {
    const unsigned wv[4] = {w.x, w.y, w.z, w.w}, xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc = fmaf(__uint_as_float(wv[i] << 16), __uint_as_float(xv[i] << 16), acc);
        acc = fmaf(__uint_as_float(wv[i] & 0xffff0000u), __uint_as_float(xv[i] & 0xffff0000u), acc);
    }
    return acc;
}

__device__ __forceinline__ float gf_gelu_tanh(float t) {
    const float u = 0.7978845608028654f * (t + 0.044715f * t * t * t);
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(u));
    return 0.5f * t * (1.0f + th);
}
__device__ __forceinline__ float gf_silu(float t) { return __fdividef(t, 1.0f + __expf(-t)); }

template <int T, int GATED>
__global__ void __launch_bounds__(GF_THREADS, 2)
gemv_few_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ W2, int N,
                int K, const __nv_bfloat16* __restrict__ x_direct, long long ldx, FewJoin j,
                void* __restrict__ out, long long ldo, int act, int rows_per_cta, int ks,
                int part_off) {
    pdl_launch_next();
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float scratch[2][GF_WARPS * T];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long r0 = (long long)blockIdx.x * rows_per_cta;
    const long long r1 = r0 + rows_per_cta < N ? r0 + rows_per_cta : N;

    // ---- before the wait: the norm weights into shared memory, the first weight batches
    // join:   [v: T x K 32-bit][h: T x K 32-bit, afterwards x in bfloat16][w_post, w_next: 2 K]
    // direct: [x: T x K bfloat16]
    // (x as 32-bit values in shared memory, with nothing to unpack per use, was slower: it
    // doubles what every piece of a weight row reads from shared memory)
    float* vs = reinterpret_cast<float*>(smem);
    float* hs = vs + (size_t)T * K;
    float* wp = hs + (size_t)T * K;
    float* wn = wp + K;
    __nv_bfloat16* xs = x_direct ? reinterpret_cast<__nv_bfloat16*>(smem)
                                 : reinterpret_cast<__nv_bfloat16*>(hs);
    if (!x_direct) {
        for (int i = tid * 4; i < K; i += GF_THREADS * 4) {
            if (j.w_post) gf_copy16(wp + i, j.w_post + i);
            gf_copy16(wn + i, j.w_next + i);
        }
    }
    const int K8 = K >> 3;
    const uint4* xq = reinterpret_cast<const uint4*>(xs);
    const int rpr = GF_WARPS / ks, slice = warp % ks, rl = warp / ks;
    const int per_slice = (K8 + ks - 1) / ks;
    const int c_lo = slice * per_slice, c_hi = min(K8, c_lo + per_slice);
    constexpr int U = GATED ? 5 : 8;          // 16-byte pieces of a row per lane and batch
    const int bpr = max(1, (c_hi - c_lo + 32 * U - 1) / (32 * U));       // batches per row
    const int my_rows = r0 + rl < r1 ? (int)((r1 - r0 - rl + rpr - 1) / rpr) : 0;
    const int n_batches = my_rows * bpr;
    float* part = reinterpret_cast<float*>(smem + part_off);   // [row of the CTA][slice][g | u][T]
    uint4 wa[U], ua[U], wb[U], ub[U];
    auto ask = [&](int batch, uint4 (&w)[U], uint4 (&u)[U]) {
        const long long r = r0 + rl + (long long)(batch / bpr) * rpr;
        const int c0 = c_lo + (batch % bpr) * 32 * U + lane;
        const uint4* wr = reinterpret_cast<const uint4*>(W + r * K);
        const uint4* ur = GATED ? reinterpret_cast<const uint4*>(W2 + r * K) : wr;
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int c = c0 + 32 * i;
            w[i] = c < c_hi ? __ldg(wr + c) : make_uint4(0, 0, 0, 0);
            if (GATED) u[i] = c < c_hi ? __ldg(ur + c) : make_uint4(0, 0, 0, 0);
        }
    };
    // (the weights are nobody's output: the first two batches are asked for before the wait;
    // so are the join's arguments, whose first read from the parameter bank is a slow one)
    if (n_batches > 0) ask(0, wa, ua);
    if (n_batches > 1) ask(1, wb, ub);
    const float* const jy = j.y;
    const float* const jh = j.h_in;
    float* const jho = j.h_out;
    const float* const jwp = j.w_post;
    const float eps_post = j.eps_post, eps_next = j.eps_next;
    const bool add = jy != nullptr;
    pdl_wait();
    if (x_direct) {
        for (int i = tid * 8; i < T * K; i += GF_THREADS * 8) {
            const int t = i / K, c = i - t * K;
            gf_copy16(xs + i, x_direct + (size_t)t * ldx + c);
        }
        gf_copies_done();
        __syncthreads();
    } else {
        for (int i = tid * 4; i < T * K; i += GF_THREADS * 4) {
            if (add) gf_copy16(vs + i, jy + i);
            gf_copy16(hs + i, jh + i);
        }
        gf_copies_done();
        __syncthreads();
        // three passes over the rows, four values of a row per thread and access (the loops
        // are short chains of shared-memory trips: wide accesses and several of them in
        // flight, or a pass costs a microsecond)
        const int K4 = K >> 2;
        float rs[T];
#pragma unroll
        for (int t = 0; t < T; ++t) rs[t] = 1.f;
        if (add && jwp) {
            float ss[T];
#pragma unroll
            for (int t = 0; t < T; ++t) {
                ss[t] = 0.f;
#pragma unroll 2
                for (int c = tid; c < K4; c += GF_THREADS) {
                    const float4 v = reinterpret_cast<const float4*>(vs + (size_t)t * K)[c];
                    ss[t] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
            }
            gf_block_sums<T>(ss, scratch[0]);
#pragma unroll
            for (int t = 0; t < T; ++t) rs[t] = 1.0f / sqrtf(ss[t] / (float)K + eps_post);
        }
        float ss2[T];
        const bool writer = blockIdx.x == 0 && jho != nullptr;
#pragma unroll
        for (int t = 0; t < T; ++t) {
            ss2[t] = 0.f;
#pragma unroll 2
            for (int c = tid; c < K4; c += GF_THREADS) {
                float4 v = reinterpret_cast<const float4*>(hs + (size_t)t * K)[c];
                if (add) {
                    const float4 y4 = reinterpret_cast<const float4*>(vs + (size_t)t * K)[c];
                    if (jwp) {
                        const float4 w4 = reinterpret_cast<const float4*>(wp)[c];
                        v.x += y4.x * rs[t] * w4.x; v.y += y4.y * rs[t] * w4.y;
                        v.z += y4.z * rs[t] * w4.z; v.w += y4.w * rs[t] * w4.w;
                    } else {
                        v.x += y4.x; v.y += y4.y; v.z += y4.z; v.w += y4.w;
                    }
                }
                reinterpret_cast<float4*>(vs + (size_t)t * K)[c] = v;
                if (writer) reinterpret_cast<float4*>(jho + (size_t)t * K)[c] = v;
                ss2[t] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        gf_block_sums<T>(ss2, scratch[1]);       // (its barrier: h is read, x may go there)
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const float r2 = 1.0f / sqrtf(ss2[t] / (float)K + eps_next);
#pragma unroll 2
            for (int c = tid; c < K4; c += GF_THREADS) {
                const float4 v = reinterpret_cast<const float4*>(vs + (size_t)t * K)[c];
                const float4 w4 = reinterpret_cast<const float4*>(wn)[c];
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * r2 * w4.x, v.y * r2 * w4.y);
                const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * r2 * w4.z, v.w * r2 * w4.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const unsigned*>(&lo);
                pk.y = *reinterpret_cast<const unsigned*>(&hi);
                reinterpret_cast<uint2*>(xs + (size_t)t * K)[c] = pk;
            }
        }
        __syncthreads();
    }

    // ---- the rows.  ks warps share a row, each on a range of K (so that a weight with few
    // rows still has every warp streaming); a warp walks its rows' ranges as batches of U
    // 16-byte pieces per lane and asks for the next batch before it multiplies this one,
    // so its loads never stop.  What the warps of a row found is added in order at the end.
    float acc[T], acu[T];
#pragma unroll
    for (int t = 0; t < T; ++t) acc[t] = acu[t] = 0.f;
    auto use = [&](int batch, const uint4 (&w)[U], const uint4 (&u)[U]) {
        const int c0 = c_lo + (batch % bpr) * 32 * U + lane;
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int c = min(c0 + 32 * i, K8 - 1);         // (beyond the range w is zero)
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const uint4 x = xq[(size_t)t * K8 + c];
                acc[t] = gf_dot8(w[i], x, acc[t]);
                if (GATED) acu[t] = gf_dot8(u[i], x, acu[t]);
            }
        }
        if (batch % bpr == bpr - 1) {                        // the row's range is done
            const int row = rl + (batch / bpr) * rpr;        // row of the CTA
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float g = warp_sum(acc[t]);
                const float u2 = GATED ? warp_sum(acu[t]) : 0.f;
                if (lane == 0) {
                    part[((row * ks + slice) * 2) * T + t] = g;
                    part[((row * ks + slice) * 2 + 1) * T + t] = u2;
                }
                acc[t] = acu[t] = 0.f;
            }
        }
    };
    for (int bt = 0; bt < n_batches; bt += 2) {
        if (bt > 0 && bt + 1 < n_batches) ask(bt + 1, wb, ub);
        use(bt, wa, ua);
        if (bt + 2 < n_batches) ask(bt + 2, wa, ua);
        if (bt + 1 < n_batches) use(bt + 1, wb, ub);
    }
    __syncthreads();
    const int rows_here = (int)(r1 - r0);
    for (int i = tid; i < rows_here * T; i += GF_THREADS) {
        const int row = i / T, t = i - row * T;
        float g = 0.f, u = 0.f;
        for (int q = 0; q < ks; ++q) {                        // in the order of the ranges
            g += part[((row * ks + q) * 2) * T + t];
            u += part[((row * ks + q) * 2 + 1) * T + t];
        }
        if (GATED)
            reinterpret_cast<__nv_bfloat16*>(out)[(size_t)t * ldo + r0 + row] =
                __float2bfloat16_rn((act == 1 ? gf_silu(g) : gf_gelu_tanh(g)) * u);
        else
            reinterpret_cast<float*>(out)[(size_t)t * ldo + r0 + row] = g;
    }
}

size_t gf_smem(int T, int K, bool join) {
    return join ? (size_t)T * K * 8 + (size_t)K * 8 : (size_t)T * K * 2;
}

template <int T, int GATED>
int gf_launch(const void* w, const void* w2, int N, int K, const void* x, long long ldx,
              const FewJoin& j, void* out, long long ldo, int act, cudaStream_t stream) {
    auto kern = gemv_few_kernel<T, GATED>;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GF_MAX_SMEM));
        int dev = 0;
        AGV_CUDA_OK(cudaGetDevice(&dev));
        AGV_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        configured = true;
    }
    // About two CTAs per SM.  A weight with fewer rows than that many warps gets 2, 4 or 8
    // warps per row, each on a range of K of at least 32 16-byte pieces.
    const long long want_warps = 2LL * sms * GF_WARPS;
    int ks = 1;
    while (ks < GF_WARPS && (long long)N * ks * 2 <= want_warps && (K / 8) / (ks * 2) >= 32) ks *= 2;
    const int rpr = GF_WARPS / ks;                            // rows a CTA works on at a time
    long long rounds = ((long long)N * ks + want_warps - 1) / want_warps;
    if (rounds < 1) rounds = 1;
    const int rows_per_cta = (int)(rounds * rpr);
    const unsigned grid = (unsigned)(((long long)N + rows_per_cta - 1) / rows_per_cta);
    const size_t part_off = (gf_smem(T, K, x == nullptr) + 15) / 16 * 16;
    const size_t smem = part_off + (size_t)rows_per_cta * ks * 2 * T * sizeof(float);
    agv_launch(kern, dim3(grid), dim3(GF_THREADS), smem, stream, (const __nv_bfloat16*)w,
               (const __nv_bfloat16*)w2, N, K, (const __nv_bfloat16*)x, ldx, j, out, ldo, act,
               rows_per_cta, ks, (int)part_off);
    AGV_LAUNCH_OK("gemv_few_kernel");
    return 0;
}

}  // namespace

// Whether agv_gemv_few takes these sizes: one to four tokens, K a multiple of 8, and the
// token rows (with the join: two 32-bit copies of them and both norm weights) within the
// shared memory of a CTA.
AGV_API int agv_gemv_few_supported(int T, int N, int K, long long ldx, int join) {
    if (T < 1 || T > 4 || N < 1 || K < 8 || K % 8 != 0) return 0;
    if (!join && ldx % 8 != 0) return 0;
    return gf_smem(T, K, join != 0) + 16 * 1024 <= (size_t)GF_MAX_SMEM ? 1 : 0;
}

// out[T, N] = x w^T in 32-bit, or with w2 the gated pair act(x w^T) * (x w2^T) in
// bfloat16 (act 0: tanh GELU, 1: SiLU); w, w2: [N, K] bfloat16 dense; out rows of stride
// ldo.  x: [T, K] bfloat16 with row stride ldx, or null: then x is formed by the join
// (see FewJoin above) from h_in [T, K] (32-bit, dense), y [T, K] or null, w_post [K] or
// null, w_next [K]; h_out [T, K] (not h_in) receives the joined stream unless null.
AGV_API int agv_gemv_few(const void* w, const void* w2, int N, int K, int T, const void* x,
                         long long ldx, const float* h_in, float* h_out, const float* y,
                         const float* w_post, const float* w_next, float eps_post, float eps_next,
                         void* out, long long ldo, int act, cudaStream_t stream) {
    AGV_REQUIRE(agv_gemv_few_supported(T, N, K, x ? ldx : 8, x ? 0 : 1),
                "gemv_few: T=%d N=%d K=%d is not a size this kernel takes", T, N, K);
    AGV_REQUIRE(w && out && ldo >= N && agv_aligned(w, 16) && (!w2 || agv_aligned(w2, 16)),
                "gemv_few: bad operands");
    FewJoin j{h_in, h_out, y, w_post, w_next, w_post ? eps_post : 0.f, eps_next};
    if (x) {
        AGV_REQUIRE(agv_aligned(x, 16) && ldx >= K, "gemv_few: x must be 16-byte aligned");
    } else {
        AGV_REQUIRE(h_in && w_next && h_out != h_in, "gemv_few: the join needs h_in and w_next, and "
                    "h_out must be another buffer");
        AGV_REQUIRE(!y || h_out, "gemv_few: a branch is added but the stream is not written back");
        AGV_REQUIRE(agv_aligned(h_in, 16) && agv_aligned(y, 16) && agv_aligned(w_post, 16) &&
                    agv_aligned(w_next, 16), "gemv_few: join operands must be 16-byte aligned");
    }
#define AGV_GF_CASE(TT)                                                                         \
    case TT:                                                                                     \
        return w2 ? gf_launch<TT, 1>(w, w2, N, K, x, ldx, j, out, ldo, act, stream)              \
                  : gf_launch<TT, 0>(w, nullptr, N, K, x, ldx, j, out, ldo, act, stream)
    switch (T) {
        AGV_GF_CASE(1);
        AGV_GF_CASE(2);
        AGV_GF_CASE(3);
        AGV_GF_CASE(4);
    }
#undef AGV_GF_CASE
    return agv_fail(-1, "gemv_few: T=%d", T);
}
