// Matrix products on the ordinary arithmetic units: out[M, N] = x[M, K] * w[N, K]^T,
// and the gated pair act(x wg^T) * (x wu^T).  This is the whole 32-bit path
// (plain FFMA, no reduced-precision mode) and the fallback of the bfloat16 path
// for shapes the tensor-core kernel refuses.
//
// Each output element is one dot product accumulated over k in ascending order
// in 32-bit, whatever M and N are, so a row's result does not depend on which
// other rows share the launch.
//
// Reference: one dot product per output row, f32 accumulation
// (src/backend/kernels/cuda/gemv_bf16.zig:6-24, gemv_f32.zig:6-21); gated
// activation src/backend/kernels/cuda/gelu_mul.zig:12-19 (here with tanhf).
#include "common.cuh"

enum AgvActivation { AGV_ACT_GELU_TANH = 0, AGV_ACT_SILU = 1 };

__device__ __forceinline__ float gelu_tanh_f(float t) {
    const float u = 0.7978845608028654f * (t + 0.044715f * t * t * t);
    return 0.5f * t * (1.0f + tanhf(u));
}
__device__ __forceinline__ float silu_f(float t) { return t / (1.0f + expf(-t)); }
__device__ __forceinline__ float activate(float t, int act) {
    return act == AGV_ACT_SILU ? silu_f(t) : gelu_tanh_f(t);
}

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
gemm_tn_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const TW* __restrict__ W2,
               TO* __restrict__ C, int M, int N, int K, long long lda, long long ldc, int act) {
    pdl_wait();
    pdl_launch_next();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float Us[GATED ? BK : 1][GATED ? BN + 4 : 1];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    float acc2[GATED ? 4 : 1][GATED ? 4 : 1] = {};
    const int lr = tid / 4, lk = (tid % 4) * 4;   // 64 rows x 16 k per tile, 4 k per thread
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int m = m0 + lr, n = n0 + lr;
            As[lk + i][lr] = (m < M && k < K) ? to_f32(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk + i][lr] = (n < N && k < K) ? to_f32(W[(size_t)n * K + k]) : 0.f;
            if (GATED) Us[lk + i][lr] = (n < N && k < K) ? to_f32(W2[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            if (GATED) {
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Us[k][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc2[i][j] = fmaf(a[i], b[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (GATED) v = activate(v, act) * acc2[i][j];
            C[(size_t)m * ldc + n] = from_f32<TO>(v);
        }
    }
}

template <typename TA, typename TW, typename TO>
static int launch_gemm(const void* A, const void* W, const void* W2, void* C, int M, int N, int K,
                       long long lda, long long ldc, int act, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (W2)
        agv_launch(gemm_tn_kernel<TA, TW, TO, true>, grid, 256, 0, stream, (const TA*)A, (const TW*)W, (const TW*)W2, (TO*)C, M, N, K, lda, ldc, act);
    else
        agv_launch(gemm_tn_kernel<TA, TW, TO, false>, grid, 256, 0, stream, (const TA*)A, (const TW*)W, nullptr, (TO*)C, M, N, K, lda, ldc, act);
    AGV_LAUNCH_OK("gemm_tn_kernel");
    return 0;
}

// x: [M, K] with row stride lda; w (and w2 for the gated form): [N, K] dense;
// out: [M, N] with row stride ldc.  in_dtype is the dtype of x and of the
// weights; out_dtype may be 32-bit for a bfloat16 product (logits).
AGV_API int agv_linear_simt(const void* x, const void* w, const void* w2, void* out, int M, int N,
                            int K, long long lda, long long ldc, int in_dtype, int out_dtype,
                            int act, cudaStream_t stream) {
    AGV_REQUIRE(M >= 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    AGV_REQUIRE(lda >= K && ldc >= N, "linear: row strides %lld, %lld shorter than rows", lda, ldc);
    AGV_REQUIRE((long long)((M + BM - 1) / BM) <= 65535, "linear: M=%d exceeds the grid limit", M);
    if (M == 0) return 0;
    if (in_dtype == AGV_F32 && out_dtype == AGV_F32)
        return launch_gemm<float, float, float>(x, w, w2, out, M, N, K, lda, ldc, act, stream);
    if (in_dtype == AGV_BF16 && out_dtype == AGV_BF16)
        return launch_gemm<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(x, w, w2, out, M, N, K, lda,
                                                                        ldc, act, stream);
    if (in_dtype == AGV_BF16 && out_dtype == AGV_F32)
        return launch_gemm<__nv_bfloat16, __nv_bfloat16, float>(x, w, w2, out, M, N, K, lda, ldc,
                                                                act, stream);
    return agv_fail(-1, "linear: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
}
