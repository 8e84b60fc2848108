// Embedding lookup, rotation tables and row-wise RMS norms (with the residual
// sum folded in).  One templated kernel per operation serves the bfloat16 and
// the 32-bit path; statistics, the residual stream and the rotation angles are
// 32-bit (angles are formed in 64-bit and rounded once).
//
// Reference formulas: embedding * sqrt(H) src/models/gemma3.zig:1017-1046;
// RMS norm with eps inside the root src/backend/kernels/cuda/rms_norm.zig:22-29;
// rotation angle src/backend/kernels/cuda/rope.zig:9-37 (here without the
// approximate sin/cos).
#include "common.cuh"
#include <type_traits>

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ out, int H, int V, float scale) {
    pdl_wait();
    pdl_launch_next();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= V) tok = 0;   // callers validate ids; never read outside the table
    const TW* row = table + (size_t)tok * H;
    float* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]) * scale;
}

AGV_API int agv_embed(const int* tokens, const void* table, int table_dtype, float* out, int T,
                      int H, int V, float scale, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && H > 0 && V > 0, "embed: bad sizes T=%d H=%d V=%d", T, H, V);
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == AGV_F32)
        agv_launch(embed_kernel<float>, T, threads, 0, stream, tokens, (const float*)table, out, H, V, scale);
    else if (table_dtype == AGV_BF16)
        agv_launch(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, tokens, (const __nv_bfloat16*)table,
                                                               out, H, V, scale);
    else
        return agv_fail(-1, "embed: unknown dtype %d", table_dtype);
    AGV_LAUNCH_OK("embed_kernel");
    return 0;
}

// ------------------------------------------------------------ rotation tables
__global__ void rope_table_kernel(const int* __restrict__ positions, float* __restrict__ cosv,
                                  float* __restrict__ sinv, int T, int half, double log_theta,
                                  double inv_factor, int rotary_dim) {
    pdl_wait();
    pdl_launch_next();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx % half;
    const double freq = exp(-log_theta * (2.0 * i) / (double)rotary_dim);
    const double a = (double)positions[t] * inv_factor * freq;
    double s, c;
    sincos(a, &s, &c);
    cosv[idx] = (float)c;
    sinv[idx] = (float)s;
}

// cos, sin: [T, rotary_dim/2] for angle = (p / factor) * theta^(-2i/rotary_dim).
AGV_API int agv_rope_table(const int* positions, float* cosv, float* sinv, int T, int rotary_dim,
                           double theta, double factor, cudaStream_t stream) {
    AGV_REQUIRE(rotary_dim > 0 && rotary_dim % 2 == 0, "rope_table: rotary_dim %d must be even",
                rotary_dim);
    AGV_REQUIRE(theta > 0 && factor > 0, "rope_table: theta and factor must be positive");
    if (T == 0) return 0;
    const int half = rotary_dim / 2, n = T * half;
    agv_launch(rope_table_kernel, (n + 127) / 128, 128, 0, stream, positions, cosv, sinv, T, half,
                                                           log(theta), 1.0 / factor, rotary_dim);
    AGV_LAUNCH_OK("rope_table_kernel");
    return 0;
}

// ----------------------------------------------------------------- RMS norms
// One block per row.  With y == nullptr: x = norm(h[rows[r]]; w_next).
// Otherwise: b = sum over splits of y; if w_post: b = norm(b; w_post);
// h += b; if w_next: x = norm(h; w_next).
template <typename TY, typename TX>
__global__ void norm_residual_kernel(float* __restrict__ h, const TY* __restrict__ y, int n_splits,
                                     size_t split_stride, const float* __restrict__ w_post,
                                     const float* __restrict__ w_next, TX* __restrict__ x,
                                     const int* __restrict__ rows, int H, float eps_post,
                                     float eps_next, int add_residual) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float row[];
    __shared__ float red[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    const size_t dst = (size_t)r * H;
    if (y) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = 0.f;
            for (int s = 0; s < n_splits; ++s) v += to_f32(y[s * split_stride + src + i]);
            row[i] = v;
            ss += v * v;
        }
        float rs = 1.f;
        if (w_post) {
            ss = block_sum(ss, red);
            rs = 1.0f / sqrtf(ss / (float)H + eps_post);
        }
        float ss2 = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = row[i];
            if (w_post) v = v * rs * w_post[i];
            if (add_residual) {
                v += h[src + i];
                h[src + i] = v;
            }
            row[i] = v;
            ss2 += v * v;
        }
        if (w_next) {
            ss2 = block_sum(ss2, red);
            const float r2 = 1.0f / sqrtf(ss2 / (float)H + eps_next);
            for (int i = threadIdx.x; i < H; i += blockDim.x)
                x[dst + i] = from_f32<TX>(row[i] * r2 * w_next[i]);
        } else if (x) {
            for (int i = threadIdx.x; i < H; i += blockDim.x) x[dst + i] = from_f32<TX>(row[i]);
        }
    } else {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = h[src + i];
            row[i] = v;
            ss += v * v;
        }
        ss = block_sum(ss, red);
        const float r2 = 1.0f / sqrtf(ss / (float)H + eps_next);
        for (int i = threadIdx.x; i < H; i += blockDim.x)
            x[dst + i] = from_f32<TX>(row[i] * r2 * w_next[i]);
    }
}

// The same arithmetic for rows of at most EPT * blockDim.x values, with every
// operand a thread needs (branch partial sums, stream, both weights) loaded up
// front into registers: the loads of one row overlap instead of queueing behind
// the reductions.  This is the variant decode steps run.
template <typename TY, typename TX, int EPT, int MAXT>
__global__ void __launch_bounds__(MAXT)
norm_residual_small_kernel(float* __restrict__ h, const TY* __restrict__ y, int n_splits,
                           size_t split_stride, const float* __restrict__ w_post,
                           const float* __restrict__ w_next, TX* __restrict__ x,
                           const int* __restrict__ rows, int H, float eps_post, float eps_next,
                           int add_residual) {
    // (the arguments are read before the wait: their first read from the parameter bank
    // is a slow one, and here nothing else hides it)
    asm volatile("" ::"l"(h), "l"(y), "l"(w_post), "l"(w_next), "l"(x), "l"(rows), "r"(H),
                 "r"(n_splits), "l"(split_stride), "f"(eps_post), "f"(eps_next), "r"(add_residual));
    pdl_wait();
    pdl_launch_next();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    const size_t dst = (size_t)r * H;
    float v[EPT], hv[EPT], wp[EPT], wn[EPT];
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        const bool in = i < H;
        v[k] = 0.f;
        hv[k] = (in && (add_residual || !y)) ? h[src + i] : 0.f;
        wp[k] = (in && w_post) ? w_post[i] : 1.f;
        wn[k] = (in && w_next) ? w_next[i] : 1.f;
    }
    if (y) {
        constexpr int U = EPT <= 2 ? 16 : (EPT <= 4 ? 8 : (EPT <= 8 ? 4 : (EPT <= 16 ? 2 : 1)));
        if (n_splits == 1) {
#pragma unroll
            for (int k = 0; k < EPT; ++k) {
                const int i = threadIdx.x + k * blockDim.x;
                v[k] = i < H ? to_f32(y[src + i]) : 0.f;
            }
        } else
        for (int s0 = 0; s0 < n_splits; s0 += U) {
            float t[U][EPT];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int k = 0; k < EPT; ++k) {
                    const int i = min(threadIdx.x + k * blockDim.x, (unsigned)(H - 1));
                    const int sp = min(s0 + u, n_splits - 1);
                    t[u][k] = to_f32(y[(size_t)sp * split_stride + src + i]);
                }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int k = 0; k < EPT; ++k) {
                    const int i = threadIdx.x + k * blockDim.x;
                    v[k] += (i < H && s0 + u < n_splits) ? t[u][k] : 0.f;
                }
        }
        if (w_post) {
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < EPT; ++k) ss += v[k] * v[k];
            ss = block_sum(ss, red);
            const float rs = 1.0f / sqrtf(ss / (float)H + eps_post);
#pragma unroll
            for (int k = 0; k < EPT; ++k) v[k] = v[k] * rs * wp[k];
        }
        if (add_residual) {
#pragma unroll
            for (int k = 0; k < EPT; ++k) {
                const int i = threadIdx.x + k * blockDim.x;
                v[k] += hv[k];
                if (i < H) h[src + i] = v[k];
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < EPT; ++k) v[k] = hv[k];
    }
    if (w_next) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < EPT; ++k) ss += v[k] * v[k];      // lanes beyond H hold 0
        ss = block_sum(ss, red);
        const float r2 = 1.0f / sqrtf(ss / (float)H + eps_next);
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < H) x[dst + i] = from_f32<TX>(v[k] * r2 * wn[k]);
        }
    } else if (x) {
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < H) x[dst + i] = from_f32<TX>(v[k]);
        }
    }
}

// Many rows (prompts), 32-bit branch input, width a multiple of 4 up to 2,048: one
// warp per row with 16-byte loads and no block-wide barrier.
template <typename TX> struct Pack4;
template <> struct Pack4<float> {
    __device__ static void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Pack4<__nv_bfloat16> {
    __device__ static void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<unsigned*>(&a);
        u.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <typename TX, int NV>
__global__ void __launch_bounds__(128)
norm_residual_warp_kernel(float* __restrict__ h, const float* __restrict__ y, int n_splits,
                          size_t split_stride, const float* __restrict__ w_post,
                          const float* __restrict__ w_next, TX* __restrict__ x, int R, int H,
                          float eps_post, float eps_next, int add_residual) {
    pdl_wait();
    pdl_launch_next();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= R) return;
    const int H4 = H >> 2;
    const size_t base = (size_t)row * H;
    float4 v[NV], hv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int idx = lane + 32 * i;
        const bool in = idx < H4;
        v[i] = in ? reinterpret_cast<const float4*>(y + base)[idx] : make_float4(0, 0, 0, 0);
        hv[i] = (in && add_residual) ? reinterpret_cast<const float4*>(h + base)[idx]
                                     : make_float4(0, 0, 0, 0);
    }
    for (int s = 1; s < n_splits; ++s) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < H4) {
                const float4 t = reinterpret_cast<const float4*>(y + s * split_stride + base)[idx];
                v[i].x += t.x; v[i].y += t.y; v[i].z += t.z; v[i].w += t.w;
            }
        }
    }
    float rs = 1.f;
    if (w_post) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        ss = warp_sum(ss);
        rs = 1.0f / sqrtf(ss / (float)H + eps_post);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int idx = lane + 32 * i;
        if (idx < H4) {
            if (w_post) {
                const float4 w = reinterpret_cast<const float4*>(w_post)[idx];
                v[i].x = v[i].x * rs * w.x; v[i].y = v[i].y * rs * w.y;
                v[i].z = v[i].z * rs * w.z; v[i].w = v[i].w * rs * w.w;
            }
            if (add_residual) {
                v[i].x += hv[i].x; v[i].y += hv[i].y; v[i].z += hv[i].z; v[i].w += hv[i].w;
                reinterpret_cast<float4*>(h + base)[idx] = v[i];
            }
            ss2 += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    if (w_next) {
        ss2 = warp_sum(ss2);
        const float r2 = 1.0f / sqrtf(ss2 / (float)H + eps_next);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < H4) {
                const float4 w = reinterpret_cast<const float4*>(w_next)[idx];
                Pack4<TX>::store(x + base + 4 * idx,
                                 make_float4(v[i].x * r2 * w.x, v[i].y * r2 * w.y,
                                             v[i].z * r2 * w.z, v[i].w * r2 * w.w));
            }
        }
    } else if (x) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < H4) Pack4<TX>::store(x + base + 4 * idx, v[i]);
        }
    }
}

// The same with one CTA of 256 threads per row, 16-byte loads issued up front, two
// block-wide sums: for rows too wide for a warp's registers (above 2,048 values), and for
// 32 to 256 rows of any width (decoding many sequences: too few rows for a warp each).
template <typename TX, int NV>
__global__ void __launch_bounds__(256)
norm_residual_row_kernel(float* __restrict__ h, const float* __restrict__ y, int n_splits,
                          size_t split_stride, const float* __restrict__ w_post,
                          const float* __restrict__ w_next, TX* __restrict__ x, int R, int H,
                          float eps_post, float eps_next, int add_residual) {
    pdl_wait();
    pdl_launch_next();
    __shared__ float red[33];
    const int lane = threadIdx.x;                   // 256 threads share the row
    const int row = blockIdx.x;
    const int H4 = H >> 2;
    const size_t base = (size_t)row * H;
    float4 v[NV], hv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int idx = lane + 256 * i;
        const bool in = idx < H4;
        v[i] = in ? reinterpret_cast<const float4*>(y + base)[idx] : make_float4(0, 0, 0, 0);
        hv[i] = (in && add_residual) ? reinterpret_cast<const float4*>(h + base)[idx]
                                     : make_float4(0, 0, 0, 0);
    }
    // the other partial sums, four at a time: their loads are issued together (a rolled
    // loop would make one trip to memory per partial sum)
    for (int s = 1; s < n_splits; s += 4) {
        float4 t[4][NV];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float* src = y + (size_t)min(s + u, n_splits - 1) * split_stride + base;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int idx = lane + 256 * i;
                t[u][i] = idx < H4 ? reinterpret_cast<const float4*>(src)[idx]
                                   : make_float4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (s + u < n_splits) {
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    v[i].x += t[u][i].x; v[i].y += t[u][i].y;
                    v[i].z += t[u][i].z; v[i].w += t[u][i].w;
                }
            }
        }
    }
    float rs = 1.f;
    if (w_post) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        ss = block_sum(ss, red);
        rs = 1.0f / sqrtf(ss / (float)H + eps_post);
    }
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int idx = lane + 256 * i;
        if (idx < H4) {
            if (w_post) {
                const float4 w = reinterpret_cast<const float4*>(w_post)[idx];
                v[i].x = v[i].x * rs * w.x; v[i].y = v[i].y * rs * w.y;
                v[i].z = v[i].z * rs * w.z; v[i].w = v[i].w * rs * w.w;
            }
            if (add_residual) {
                v[i].x += hv[i].x; v[i].y += hv[i].y; v[i].z += hv[i].z; v[i].w += hv[i].w;
                reinterpret_cast<float4*>(h + base)[idx] = v[i];
            }
            ss2 += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    if (w_next) {
        ss2 = block_sum(ss2, red);
        const float r2 = 1.0f / sqrtf(ss2 / (float)H + eps_next);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 256 * i;
            if (idx < H4) {
                const float4 w = reinterpret_cast<const float4*>(w_next)[idx];
                Pack4<TX>::store(x + base + 4 * idx,
                                 make_float4(v[i].x * r2 * w.x, v[i].y * r2 * w.y,
                                             v[i].z * r2 * w.z, v[i].w * r2 * w.w));
            }
        }
    } else if (x) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 256 * i;
            if (idx < H4) Pack4<TX>::store(x + base + 4 * idx, v[i]);
        }
    }
}

template <typename TX>
static bool launch_norm_warp(float* h, const float* y, int n_splits, size_t split_stride,
                             const float* w_post, const float* w_next, TX* x, int R, int H,
                             float eps_post, float eps_next, int add_residual,
                             cudaStream_t stream) {
    const int nv = (H / 4 + 31) / 32;
    const unsigned grid = (unsigned)((R + 3) / 4);
#define AGV_WARP(NV)                                                                            \
    agv_launch(norm_residual_warp_kernel<TX, NV>, grid, 128, 0, stream, h, y, n_splits,         \
               split_stride, w_post, w_next, x, R, H, eps_post, eps_next, add_residual)
    if (nv <= 2) AGV_WARP(2);
    else if (nv <= 4) AGV_WARP(4);
    else if (nv <= 6) AGV_WARP(6);
    else if (nv <= 8) AGV_WARP(8);
    else if (nv <= 10) AGV_WARP(10);
    else if (nv <= 12) AGV_WARP(12);
    else if (nv <= 16) AGV_WARP(16);
    else return false;
#undef AGV_WARP
    return true;
}

template <typename TX>
static bool launch_norm_row(float* h, const float* y, int n_splits, size_t split_stride,
                            const float* w_post, const float* w_next, TX* x, int R, int H,
                            float eps_post, float eps_next, int add_residual,
                            cudaStream_t stream) {
    const int nv = (H / 4 + 255) / 256;
#define AGV_ROW(NV)                                                                             \
    agv_launch(norm_residual_row_kernel<TX, NV>, (unsigned)R, 256, 0, stream, h, y, n_splits,   \
               split_stride, w_post, w_next, x, R, H, eps_post, eps_next, add_residual)
    if (nv <= 2) AGV_ROW(2);
    else if (nv <= 4) AGV_ROW(4);
    else if (nv <= 6) AGV_ROW(6);
    else if (nv <= 8) AGV_ROW(8);
    else return false;
#undef AGV_ROW
    return true;
}

template <typename TY, typename TX>
static int launch_norm(float* h, const void* y, int n_splits, size_t split_stride,
                       const float* w_post, const float* w_next, void* x, const int* rows, int R,
                       int H, float eps_post, float eps_next, int add_residual,
                       cudaStream_t stream) {
    // many rows with a 32-bit branch input: one warp per row
    if constexpr (std::is_same<TY, float>::value) {
        if (R > 256 && y && !rows && H % 4 == 0 && H <= 2048 && agv_aligned(y, 16) &&
            agv_aligned(h, 16) && agv_aligned(x, 16) && split_stride % 4 == 0 &&
            (!w_post || agv_aligned(w_post, 16)) && (!w_next || agv_aligned(w_next, 16)) &&
            (add_residual || !h || true)) {
            if (launch_norm_warp<TX>(h, (const float*)y, n_splits, split_stride, w_post, w_next,
                                     (TX*)x, R, H, eps_post, eps_next, add_residual, stream)) {
                AGV_LAUNCH_OK("norm_residual_warp_kernel");
                return 0;
            }
        }
        if (((R > 256 && H > 2048) || (R >= 32 && R <= 256)) && y && !rows && H % 4 == 0 && H <= 8192 && agv_aligned(y, 16) &&
            agv_aligned(h, 16) && agv_aligned(x, 16) && split_stride % 4 == 0 &&
            (!w_post || agv_aligned(w_post, 16)) && (!w_next || agv_aligned(w_next, 16))) {
            if (launch_norm_row<TX>(h, (const float*)y, n_splits, split_stride, w_post, w_next,
                                    (TX*)x, R, H, eps_post, eps_next, add_residual, stream)) {
                AGV_LAUNCH_OK("norm_residual_row_kernel");
                return 0;
            }
        }
    }
    // the register-resident kernel, one row per CTA: many threads per row when the
    // rows are few (decode, final norm), few threads per row when they are many
    if (H <= 8 * 1024) {
        const int threads = R <= 256 ? (H <= 256 ? 128 : H <= 1024 ? 512 : 1024)
                               : (H <= 512 ? 128 : 256);

        const int ept = (H + threads - 1) / threads;
#define AGV_SMALL(E, MT)                                                                        \
    agv_launch(norm_residual_small_kernel<TY, TX, E, MT>, R, threads, 0, stream, h,             \
               (const TY*)y, n_splits, split_stride, w_post, w_next, (TX*)x, rows, H, eps_post, \
               eps_next, add_residual)
        if (threads > 256) {
            if (ept <= 1) AGV_SMALL(1, 1024);
            else if (ept <= 2) AGV_SMALL(2, 1024);
            else if (ept <= 4) AGV_SMALL(4, 1024);
            else AGV_SMALL(8, 1024);
        } else {
            if (ept <= 1) AGV_SMALL(1, 256);
            else if (ept <= 2) AGV_SMALL(2, 256);
            else if (ept <= 4) AGV_SMALL(4, 256);
            else if (ept <= 8) AGV_SMALL(8, 256);
            else if (ept <= 16) AGV_SMALL(16, 256);
            else AGV_SMALL(32, 256);
        }
#undef AGV_SMALL
        AGV_LAUNCH_OK("norm_residual_small_kernel");
        return 0;
    }
    const size_t smem = (size_t)H * sizeof(float);
    auto kern = norm_residual_kernel<TY, TX>;
    if (smem > 48 * 1024) {
        AGV_REQUIRE(smem <= 200 * 1024, "norm: row width %d needs %zu bytes of shared memory, "
                    "more than the 200 KB this kernel may take", H, smem);
        AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    agv_launch(kern, R, threads, smem, stream, h, (const TY*)y, n_splits, split_stride, w_post, w_next,
                                       (TX*)x, rows, H, eps_post, eps_next, add_residual);
    AGV_LAUNCH_OK("norm_residual_kernel");
    return 0;
}

// h: [*, H] 32-bit residual stream.  y: [n_splits, R, H] branch output (y_dtype)
// or null.  x: [R, H] output (x_dtype) or null.  rows: optional gather of h rows
// (only with y == null).  See norm_residual_kernel for the arithmetic.
AGV_API int agv_norm_residual(float* h, const void* y, int y_dtype, int n_splits,
                              long long split_stride, const float* w_post, const float* w_next,
                              void* x, int x_dtype, const int* rows, int R, int H, float eps_post,
                              float eps_next, int add_residual, cudaStream_t stream) {
    AGV_REQUIRE(R >= 0 && H > 0, "norm: bad sizes R=%d H=%d", R, H);
    AGV_REQUIRE(y || (w_next && x && h), "norm: without a branch input, h, w_next and x are needed");
    AGV_REQUIRE(!y || n_splits >= 1, "norm: n_splits must be >= 1");
    AGV_REQUIRE(!(y && rows), "norm: row gather is only for the plain norm");
    AGV_REQUIRE(!add_residual || h, "norm: the residual sum needs h");
    AGV_REQUIRE(!w_next || x, "norm: w_next given without an output");
    if (R == 0) return 0;
#define AGV_NORM_CASE(TY, TX)                                                                   \
    return launch_norm<TY, TX>(h, y, n_splits, (size_t)split_stride, w_post, w_next, x, rows, R, \
                               H, eps_post, eps_next, add_residual, stream)
    const int yd = y ? y_dtype : AGV_F32;
    const int xd = x ? x_dtype : AGV_F32;
    if (yd == AGV_F32 && xd == AGV_F32) AGV_NORM_CASE(float, float);
    if (yd == AGV_F32 && xd == AGV_BF16) AGV_NORM_CASE(float, __nv_bfloat16);
    if (yd == AGV_BF16 && xd == AGV_BF16) AGV_NORM_CASE(__nv_bfloat16, __nv_bfloat16);
    if (yd == AGV_BF16 && xd == AGV_F32) AGV_NORM_CASE(__nv_bfloat16, float);
#undef AGV_NORM_CASE
    return agv_fail(-1, "norm: unknown dtypes y=%d x=%d", y_dtype, x_dtype);
}
