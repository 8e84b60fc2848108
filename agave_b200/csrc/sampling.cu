// Choosing the next token on the device: arg max, and temperature / top-k /
// top-p sampling; plus the repeat penalty.  One block per sequence over the
// whole vocabulary; logits are 32-bit.
//
// Reference (src/ops/math.zig): arg max takes the first index on ties (32-50);
// sampling divides by the temperature, keeps values >= the k-th greatest,
// forms exp(x - max), keeps weights >= the weight at which the descending
// running sum first reaches top_p * total, and draws by a linear scan of the
// running sum in index order, falling back to the last index (209-371); the
// repeat penalty divides positive logits and multiplies the others, once per
// occurrence (186-197).
//
// Sums that decide something (the top-p cut and the draw) are kept in 64-bit
// fixed point, so the same seed gives the same token whatever the order in
// which threads add.  The uniform number comes from a hash of (seed, sequence
// id, step): a sequence's draws do not depend on its batch.
#include "common.cuh"

constexpr int SM_THREADS = 1024;
// Sampling options as words on the device, so that one recorded decode step serves
// every setting: [1 / temperature (float bits), top_k, top_p (float bits), seed low,
// seed high, repeat penalty (float bits)]; two spare words.
enum { SP_INV_TEMPERATURE = 0, SP_TOP_K, SP_TOP_P, SP_SEED_LO, SP_SEED_HI, SP_PENALTY, SP_WORDS = 8 };
constexpr double FIX_ONE = 1099511627776.0;    // 2^40

// ----------------------------------------------------------------- arg max
// Two stages so that a few rows still fill the GPU: AM_PARTS CTAs per row each
// find (greatest value, first index) over a slice, the CTA that finishes last for
// a row reduces the slices.  Ties go to the lowest index in both stages.
constexpr int AM_PARTS = 64;
constexpr int AM_THREADS = 256;
constexpr int AM_MAX_ROWS = 4096;
__device__ float g_am_val[AM_MAX_ROWS * AM_PARTS];
__device__ int g_am_idx[AM_MAX_ROWS * AM_PARTS];
__device__ int g_am_count[AM_MAX_ROWS];       // zero between launches

__device__ __forceinline__ void am_better(float& best, int& idx, float ov, int oi) {
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
}

__global__ void __launch_bounds__(AM_THREADS)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int V, int* __restrict__ out,
              int row0) {
    pdl_wait();
    pdl_launch_next();
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ int s_last;
    const int row = blockIdx.y, part = blockIdx.x;
    const float* src = logits + (size_t)(row0 + row) * row_stride;
    const int per = (V + AM_PARTS - 1) / AM_PARTS;
    const int lo = part * per, hi = min(V, lo + per);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += AM_THREADS) am_better(best, idx, src[i], i);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        am_better(best, idx, __shfl_xor_sync(0xffffffffu, best, o),
                  __shfl_xor_sync(0xffffffffu, idx, o));
    if (lane == 0) { sv[warp] = best; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < AM_THREADS / 32 ? sv[lane] : -INFINITY;
        idx = lane < AM_THREADS / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            am_better(best, idx, __shfl_xor_sync(0xffffffffu, best, o),
                      __shfl_xor_sync(0xffffffffu, idx, o));
        if (lane == 0) {
            g_am_val[row * AM_PARTS + part] = best;
            g_am_idx[row * AM_PARTS + part] = idx;
            __threadfence();
            s_last = atomicAdd(&g_am_count[row], 1) == AM_PARTS - 1;
        }
    }
    __syncthreads();
    if (!s_last || warp != 0) return;
    __threadfence();
    best = -INFINITY;
    idx = 0x7fffffff;
    for (int i = lane; i < AM_PARTS; i += 32)
        am_better(best, idx, __ldcg(&g_am_val[row * AM_PARTS + i]),
                  __ldcg(&g_am_idx[row * AM_PARTS + i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        am_better(best, idx, __shfl_xor_sync(0xffffffffu, best, o),
                  __shfl_xor_sync(0xffffffffu, idx, o));
    if (lane == 0) {
        out[row0 + row] = idx == 0x7fffffff ? 0 : idx;
        g_am_count[row] = 0;
    }
}

// out[b] = first index of the greatest logits[b, :].  Calls on different streams
// must not overlap: the stages share one table of partial results.
AGV_API int agv_argmax(const float* logits, long long row_stride, int B, int V, int* out,
                       cudaStream_t stream) {
    AGV_REQUIRE(B >= 0 && V > 0 && row_stride >= V, "argmax: bad sizes B=%d V=%d", B, V);
    for (int row0 = 0; row0 < B; row0 += AM_MAX_ROWS) {
        const int rows = B - row0 < AM_MAX_ROWS ? B - row0 : AM_MAX_ROWS;
        agv_launch(argmax_kernel, dim3(AM_PARTS, rows), AM_THREADS, 0, stream, logits, row_stride, V, out,
                                                                      row0);
        AGV_LAUNCH_OK("argmax_kernel");
    }
    return 0;
}

// ------------------------------------------------------------ repeat penalty
// Generated ids are kept per cache slot on the device: hist [n_slots, cap] and
// hist_len [n_slots].  A decode step appends its input token (the token chosen
// in the step before), so at any step the history is "everything generated so
// far", which is what the reference penalises (src/main.zig:2350-2352).
__global__ void history_append_kernel(const int* __restrict__ tokens, const int* __restrict__ slots,
                                      int* __restrict__ hist, int* __restrict__ hist_len, int cap,
                                      int B) {
    pdl_wait();
    pdl_launch_next();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int slot = slots[b];
    if (slot < 0) return;
    const int n = hist_len[slot];
    if (n < cap) {
        hist[(size_t)slot * cap + n] = tokens[b];
        hist_len[slot] = n + 1;
    }
}

AGV_API int agv_history_append(const int* tokens, const int* slots, int* hist, int* hist_len,
                               int cap, int B, cudaStream_t stream) {
    AGV_REQUIRE(cap > 0 && B >= 0, "history_append: bad sizes");
    if (B == 0) return 0;
    agv_launch(history_append_kernel, (B + 127) / 128, 128, 0, stream, tokens, slots, hist, hist_len, cap, B);
    AGV_LAUNCH_OK("history_append_kernel");
    return 0;
}

// A decode step launched before the host has read the step before it takes its
// input tokens from that step's choices on the device: tokens[b] = prev[b] when
// *take is set (ids outside the vocabulary, possible only in padding rows, become 0).
__global__ void take_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ prev,
                                   const int* __restrict__ take, int B, int V) {
    pdl_wait();
    pdl_launch_next();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B || !*take) return;
    const int t = prev[b];
    tokens[b] = (t >= 0 && t < V) ? t : 0;
}

AGV_API int agv_take_tokens(int* tokens, const int* prev, const int* take, int B, int V,
                            cudaStream_t stream) {
    AGV_REQUIRE(B >= 0 && V > 0, "take_tokens: bad sizes");
    if (B == 0) return 0;
    agv_launch(take_tokens_kernel, (B + 127) / 128, 128, 0, stream, tokens, prev, take, B, V);
    AGV_LAUNCH_OK("take_tokens_kernel");
    return 0;
}

// The thread of an id's first occurrence applies the penalty once per
// occurrence, so no two threads touch one logit.
__global__ void repeat_penalty_kernel(float* __restrict__ logits, long long row_stride, int V,
                                      const int* __restrict__ slots, const int* __restrict__ hist,
                                      const int* __restrict__ hist_len, int cap, float penalty,
                                      const int* __restrict__ dev_params) {
    pdl_wait();
    pdl_launch_next();
    if (dev_params) penalty = __int_as_float(dev_params[SP_PENALTY]);
    if (penalty == 1.0f) return;
    const int b = blockIdx.y;
    const int slot = slots[b];
    if (slot < 0) return;
    const int n = min(hist_len[slot], cap);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int* hrow = hist + (size_t)slot * cap;
    const int id = hrow[i];
    if (id < 0 || id >= V) return;
    int count = 0;
    for (int j = 0; j < n; ++j) {
        if (hrow[j] == id) {
            if (j < i) return;
            ++count;
        }
    }
    float* p = logits + (size_t)b * row_stride + id;
    float v = *p;
    for (int c = 0; c < count; ++c) v = v > 0.f ? v / penalty : v * penalty;
    *p = v;
}

// logits [B, V] in place; slots [B]; hist [n_slots, cap]; hist_len [n_slots].
// dev_params (or null): the sampling words on the device (see agv_sample); the penalty
// is then read from them when the kernel runs, not from the argument.
AGV_API int agv_repeat_penalty(float* logits, long long row_stride, int B, int V, const int* slots,
                               const int* hist, const int* hist_len, int cap, float penalty,
                               const int* dev_params, cudaStream_t stream) {
    AGV_REQUIRE(dev_params || penalty > 0.f, "repeat_penalty: penalty must be positive");
    AGV_REQUIRE(cap > 0, "repeat_penalty: bad history capacity");
    if (B == 0) return 0;
    dim3 grid((cap + 255) / 256, B);
    agv_launch(repeat_penalty_kernel, grid, 256, 0, stream, logits, row_stride, V, slots, hist, hist_len,
                                                    cap, penalty, dev_params);
    AGV_LAUNCH_OK("repeat_penalty_kernel");
    return 0;
}

// ------------------------------------------------------------------ sampling
__device__ __forceinline__ unsigned ordered_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__device__ __forceinline__ unsigned long long to_fixed(float w) {
    return (unsigned long long)((double)w * FIX_ONE);
}

struct SampleShared {
    unsigned long long hist[256];
    unsigned long long chunk[SM_THREADS];
    float red[33];
    unsigned prefix;
    unsigned long long above;
    int done;
    int result;
};

// Descends the 32-bit key space 8 bits at a time.  COUNT: finds the key of the
// k-th greatest element (target = k, each element weighs 1).  Otherwise finds
// the greatest key whose tail mass reaches target (each element weighs its
// fixed-point weight).
template <bool COUNT, typename KeyFn, typename MassFn>
__device__ unsigned radix_descend(SampleShared& sh, int V, unsigned long long target, KeyFn key,
                                  MassFn mass) {
    if (threadIdx.x == 0) { sh.prefix = 0; sh.above = 0; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.hist[i] = 0;
        __syncthreads();
        const unsigned prefix = sh.prefix;
        const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const unsigned kk = key(i);
            if ((kk & himask) == prefix) {
                const unsigned long long m = COUNT ? 1ull : mass(i);
                if (m) atomicAdd(&sh.hist[(kk >> shift) & 255u], m);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long acc = sh.above;
            int bin = 255;
            for (; bin > 0; --bin) {
                if (acc + sh.hist[bin] >= target) break;
                acc += sh.hist[bin];
            }
            sh.above = acc;
            sh.prefix = prefix | ((unsigned)bin << shift);
        }
        __syncthreads();
    }
    return sh.prefix;
}

__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
              int* __restrict__ out, float inv_temperature, int top_k, float top_p,
              unsigned long long seed, const long long* __restrict__ seq_ids,
              const int* __restrict__ steps, const int* __restrict__ dev_params) {
    pdl_wait();
    pdl_launch_next();
    if (dev_params) {
        inv_temperature = __int_as_float(dev_params[SP_INV_TEMPERATURE]);
        top_k = dev_params[SP_TOP_K];
        top_p = __int_as_float(dev_params[SP_TOP_P]);
        seed = (unsigned long long)(unsigned)dev_params[SP_SEED_LO] |
               ((unsigned long long)(unsigned)dev_params[SP_SEED_HI] << 32);
    }
    __shared__ SampleShared sh;
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    auto xval = [&](int i) { return row[i] * inv_temperature; };

    // 1. top-k threshold on the scaled logits
    unsigned kth_key = 0;
    if (top_k > 0 && top_k < V)
        kth_key = radix_descend<true>(sh, V, (unsigned long long)top_k,
                                      [&](int i) { return ordered_key(xval(i)); },
                                      [&](int) { return 1ull; });
    // 2. maximum (always kept)
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, xval(i));
    mx = block_max(mx, sh.red);
    auto weight = [&](int i) -> float {
        const float x = xval(i);
        if (ordered_key(x) < kth_key) return 0.f;
        return expf(x - mx);
    };
    // 3. top-p threshold on the weights (all >= 0, so their bits order them)
    unsigned cut_bits = 0;
    if (top_p > 0.f && top_p < 1.f) {
        unsigned long long part = 0;
        for (int i = threadIdx.x; i < V; i += blockDim.x) part += to_fixed(weight(i));
        if (threadIdx.x == 0) sh.above = 0;
        __syncthreads();
        atomicAdd(&sh.above, part);
        __syncthreads();
        const unsigned long long total = sh.above;
        __syncthreads();
        const unsigned long long target = (unsigned long long)((double)top_p * (double)total);
        cut_bits = radix_descend<false>(sh, V, target > 0 ? target : 1ull,
                                        [&](int i) { return __float_as_uint(weight(i)); },
                                        [&](int i) { return to_fixed(weight(i)); });
    }
    auto kept = [&](int i) -> unsigned long long {
        const float w = weight(i);
        return __float_as_uint(w) >= cut_bits ? to_fixed(w) : 0ull;
    };
    // 4. draw in index order: contiguous chunk per thread, scan of chunk sums
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int lo = min(V, (int)threadIdx.x * per), hi = min(V, lo + per);
    unsigned long long mine = 0;
    for (int i = lo; i < hi; ++i) mine += kept(i);
    sh.chunk[threadIdx.x] = mine;
    if (threadIdx.x == 0) { sh.done = 0; sh.result = V - 1; }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long run = 0;
        for (int i = 0; i < (int)blockDim.x; ++i) {
            const unsigned long long c = sh.chunk[i];
            sh.chunk[i] = run;
            run += c;
        }
        sh.above = run;
    }
    __syncthreads();
    const unsigned long long total = sh.above;
    const unsigned long long h =
        splitmix64(splitmix64(seed ^ 0xA5A5A5A5DEADBEEFull) ^
                   splitmix64((unsigned long long)seq_ids[blockIdx.x] * 0x100000001B3ull +
                              (unsigned long long)(unsigned)steps[blockIdx.x]));
    const double u = (double)(h >> 11) * (1.0 / 9007199254740992.0);     // [0, 1)
    const unsigned long long thr = (unsigned long long)(u * (double)total);
    const unsigned long long before = sh.chunk[threadIdx.x];
    if (mine > 0 && before <= thr && thr < before + mine) {
        unsigned long long run = before;
        for (int i = lo; i < hi; ++i) {
            run += kept(i);
            if (thr < run) { sh.result = i; break; }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) out[blockIdx.x] = sh.result;
}

// One token per row of logits [B, V].  temperature > 0; top_k 0 = off; top_p
// outside (0, 1) = off.  seq_ids[b] and steps[b] key the draw of row b.
// dev_params (or null): SP_WORDS ints on the device that replace temperature, top_k,
// top_p and seed when the kernel runs (a recorded launch then serves every setting).
AGV_API int agv_sample(const float* logits, long long row_stride, int B, int V, int* out,
                       float temperature, int top_k, float top_p, unsigned long long seed,
                       const long long* seq_ids, const int* steps, const int* dev_params,
                       cudaStream_t stream) {
    AGV_REQUIRE(B >= 0 && V > 0 && row_stride >= V, "sample: bad sizes B=%d V=%d", B, V);
    AGV_REQUIRE(dev_params || temperature > 0.f,
                "sample: temperature must be positive (0 is arg max)");
    AGV_REQUIRE(top_k >= 0, "sample: top_k must be >= 0");
    if (B == 0) return 0;
    agv_launch(sample_kernel, B, SM_THREADS, 0, stream, logits, row_stride, V, out,
               dev_params ? 1.0f : 1.0f / temperature, top_k, top_p, seed, seq_ids, steps,
               dev_params);
    AGV_LAUNCH_OK("sample_kernel");
    return 0;
}
