// Decode attention over the paged cache, split along the keys.
//
// One CTA takes one sequence, one group of query heads that share a kv head,
// and one chunk of CH consecutive key positions.  It copies the chunk's key and
// value rows into shared memory with cp.async (every row in flight at once, so
// the cost is one trip to HBM, not one per key), computes the scores of the
// group's heads, their softmax weights relative to the chunk's own maximum, and
// the weighted sum of the values; it writes that partial result (sum, maximum,
// normaliser) to scratch memory and counts itself in; the CTA that arrives last
// for a (sequence, head group) merges the chunks in chunk order and writes the
// output (a sequence with a single chunk is written directly).  Chunks past a
// sequence's end exit at once, so the grid can be sized for the longest
// sequence the cache allows and the launch replayed from a CUDA graph.  Scores,
// softmax and sums are 32-bit.  The arrival counters must be zero before a
// launch; every launch leaves them zero.  (The bfloat16 tensor-core form below
// shares a sequence's tiles among a number of CTAs that follows the batch size
// instead; see attention_decode_mma_kernel.)
//
// Reference: one block per head, scores of all positions in shared memory,
// softmax by the first 32 threads (src/backend/kernels/cuda/sdpa.zig:16-104);
// score = (q . k) * scale, kv head = h / (nh / nkv)
// (src/backend/kernels/cpu/sdpa.zig:36-37,58); window start sl - W
// (src/models/gemma4.zig:1153-1155).  No value row is skipped for a small weight.
#include "common.cuh"
#include "tcgen05.cuh"
#include <map>
#include <tuple>

namespace {

constexpr int AD_THREADS = 128;
constexpr int AD_GC = 4;              // query heads of a group handled together
constexpr int AD_MAX_HD = 512;
constexpr int AD_MAX_SMEM = 160 * 1024;

template <typename T> struct Vec16;   // 16-byte vector of T
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
// waits until at most one group of copies, the one committed last, is still in flight
__device__ __forceinline__ void cp_async_wait_but_one() {
    asm volatile("cp.async.wait_group 1;" ::: "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ void load_vec(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ float2 load_pair(const float* p) {
    return *reinterpret_cast<const float2*>(p);
}
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
    const unsigned w = *reinterpret_cast<const unsigned*>(p);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

struct DecodeArgs {
    const void* q;             // [B, nh, hd] rows of stride q_stride
    long long q_stride;
    void* out;                 // [B, nh * hd]
    const void* k_pool;        // [n_pages, page, nkv, hd] of this layer
    const void* v_pool;
    const int* page_table;     // [n_slots, max_pages]
    const int* slots;          // [B]; negative = padding entry
    const int* positions;      // [B] position of the query (its key is stored already)
    float* part_acc;           // [B, nh, S, hd]
    float* part_ml;            // [B, nh, S, 2]
    int* counters;             // [B * gridDim.y], zero before and after a launch
    int max_pages, page, cap, nh, nkv, hd, window, n_splits, chunk;
    float scale;
};

// The decode step's q/k norm, rotation and cache store done by the attention kernel
// itself (bfloat16 tensor-core form, head sizes 64, 128, 256): with part != null the
// queries are not read from q but formed from the projection's 32-bit partial sums,
//     x = sum_g part[g][b][head];  x = x * rsqrt(mean(x^2) + eps) * w  (if w);
//     pairs (i, i + hd/2) rotated by cos / sin [B, hd/2]  (if cos),
// and with store_kv the CTA whose tiles hold position p forms the new key (the same
// way, with wk) and value (the sum alone), uses them and writes them to the cache.
// That removes a launch, and a trip of q, k and v through global memory, from a chain
// of dependent kernels.
struct FuseQK {
    const float* part;         // [G, B, (nh + 2 nkv) * hd]; null: not fused
    int G;
    const float* wq;           // [hd] or null
    const float* wk;
    float eps;
    const float* cosv;         // [B, hd / 2] or null
    const float* sinv;
    int store_kv;
};

// Writes this chunk's (maximum, normaliser), counts the chunk in and, in the
// CTA that arrives last for the (sequence, head group), merges all chunks:
// out = sum_s e^{m_s - M} acc_s / sum_s e^{m_s - M} l_s, in chunk order.
// stat: shared [gc][2] holding this chunk's (m, l); wts: shared scratch of wcap
// floats (free by now); s_last: a shared int.
template <typename T>
__device__ __forceinline__ void finish_split(const DecodeArgs& a, int b, int h0, int gc, int used,
                                             int split, float* stat, float* wts, int wcap,
                                             int* s_last, T* outp, int arrivals = 0,
                                             bool write_ml = true) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nthreads = blockDim.x, nwarps = nthreads >> 5;
    const int hd = a.hd;
    if (arrivals == 0) arrivals = used;        // one arrival per partial result
    if (write_ml && tid < gc) {
        float* dst = a.part_ml + (((size_t)b * a.nh + h0 + tid) * a.n_splits + split) * 2;
        dst[0] = stat[tid * 2];
        dst[1] = stat[tid * 2 + 1];
    }
    __threadfence();
    __syncthreads();
    int* counter = a.counters + (size_t)b * gridDim.y + blockIdx.y;
    if (tid == 0) {
        const int seen = atomicAdd(counter, 1);
        *s_last = (seen == arrivals - 1);
    }
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    if (tid == 0) *counter = 0;                         // ready for the next launch
    // pass 1: the overall maximum and normaliser of each head
    for (int hh = warp; hh < gc; hh += nwarps) {
        const float* ml = a.part_ml + ((size_t)b * a.nh + h0 + hh) * a.n_splits * 2;
        float M = -INFINITY;
        for (int sp = lane; sp < used; sp += 32) M = fmaxf(M, __ldcg(ml + 2 * sp));
        M = warp_max(M);
        float L = 0.f;
        for (int sp = lane; sp < used; sp += 32)
            L += expf(__ldcg(ml + 2 * sp) - M) * __ldcg(ml + 2 * sp + 1);
        L = warp_sum(L);
        if (lane == 0) {
            stat[hh * 2] = M;
            stat[hh * 2 + 1] = L;
        }
    }
    __syncthreads();
    // pass 2: chunks in segments whose weights fit the shared scratch.  The loads
    // of a step are issued together, with no branch between them, so they overlap.
    constexpr int EP = 8, U = 4;        // outputs per thread, chunks per step
    const int seg = max(1, min(used, wcap / gc));
    for (int base = 0; base < gc * hd; base += nthreads * EP) {
        const float* accp[EP];
        int hk[EP];
        float v[EP];
#pragma unroll
        for (int k = 0; k < EP; ++k) {
            const int i = min(base + tid + k * nthreads, gc * hd - 1);
            hk[k] = i / hd;
            accp[k] = a.part_acc + ((size_t)b * a.nh + h0 + hk[k]) * a.n_splits * hd + i % hd;
            v[k] = 0.f;
        }
        for (int s0 = 0; s0 < used; s0 += seg) {
            const int ns = min(seg, used - s0);
            __syncthreads();
            for (int i = tid; i < gc * ns; i += nthreads) {
                const int hh = i / ns, sp = s0 + i % ns;
                const float* ml = a.part_ml + ((size_t)b * a.nh + h0 + hh) * a.n_splits * 2;
                wts[hh * seg + (sp - s0)] = expf(__ldcg(ml + 2 * sp) - stat[hh * 2]);
            }
            __syncthreads();
            for (int sp = 0; sp < ns; sp += U) {
                float t[U][EP];
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int k = 0; k < EP; ++k)
                        t[u][k] = __ldcg(accp[k] + (size_t)(s0 + min(sp + u, ns - 1)) * hd);
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int k = 0; k < EP; ++k) {
                        const float w = sp + u < ns ? wts[hk[k] * seg + sp + u] : 0.f;
                        v[k] = fmaf(w, t[u][k], v[k]);
                    }
            }
        }
#pragma unroll
        for (int k = 0; k < EP; ++k) {
            const int i = base + tid + k * nthreads;
            if (i < gc * hd) outp[i] = from_f32<T>(v[k] / stat[hk[k] * 2 + 1]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(AD_THREADS)
attention_decode_split_kernel(DecodeArgs a) {
    pdl_wait();
    pdl_launch_next();
    constexpr int VEC = Vec16<T>::N;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_last;
    const int b = blockIdx.z, split = blockIdx.x;
    const int G = a.nh / a.nkv;
    const int chunks_per_group = (G + AD_GC - 1) / AD_GC;
    const int g = blockIdx.y / chunks_per_group;              // kv head
    const int h0 = g * G + (blockIdx.y % chunks_per_group) * AD_GC;   // first query head
    const int gc = min(AD_GC, g * G + G - h0);                // heads handled here
    const int hd = a.hd, CH = a.chunk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    T* outp = (T*)a.out + ((size_t)b * a.nh + h0) * hd;
    const int slot = a.slots[b];
    if (slot < 0) {
        if (split == 0)
            for (int i = tid; i < gc * hd; i += AD_THREADS) outp[i] = from_f32<T>(0.f);
        return;
    }
    const int p = a.positions[b];
    const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    const int j0 = lo + split * a.chunk;
    if (j0 > p) return;
    const int n = min(a.chunk, p - j0 + 1);                   // keys of this chunk
    const int used = (p - lo) / a.chunk + 1;                  // chunks this sequence has

    T* Ks = reinterpret_cast<T*>(smem_raw);
    T* Vs = Ks + (size_t)CH * hd;
    float* qs = reinterpret_cast<float*>(Vs + (size_t)CH * hd);   // [AD_GC][hd]
    float* sc = qs + AD_GC * hd;                                  // [AD_GC][CH]
    float* stat = sc + AD_GC * CH;                                // [AD_GC][2]
    int* rowoff = reinterpret_cast<int*>(stat + AD_GC * 2);       // [CH] row index in the pool

    // ---- where each key row of the chunk lives (one page-table read per row)
    const int* table = a.page_table + (size_t)slot * a.max_pages;
    for (int r = tid; r < n; r += AD_THREADS) {
        const int row = (j0 + r) % a.cap;
        rowoff[r] = table[row / a.page] * a.page + row % a.page;
    }
    // ---- the group's queries, 32-bit
    for (int i = tid; i < gc * hd; i += AD_THREADS) {
        const int hh = i / hd, e = i % hd;
        qs[hh * hd + e] =
            to_f32(((const T*)a.q)[(size_t)b * a.q_stride + (size_t)(h0 + hh) * hd + e]);
    }
    __syncthreads();
    // ---- keys and values of the chunk into shared memory, all copies in flight
    const int vec_per_row = hd / VEC;
    for (int i = tid; i < n * vec_per_row; i += AD_THREADS) {
        const int r = i / vec_per_row, c = (i % vec_per_row) * VEC;
        const size_t off = ((size_t)rowoff[r] * a.nkv + g) * hd + c;
        cp_async16(Ks + (size_t)r * hd + c, (const T*)a.k_pool + off);
        cp_async16(Vs + (size_t)r * hd + c, (const T*)a.v_pool + off);
    }
    cp_async_wait_all();
    __syncthreads();
    // ---- scores: one warp per key, lanes across the head dimension
    for (int r = warp; r < n; r += AD_THREADS / 32) {
        float s[AD_GC] = {0.f, 0.f, 0.f, 0.f};
        for (int e = lane * VEC; e < hd; e += 32 * VEC) {
            float kv[VEC];
            load_vec(Ks + (size_t)r * hd + e, kv);
#pragma unroll
            for (int hh = 0; hh < AD_GC; ++hh) {
                if (hh < gc) {
#pragma unroll
                    for (int i = 0; i < VEC; i += 4) {
                        const float4 qv = *reinterpret_cast<const float4*>(qs + hh * hd + e + i);
                        s[hh] = fmaf(qv.x, kv[i], s[hh]);
                        s[hh] = fmaf(qv.y, kv[i + 1], s[hh]);
                        s[hh] = fmaf(qv.z, kv[i + 2], s[hh]);
                        s[hh] = fmaf(qv.w, kv[i + 3], s[hh]);
                    }
                }
            }
        }
#pragma unroll
        for (int hh = 0; hh < AD_GC; ++hh) {
            const float t = warp_sum(s[hh]) * a.scale;
            if (lane == 0 && hh < gc) sc[hh * CH + r] = t;
        }
    }
    __syncthreads();
    // ---- softmax weights relative to the chunk's maximum: warp hh takes head hh
    for (int hh = warp; hh < gc; hh += AD_THREADS / 32) {
        float m = -INFINITY;
        for (int r = lane; r < n; r += 32) m = fmaxf(m, sc[hh * CH + r]);
        m = warp_max(m);
        float l = 0.f;
        for (int r = lane; r < n; r += 32) {
            const float w = expf(sc[hh * CH + r] - m);
            sc[hh * CH + r] = w;
            l += w;
        }
        l = warp_sum(l);
        if (lane == 0) {
            stat[hh * 2] = m;
            stat[hh * 2 + 1] = l;
        }
    }
    __syncthreads();
    // ---- weighted sum of the values: each thread owns pairs of output dimensions
    for (int d = tid * 2; d < hd; d += AD_THREADS * 2) {
        float acc[AD_GC][2] = {};
        for (int r = 0; r < n; ++r) {
            const float2 vv = load_pair(Vs + (size_t)r * hd + d);
#pragma unroll
            for (int hh = 0; hh < AD_GC; ++hh) {
                if (hh < gc) {
                    const float w = sc[hh * CH + r];
                    acc[hh][0] = fmaf(w, vv.x, acc[hh][0]);
                    acc[hh][1] = fmaf(w, vv.y, acc[hh][1]);
                }
            }
        }
#pragma unroll
        for (int hh = 0; hh < AD_GC; ++hh) {
            if (hh < gc) {
                if (used == 1) {
                    const float inv = 1.0f / stat[hh * 2 + 1];
                    outp[hh * hd + d] = from_f32<T>(acc[hh][0] * inv);
                    outp[hh * hd + d + 1] = from_f32<T>(acc[hh][1] * inv);
                } else {
                    float* dst = a.part_acc +
                                 (((size_t)b * a.nh + h0 + hh) * a.n_splits + split) * hd + d;
                    dst[0] = acc[hh][0];
                    dst[1] = acc[hh][1];
                }
            }
        }
    }
    if (used == 1) return;
    finish_split<T>(a, b, h0, gc, used, split, stat, reinterpret_cast<float*>(smem_raw),
                    (int)(((size_t)2 * CH * hd * sizeof(T)) / sizeof(float)), &s_last, outp);
}

// ------------------------------------------------------- tensor-core variant
// bfloat16, head sizes in steps of 8 up to 256: the same split of the keys, but
// a chunk's scores and weighted values are mma.sync m16n8k16 products.  The rows
// of the left operand are the query heads that share the kv head (up to 16 per
// CTA), so a group's keys and values are read once for all its heads.
constexpr int DM_HEADS = 16, DM_KEYS = 64;
// How a CTA's warps share a tile.  The arithmetic of a tile is a chain of short
// dependent instructions, so its time goes with the work per warp, not with the tensor
// pipe: head sizes above 64 take eight warps (8 keys of the scores, 2 rows of the
// softmax and an eighth of the head dimension each), head size 64 four.
template <int HDP>
struct DmShape {
    static constexpr int NT = HDP >= 128 ? 256 : 128;   // threads
    static constexpr int NW = NT / 32;                  // warps
    static constexpr int KW = DM_KEYS / NW;             // keys per warp in the scores: 16 or 8
    static constexpr int RW = DM_HEADS / NW;            // rows per warp in the softmax
    static constexpr int DW = HDP / NW;                 // dims per warp in the weighted sum
    static constexpr int NP = DW / 16;                  // pairs of 8-wide column tiles per warp
    // Tiles of keys and values in shared memory: head sizes up to 128 leave room for a
    // second one, so that a CTA that walks several tiles has the next one under way while it
    // works on this one (at 256 a second tile would cost the second CTA of the SM)
    static constexpr int NBUF = HDP <= 128 ? 2 : 1;
    // By TMA a request costs the threads next to nothing, so a third tile goes where the
    // one before this one was as soon as everybody is past it, with no barrier of its own.
    static constexpr int NBUF_TMA = HDP <= 128 ? 3 : 1;
    static_assert(DW % 16 == 0 && (KW == 16 || KW == 8), "unsupported split of a tile over warps");
};

__device__ __forceinline__ unsigned dm_smem(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void dm_ldsm4(unsigned addr, unsigned (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void dm_ldsm4t(unsigned addr, unsigned (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void dm_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0,
                                       unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// [rows][W] bf16 tiles: the 16-byte chunk c of row r sits at (c & ~7) | ((c ^ r) & 7).
template <int W>
__device__ __forceinline__ int dm_swz(int row, int chunk) {
    return row * W + (((chunk & ~7) | ((chunk ^ row) & 7)) << 3);
}
// The layout TMA leaves a [64 keys][W] tile in when it comes as W / 64 boxes of [64 rows x
// 128 bytes] with the 128-byte swizzle: box after box, inside a box row after row, the
// 16-byte chunk c of row r at c ^ (r & 7).  (The tile starts on a 1024-byte boundary.)
template <int W>
__device__ __forceinline__ int tm_swz(int row, int chunk) {
    return (chunk >> 3) * (DM_KEYS * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}
// A key / value tile's layout: as the 16-byte copies write it, or as TMA does.
template <int W, bool TMA>
__device__ __forceinline__ int kv_swz(int row, int chunk) {
    return TMA ? tm_swz<W>(row, chunk) : dm_swz<W>(row, chunk);
}
__device__ int g_decode_status = 0;   // 0, or 1 + the tile whose bounded wait gave up first

__device__ __forceinline__ void dm_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float dm_ld_peer(const float* local, unsigned rank) {
    unsigned remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(dm_smem(local)),
                 "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}


// N consecutive floats (N = 1, 2, 4; p aligned to N floats) in one load.
template <int N>
__device__ __forceinline__ void dm_ld_run(const float* p, float* dst) {
    if constexpr (N == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
    } else if constexpr (N == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        dst[0] = t.x; dst[1] = t.y;
    } else {
        dst[0] = *p;
    }
}

// One warp forms one head (hd = 64 * HALF values) from the projection's partial sums:
// a lane holds the runs [lane * HALF, +HALF) of both halves of the head, so that the
// partners of the rotation are its own.  Optional norm (w) and rotation (cs / sn rows of
// hd / 2).  The result goes, as bfloat16, to a row of a swizzled [rows][HDP] tile in
// shared memory (TMA_TILE: a key / value tile in the layout TMA writes) and, if gdst is
// given, to global memory.  Weights and angles are
// requested before the sums, so that all loads are in flight together.
template <int HDP, bool TMA_TILE = false>
__device__ __forceinline__ void dm_head_from_partials(const float* __restrict__ src, int G,
                                                      size_t split_stride,
                                                      const float* __restrict__ w, float eps,
                                                      const float* __restrict__ cs,
                                                      const float* __restrict__ sn,
                                                      __nv_bfloat16* tile, int row,
                                                      __nv_bfloat16* gdst, int lane) {
    constexpr int HALF = HDP / 64, H2 = HDP / 2;
    const int e0 = lane * HALF;
    float wv[2 * HALF], cv[HALF], sv[HALF];
    if (w) {
        dm_ld_run<HALF>(w + e0, wv);
        dm_ld_run<HALF>(w + H2 + e0, wv + HALF);
    }
    if (cs) {
        dm_ld_run<HALF>(cs + e0, cv);
        dm_ld_run<HALF>(sn + e0, sv);
    }
    float v[2 * HALF];
#pragma unroll
    for (int i = 0; i < 2 * HALF; ++i) v[i] = 0.f;
    constexpr int U = 4;                                  // partial sums loaded together
    for (int g0 = 0; g0 < G; g0 += U) {
        float t[U][2 * HALF];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float* r = src + (size_t)min(g0 + u, G - 1) * split_stride + e0;
            dm_ld_run<HALF>(r, t[u]);
            dm_ld_run<HALF>(r + H2, t[u] + HALF);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int i = 0; i < 2 * HALF; ++i) v[i] += g0 + u < G ? t[u][i] : 0.f;
    }
    if (w) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 2 * HALF; ++i) ss += v[i] * v[i];
        ss = warp_sum(ss);
        const float rs = 1.0f / sqrtf(ss / (float)HDP + eps);
#pragma unroll
        for (int i = 0; i < 2 * HALF; ++i) v[i] = v[i] * rs * wv[i];
    }
    if (cs) {
#pragma unroll
        for (int i = 0; i < HALF; ++i) {
            const float re = v[i], im = v[HALF + i];
            v[i] = re * cv[i] - im * sv[i];
            v[HALF + i] = re * sv[i] + im * cv[i];
        }
    }
    // (HALF consecutive values of each half: 2 * HALF bytes, inside one 16-byte chunk)
#pragma unroll
    for (int i = 0; i < 2 * HALF; ++i) {
        const int e = (i < HALF ? e0 + i : H2 + e0 + i - HALF);
        const __nv_bfloat16 x = __float2bfloat16_rn(v[i]);
        tile[kv_swz<HDP, TMA_TILE>(row, e >> 3) + (e & 7)] = x;
        if (gdst) gdst[e] = x;
    }
}

// The tensor-core form (bfloat16).  The gridDim.x CTAs of a (sequence, head group)
// share the sequence's tiles of 64 keys by stride, each with a running softmax over
// the tiles it walks.  cs = 2, 4, 8: every cs of them form a thread-block cluster
// and merge through distributed shared memory; with more than one cluster per
// sequence each cluster leaves one partial result in global scratch and the last
// CTA to arrive merges them.  cs = 1 with several CTAs: every CTA's partial result
// goes through scratch.
//
// TMA: the tiles are the cache's pages (page and tile are 64 positions, hd == HDP, the ring
// a whole number of pages): tile k holds positions 64 k .. 64 k + 63, and one thread asks
// for it with a box of [64 rows x 128 bytes] per 128 bytes of head width and operand (maps
// over the pools as [rows, kv heads, hd]) instead of all threads with 16 bytes each, whose
// issue alone took a third of a tile's time.  The first page of a window and the last of
// the sequence are masked by position, and value rows outside lo .. p are zeroed in shared
// memory, since what a page holds there is left over from an earlier user.  The waits for
// a tile are bounded; one that gives up leaves a code for agv_attention_decode_status and
// the kernel goes on (its result is void).
// The pools' tensor maps are a kernel argument of the TMA form only.
template <bool TMA>
struct PoolMaps {
    CUtensorMap k, v;
};
template <>
struct PoolMaps<false> {};

template <int HDP, bool TMA>
__global__ void __launch_bounds__(DmShape<HDP>::NT, DmShape<HDP>::NT == 256 ? 2 : 3)
attention_decode_mma_kernel(DecodeArgs a, int cs, FuseQK fq,
                            const __grid_constant__ PoolMaps<TMA> maps) {
    typedef DmShape<HDP> Sh;
    constexpr int DM_THREADS = Sh::NT;
    // Slots, positions and page tables are written by copies at the start of the step,
    // before any kernel of it runs, so they are read before this kernel waits for its
    // predecessor (which writes q and the new key and value): two dependent trips to
    // memory leave the chain.
    pdl_launch_next();
    typedef __nv_bfloat16 T;
    extern __shared__ __align__(128) unsigned char smem_raw0[];
    __shared__ int s_last;
    __shared__ uint64_t kv_bar[3];                          // TMA: a tile's bytes have arrived
    constexpr int NBUF = TMA ? Sh::NBUF_TMA : Sh::NBUF;
    constexpr int TILE = DM_KEYS * HDP;
    // (tiles that TMA writes with the 128-byte swizzle start on 1024-byte boundaries)
    unsigned char* smem_raw =
        TMA ? (unsigned char*)(((uintptr_t)smem_raw0 + 1023) & ~(uintptr_t)1023) : smem_raw0;
    T* Ks = reinterpret_cast<T*>(smem_raw);                 // [64][HDP]
    T* Vs = Ks + DM_KEYS * HDP;                             // [64][HDP]
    T* Ks1 = Vs + DM_KEYS * HDP;                            // the second tile (and the third after it)
    T* Vs1 = Ks1 + DM_KEYS * HDP;
    T* Qs = Ks + 2 * NBUF * TILE;                           // [16][HDP]
    T* Ps = Qs + DM_HEADS * HDP;                            // [16][64]
    float* Ss = reinterpret_cast<float*>(Ps + DM_HEADS * DM_KEYS);   // [16][64]
    float* stat = Ss + DM_HEADS * DM_KEYS;                  // [16][2] running maximum and sum
    float* fac = stat + DM_HEADS * 2;                       // [16] what a new maximum scales O by
    int* rowoff = reinterpret_cast<int*>(fac + DM_HEADS);   // [2][64]: this tile's and the next

    // The W = gridDim.x CTAs of a sequence share its tiles of 64 keys: CTA w walks the
    // tiles w, w + W, w + 2 W, ... with a running softmax.  W is chosen from the batch
    // (all CTAs of a launch resident at once), not from the context length, so a short
    // sequence leaves no CTA without work but the last ones, and a long one costs more
    // tiles per CTA, not more CTAs.
    const int W = gridDim.x;
    const int b = blockIdx.z, split = blockIdx.x;
    const int G = a.nh / a.nkv;
    const int groups_per_kv = (G + DM_HEADS - 1) / DM_HEADS;
    const int g = blockIdx.y / groups_per_kv;
    const int h0 = g * G + (blockIdx.y % groups_per_kv) * DM_HEADS;
    const int gc = min(DM_HEADS, g * G + G - h0);
    const int hd = a.hd;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tig = lane & 3;
    T* outp = (T*)a.out + ((size_t)b * a.nh + h0) * hd;
    const int slot = a.slots[b];
    if (slot < 0) {
        pdl_wait();
        if (split == 0)
            for (int i = tid; i < gc * hd; i += DM_THREADS) outp[i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int p = a.positions[b];
    const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    // Tiles this sequence has: from its first key on, or (TMA) the cache pages it touches.
    // A full window in a ring of its own size is the ring's pages, every row of them: the
    // tiles are then counted in ring rows (tile k is the ring's page k), which saves the
    // page that a window's two ragged ends would otherwise cost.
    const bool ringed = TMA && a.window > 0 && a.cap == a.window && p >= a.window - 1;
    const int pt = ringed ? p % a.cap : p;                    // p on the scale the tiles are counted in
    const int k0 = TMA && !ringed ? lo / DM_KEYS : 0;
    const int all_tiles = ringed ? a.cap / DM_KEYS
                          : TMA  ? p / DM_KEYS - k0 + 1 : (p - lo) / DM_KEYS + 1;
    const int used = min(W, all_tiles);                       // CTAs of it with work
    const int cid = split / cs, crank = split % cs;
    const int used_clusters = (used + cs - 1) / cs;
    if (cid >= used_clusters) {                               // the whole cluster is without work
        pdl_wait();
        return;
    }
    const bool has = split < all_tiles;                       // (always true when cs == 1)
    const int n_tiles = has ? (all_tiles - 1 - split) / W + 1 : 0;    // tiles this CTA walks
    // first key of its first tile
    const int j0 = TMA ? (k0 + split) * DM_KEYS : lo + split * DM_KEYS;
    float* Osm = reinterpret_cast<float*>(Ks);                // [16][HDP], after the scores are done
    const int* table = a.page_table + (size_t)slot * a.max_pages;
    // cache row of key (first + tid), or -1 beyond position p
    auto row_of = [&](int first) {
        const int key = first + tid;
        const int row = key % a.cap;
        return key <= p ? table[row / a.page] * a.page + row % a.page : -1;
    };
    if (!TMA && has && tid < DM_KEYS) {
        rowoff[tid] = row_of(j0);
        if (NBUF == 2 && n_tiles > 1) rowoff[DM_KEYS + tid] = row_of(j0 + W * DM_KEYS);
    }
    // A CTA that walks more tiles than it has buffers looks their rows up inside the walk,
    // between two barriers, where a division by a runtime value (a hundred cycles) shows:
    // thread t keeps the key it looks up next and that key's place in the ring and steps
    // both by a tile's distance.  (Set up only for such a CTA: a CTA with a single tile,
    // the common case of a short batch, is better off without the set-up; and only where
    // the registers are there for it: with heads of 256 they are not.)
    constexpr bool WALK = !TMA && HDP <= 128;
    const int pshift = (a.page & (a.page - 1)) == 0 ? 31 - __clz(a.page) : -1;
    int look_key = 0, look_ring = 0, step_ring = 0;
    if (WALK && n_tiles > NBUF && tid < DM_KEYS) {
        look_key = j0 + NBUF * W * DM_KEYS + tid;
        look_ring = look_key % a.cap;
        step_ring = (W * DM_KEYS) % a.cap;
    }
    // cache row of this thread's key of the next tile, or -1 beyond position p
    auto next_lookup = [&]() {
        int r = -1;
        if (look_key <= p)
            r = pshift >= 0 ? (table[look_ring >> pshift] << pshift) + (look_ring & (a.page - 1))
                            : table[look_ring / a.page] * a.page + look_ring % a.page;
        look_key += W * DM_KEYS;
        look_ring += step_ring;
        if (look_ring >= a.cap) look_ring -= a.cap;
        return r;
    };
    if (TMA && tid == 0) {
        tc5::mbar_init(&kv_bar[0], 1);
        tc5::mbar_init(&kv_bar[1], 1);
        tc5::mbar_init(&kv_bar[2], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    constexpr int CPR = HDP / 8;
    // TMA: a tile is asked for box by box, each box by the first lane of a warp of its own
    // (a request holds its thread for a hundred cycles, and every warp is needed at the
    // next barrier).  Those lanes step tile and ring place as above (look_key is the
    // tile's first position there, a multiple of 64; the ring holds whole pages).  The
    // barrier of the tile's buffer counts its bytes in.
    const bool asks = TMA && lane == 0 && warp < 2 * (HDP / 64);
    if (asks) {
        look_ring = j0 % a.cap;
        step_ring = (W * DM_KEYS) % a.cap;
    }
    auto next_page = [&]() {                                   // its first cache row
        const int row0 = table[look_ring >> 6] << 6;
        look_ring += step_ring;
        if (look_ring >= a.cap) look_ring -= a.cap;
        return row0;
    };
    auto request_page = [&](int buf, int row0) {               // (only where asks)
        uint64_t* bar = &kv_bar[buf];
        if (warp == 0) tc5::mbar_expect_tx(bar, 2 * TILE * (unsigned)sizeof(T));
        const int x = warp >> 1;
        if constexpr (TMA)
            tc5::tma_load_3d(Ks + (buf * 2 + (warp & 1)) * TILE + x * DM_KEYS * 64,
                             warp & 1 ? &maps.v : &maps.k, x * 64, g, row0, bar);
    };
    // With a single buffer (head size 256) keys and values are asked for apart, each as soon
    // as its half of the buffer is free: the next tile's keys when everybody has this tile's
    // scores, its values when everybody has this tile's weighted sum (kv_bar[0] counts the
    // keys in, kv_bar[1] the values), so that a trip to memory runs beside half a tile's work
    // instead of beside none.
    constexpr bool APART = TMA && NBUF == 1;
    auto request_half = [&](int which, int row0) {             // (only where asks)
        if ((warp & 1) != which) return;
        uint64_t* bar = &kv_bar[which];
        if (warp == which) tc5::mbar_expect_tx(bar, TILE * (unsigned)sizeof(T));
        const int x = warp >> 1;
        if constexpr (TMA)
            tc5::tma_load_3d(Ks + which * TILE + x * DM_KEYS * 64, which ? &maps.v : &maps.k,
                             x * 64, g, row0, bar);
    };
    // Keys and values of earlier positions were stored by earlier steps: their copies
    // start before the wait too.  Only the row of position p is the predecessor's.
    const int r_new = p - j0;                                 // in [0, 64): the first tile holds p
    // One tile's keys and values into shared memory as one group of copies.  ro: the
    // tile's cache rows (-1 beyond position p); skip: the row of the new position, which is
    // not in the cache yet (or out of the tile).
    auto request_tile = [&](T* kd, T* vd, const int* ro, int skip) {
#pragma unroll 2
        for (int i = tid; i < DM_KEYS * CPR; i += DM_THREADS) {
            const int r = i / CPR, c = i % CPR;
            const int off = dm_swz<HDP>(r, c);
            if (r == skip) continue;
            if (ro[r] >= 0 && c * 8 < hd) {
                const size_t src = ((size_t)ro[r] * a.nkv + g) * hd + c * 8;
                cp_async16(kd + off, (const T*)a.k_pool + src);
                cp_async16(vd + off, (const T*)a.v_pool + src);
            } else {
                *reinterpret_cast<uint4*>(kd + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + off) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };
    if (TMA) {
        if (has && asks) {
            if (APART) {
                const int row0 = next_page();
                request_half(0, row0);
                request_half(1, row0);
            } else {
                for (int t = 0; t < min(n_tiles, NBUF); ++t) request_page(t, next_page());
            }
        }
    } else if (has) {
        // the first tile (and the second, where there is room for it); the others are
        // requested inside the walk below
        request_tile(Ks, Vs, rowoff, r_new);
        if (NBUF == 2 && n_tiles > 1)
            request_tile(Ks1, Vs1, rowoff + DM_KEYS, p - (j0 + W * DM_KEYS));
    }
    int p_row = -1;                                         // TMA: the cache row of position p
    if (TMA) {
        const int pr = p % a.cap;
        p_row = (table[pr >> 6] << 6) + (pr & 63);
    }
    const bool fused = fq.part != nullptr;                  // (then hd == HDP)
    if (has && fused) {
        // rows of the query tile beyond the group's heads are zero: nothing of the
        // predecessor's, so they are written before the wait
        for (int i = tid; i < (DM_HEADS - gc) * CPR; i += DM_THREADS)
            *reinterpret_cast<uint4*>(Qs + dm_swz<HDP>(gc + i / CPR, i % CPR)) = make_uint4(0, 0, 0, 0);
    }
    pdl_wait();
    if (has) {
    const size_t f_width = (size_t)(a.nh + 2 * a.nkv) * hd;  // a row of the projection
    const size_t f_stride = (size_t)gridDim.z * f_width;     // one partial sum of the batch
    const float* f_cos = fused && fq.cosv ? fq.cosv + (size_t)b * (hd / 2) : nullptr;
    const float* f_sin = fused && fq.cosv ? fq.sinv + (size_t)b * (hd / 2) : nullptr;
    // queries of the group: rows beyond the group's heads and dims beyond hd are zero
    if (!fused) {
#pragma unroll 1
    for (int i = tid; i < DM_HEADS * CPR; i += DM_THREADS) {
        const int r = i / CPR, c = i % CPR;
        T* dst = Qs + dm_swz<HDP>(r, c);
        if (r < gc && c * 8 < hd) {
            cp_async16(dst, (const T*)a.q + (size_t)b * a.q_stride + (size_t)(h0 + r) * hd +
                                c * 8);
        } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
    }
    if (fused)
        for (int r = warp; r < gc; r += DM_THREADS / 32)
            dm_head_from_partials<HDP>(fq.part + (size_t)b * f_width + (size_t)(h0 + r) * hd, fq.G,
                                       f_stride, fq.wq, fq.eps, f_cos, f_sin, Qs, r, nullptr, lane);
    // the new position's key and value: from the cache, or formed here and stored
    auto new_row = [&](T* Ks, T* Vs, int r, int cache_row) {
        if (fused && fq.store_kv) {
            const bool writer = blockIdx.y % groups_per_kv == 0 && cache_row >= 0;
            T* kd = writer ? (T*)a.k_pool + ((size_t)cache_row * a.nkv + g) * hd : nullptr;
            T* vd = writer ? (T*)a.v_pool + ((size_t)cache_row * a.nkv + g) * hd : nullptr;
            const float* src = fq.part + (size_t)b * f_width;
            // (by the warps after those that form the queries, if there are any)
            if (warp == gc % Sh::NW)
                dm_head_from_partials<HDP, TMA>(src + (size_t)(a.nh + g) * hd, fq.G, f_stride,
                                                fq.wk, fq.eps, f_cos, f_sin, Ks, r, kd, lane);
            else if (warp == (gc + 1) % Sh::NW)
                dm_head_from_partials<HDP, TMA>(src + (size_t)(a.nh + a.nkv + g) * hd, fq.G,
                                                f_stride, nullptr, 0.f, nullptr, nullptr, Vs, r,
                                                vd, lane);
            return;
        }
        for (int c = tid; c < CPR; c += DM_THREADS) {
            const int off = kv_swz<HDP, TMA>(r, c);
            if (cache_row >= 0 && c * 8 < hd) {
                const size_t src = ((size_t)cache_row * a.nkv + g) * hd + c * 8;
                cp_async16(Ks + off, (const T*)a.k_pool + src);
                cp_async16(Vs + off, (const T*)a.v_pool + src);
            } else {
                *reinterpret_cast<uint4*>(Ks + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(Vs + off) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    if (!TMA && r_new >= 0 && r_new < DM_KEYS) new_row(Ks, Vs, r_new, rowoff[r_new]);
    constexpr int NP = Sh::NP;
    float o[NP * 2][4] = {};
    int ahead_row0 = -1;                                    // TMA: first cache row of the page asked for next
    for (int tt = 0; tt < n_tiles; ++tt) {
    const int jt = j0 + tt * W * DM_KEYS;                   // first key of this tile
    const int n = ringed ? DM_KEYS : min(DM_KEYS, p - jt + 1);    // its keys: rows nlo .. n - 1
    const int nlo = TMA && !ringed ? max(0, lo - jt) : 0;
    const bool last = tt + 1 == n_tiles;
    // this tile's buffers (the tiles take turns where there are two or three)
    const int buf = NBUF == 1 ? 0 : NBUF == 2 ? tt & 1 : tt % NBUF;
    T* const Kt = Ks + buf * 2 * TILE;
    T* const Vt = Kt + TILE;
    bool top_barrier = true, values_here = true;
    // the rows of the tile that is requested next (the next one; with two buffers the one
    // after it): the lookup runs beside this tile's work
    const int ahead = NBUF * W * DM_KEYS;
    int next_row = -1;
    if (!TMA && tt + NBUF < n_tiles && tid < DM_KEYS)
        next_row = WALK ? next_lookup() : row_of(jt + ahead);
    if constexpr (TMA) {
        if (NBUF == 1 && tt > 0) {
            // the tile before has been used up: this one's values replace its values (this
            // one's keys were asked for when the scores of the tile before were done)
            __syncthreads();
            if (asks) request_half(1, ahead_row0);
        }
        // The page that is asked for next is looked up beside this tile's work: with one
        // buffer the next tile's, asked for at the top of the next round; with three the
        // tile after the next, asked for below as soon as everybody is past the tile before
        // this one, whose buffer it takes (tiles 0 to 2 were asked for at the start).
        if (asks && (NBUF == 1 ? tt + 1 < n_tiles : tt >= 1 && tt + 2 < n_tiles))
            ahead_row0 = next_page();
        if (!tc5::mbar_wait(&kv_bar[buf], (tt / NBUF) & 1) && tid == 0)
            atomicCAS(&g_decode_status, 0, 1 + tt);
        const int rn0 = pt - jt;
        values_here = !APART;
        if (APART && ((rn0 >= 0 && rn0 < DM_KEYS) || nlo > 0 || n < DM_KEYS)) {
            // a tile that is written into by hand: its values have to be there as well
            if (!tc5::mbar_wait(&kv_bar[1], tt & 1) && tid == 0)
                atomicCAS(&g_decode_status, 0, 1 + tt);
            values_here = true;
        }
        // the tile has landed: the new position's row goes over what the page held there,
        // and the value rows of positions that do not count are zeroed (written by hand,
        // so ordered here before the copy that may overwrite the buffer later)
        const int rn = pt - jt;
        const int dead = nlo + (DM_KEYS - n);                 // rows 0 .. nlo - 1 and n .. 63
        const bool holds_new = rn >= 0 && rn < DM_KEYS;
        if (holds_new) new_row(Kt, Vt, rn, p_row);
        for (int i = tid; i < dead * CPR; i += DM_THREADS) {
            const int q = i / CPR, r = q < nlo ? q : n + q - nlo;
            *reinterpret_cast<uint4*>(Vt + tm_swz<HDP>(r, i % CPR)) = make_uint4(0, 0, 0, 0);
        }
        if (holds_new || dead > 0) tc5::fence_async_shared();
        // between two tiles that came whole nobody has written anything the others read
        // before the next barrier, so the walk goes on without one
        top_barrier = tt == 0 || holds_new || dead > 0;
    } else if (tt > 0) {
        const int* ro = rowoff + (tt & 1) * DM_KEYS;
        const int rn = p - jt;                               // the new position's row, if in this tile
        if (NBUF == 1) {
            // the tile before has been used up: this one replaces it
            __syncthreads();
            request_tile(Kt, Vt, ro, rn);
        }
        if (rn >= 0 && rn < DM_KEYS) new_row(Kt, Vt, rn, ro[rn]);
    }
    // (with two buffers the tile after this one stays in flight; the first tile waits for
    // everything because the queries' copies, made after the dependency wait, are among it,
    // and so does a CTA's last tile, which may hold the new position)
    if (!TMA && NBUF == 2 && !last && tt > 0) cp_async_wait_but_one(); else cp_async_wait_all();
    if (top_barrier) __syncthreads();
    // ---- scores of 16 heads x this warp's keys
    if constexpr (Sh::KW == 16) {
        float s[2][4] = {};
#pragma unroll
        for (int kk = 0; kk < HDP / 16; ++kk) {
            unsigned af[4], bf[4];
            dm_ldsm4(dm_smem(Qs + dm_swz<HDP>(lane & 15, kk * 2 + (lane >> 4))), af);
            const int mat = lane >> 3, r = lane & 7;
            dm_ldsm4(dm_smem(Kt + kv_swz<HDP, TMA>(warp * 16 + r + (mat >> 1) * 8,
                                                   kk * 2 + (mat & 1))), bf);
            dm_mma(s[0], af, bf[0], bf[1]);
            dm_mma(s[1], af, bf[2], bf[3]);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = warp * 16 + i * 8 + tig * 2 + (e & 1);
                const int row = gid + (e >> 1) * 8;
                Ss[row * DM_KEYS + key] =
                    key >= nlo && key < n ? s[i][e] * a.scale : -INFINITY;
            }
    } else {
        // 8 keys: one load brings their chunks of 32 dims, two products into sums of
        // their own; four such sums in turn, so that a product waits for the one two loads
        // back and not for its neighbour, added at the end
        float s[4][4] = {};
#pragma unroll
        for (int k2 = 0; k2 < HDP / 32; ++k2) {
            unsigned a0[4], a1[4], bf[4];
            dm_ldsm4(dm_smem(Qs + dm_swz<HDP>(lane & 15, k2 * 4 + (lane >> 4))), a0);
            dm_ldsm4(dm_smem(Qs + dm_swz<HDP>(lane & 15, k2 * 4 + 2 + (lane >> 4))), a1);
            dm_ldsm4(dm_smem(Kt + kv_swz<HDP, TMA>(warp * 8 + (lane & 7), k2 * 4 + (lane >> 3))),
                     bf);
            dm_mma(s[(k2 & 1) * 2], a0, bf[0], bf[1]);
            dm_mma(s[(k2 & 1) * 2 + 1], a1, bf[2], bf[3]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = warp * 8 + tig * 2 + (e & 1);
            const int row = gid + (e >> 1) * 8;
            Ss[row * DM_KEYS + key] = key >= nlo && key < n
                ? ((s[0][e] + s[1][e]) + (s[2][e] + s[3][e])) * a.scale : -INFINITY;
        }
    }
    __syncthreads();
    if (TMA && NBUF == 3 && asks && tt >= 1 && tt + 2 < n_tiles)
        request_page((tt + 2) % NBUF, ahead_row0);      // everybody is past the tile before this one
    if (APART && asks && tt + 1 < n_tiles)
        request_half(0, ahead_row0);                    // everybody is past this tile's keys
    // ---- softmax weights relative to the running maximum.  Rows are dealt round the
    // warps, so that the few heads of a small group get a warp each; rows beyond the
    // group's heads are padding whose products nobody reads, and are left as they are.
#pragma unroll
    for (int rr = 0; rr < Sh::RW; ++rr) {
        const int row = rr * Sh::NW + warp;
        if (row >= gc) break;
        const float s0 = Ss[row * DM_KEYS + lane], s1 = Ss[row * DM_KEYS + lane + 32];
        const float m_old = tt > 0 ? stat[row * 2] : -INFINITY;
        const float l_old = tt > 0 ? stat[row * 2 + 1] : 0.f;
        const float m = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
        const float alpha = tt > 0 ? expf(m_old - m) : 0.f;
        const float w0 = expf(s0 - m), w1 = expf(s1 - m);
        const float l = fmaf(l_old, alpha, warp_sum(w0 + w1));
        Ps[dm_swz<DM_KEYS>(row, lane >> 3) + (lane & 7)] = __float2bfloat16_rn(w0);
        Ps[dm_swz<DM_KEYS>(row, (lane >> 3) + 4) + (lane & 7)] = __float2bfloat16_rn(w1);
        __syncwarp();                              // every lane has read the old values
        if (lane == 0) {
            stat[row * 2] = m;
            stat[row * 2 + 1] = l;
            fac[row] = alpha;
        }
    }
    __syncthreads();
    if (APART && !values_here && !tc5::mbar_wait(&kv_bar[1], tt & 1) && tid == 0)
        atomicCAS(&g_decode_status, 0, 1 + tt);
    // ---- weighted values: this warp's share of the head dimension
    {
        if (tt > 0) {
            const float f0 = fac[gid], f1 = fac[gid + 8];
#pragma unroll
            for (int i = 0; i < NP * 2; ++i) {
                o[i][0] *= f0, o[i][1] *= f0;
                o[i][2] *= f1, o[i][3] *= f1;
            }
        }
#pragma unroll
        for (int kk = 0; kk < DM_KEYS / 16; ++kk) {
            unsigned af[4];
            dm_ldsm4(dm_smem(Ps + dm_swz<DM_KEYS>(lane & 15, kk * 2 + (lane >> 4))), af);
#pragma unroll
            for (int nn = 0; nn < NP; ++nn) {
                unsigned bf[4];
                const int mat = lane >> 3, r = lane & 7;
                dm_ldsm4t(dm_smem(Vt + kv_swz<HDP, TMA>(kk * 16 + r + (mat & 1) * 8,
                                                        warp * (Sh::DW / 8) + nn * 2 + (mat >> 1))),
                          bf);
                dm_mma(o[nn * 2], af, bf[0], bf[1]);
                dm_mma(o[nn * 2 + 1], af, bf[2], bf[3]);
            }
        }
    }
    if (TMA) {
        // (asked for above, or at the top of the next round)
    } else if (NBUF == 2) {
        if (tt + 2 < n_tiles) {
            // this tile's buffers are used up: the tile after the next goes there
            if (tid < DM_KEYS) rowoff[(tt & 1) * DM_KEYS + tid] = next_row;
            __syncthreads();
            request_tile(Kt, Vt, rowoff + (tt & 1) * DM_KEYS, p - (jt + ahead));
        }
    } else if (!last && tid < DM_KEYS) {
        rowoff[((tt + 1) & 1) * DM_KEYS + tid] = next_row;
    }
    }   // tiles
    {
        if (cs > 1 && used > 1) __syncthreads();   // Osm lies over the last key tile
#pragma unroll
        for (int i = 0; i < NP * 2; ++i) {
            const int d = warp * Sh::DW + i * 8 + tig * 2;
            if (d >= hd) continue;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = gid + half * 8;
                if (row >= gc) continue;
                const float v0 = o[i][half * 2], v1 = o[i][half * 2 + 1];
                if (used == 1) {
                    const float inv = 1.0f / stat[row * 2 + 1];
                    outp[row * hd + d] = __float2bfloat16_rn(v0 * inv);
                    outp[row * hd + d + 1] = __float2bfloat16_rn(v1 * inv);
                } else if (cs > 1) {
                    Osm[row * HDP + d] = v0;
                    Osm[row * HDP + d + 1] = v1;
                } else {
                    float* dst = a.part_acc +
                                 (((size_t)b * a.nh + h0 + row) * a.n_splits + split) * hd + d;
                    dst[0] = v0;
                    dst[1] = v1;
                }
            }
        }
    }
    } else if (tid < DM_HEADS) {
        // a chunk past the sequence's end inside a live cluster contributes nothing
        stat[tid * 2] = -INFINITY;
        stat[tid * 2 + 1] = 0.f;
    }
    if (used == 1) return;                     // (one chunk: its cluster has no other live CTA)
    const int wcap = (int)((size_t)2 * DM_KEYS * HDP * sizeof(T) / sizeof(float));
    if (cs == 1) {
        finish_split<T>(a, b, h0, gc, used, split, stat, reinterpret_cast<float*>(smem_raw), wcap,
                        &s_last, outp);
        return;
    }
    // ---- merge inside the cluster: rank r owns a slice of the head dimension
    dm_cluster_sync();
    {
        const int DS = HDP / cs;                               // dims per rank
        for (int item = tid; item < gc * DS; item += DM_THREADS) {
            const int row = item / DS, d = crank * DS + item % DS;
            float mq[8], lq[8], oq[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const unsigned qq = q < cs ? q : 0;
                mq[q] = dm_ld_peer(stat + row * 2, qq);
                lq[q] = dm_ld_peer(stat + row * 2 + 1, qq);
                oq[q] = dm_ld_peer(Osm + row * HDP + d, qq);
            }
            float M = -INFINITY;
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (q < cs) M = fmaxf(M, mq[q]);
            float L = 0.f, O = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                if (q < cs && lq[q] > 0.f) {                  // a peer without keys holds no data
                    const float w = expf(mq[q] - M);
                    L = fmaf(w, lq[q], L);
                    O = fmaf(w, oq[q], O);
                }
            }
            if (d < hd) {
                if (used_clusters == 1) {
                    outp[row * hd + d] = __float2bfloat16_rn(O / L);
                } else {
                    a.part_acc[(((size_t)b * a.nh + h0 + row) * a.n_splits + cid) * hd + d] = O;
                    if (d == 0) {
                        float* ml = a.part_ml + (((size_t)b * a.nh + h0 + row) * a.n_splits + cid) * 2;
                        ml[0] = M;
                        ml[1] = L;
                    }
                }
            }
        }
    }
    dm_cluster_sync();                         // nobody leaves while a peer may still read it
    if (used_clusters == 1) return;
    // a long sequence: one partial result per cluster, merged by the last CTA to arrive
    finish_split<T>(a, b, h0, gc, used_clusters, cid, stat, reinterpret_cast<float*>(smem_raw), wcap,
                    &s_last, outp, used_clusters * cs, false);
}

// A pool [rows, nkv, hd] bfloat16 as a 3-D tensor map read in boxes of [64 rows, 1 head, 64
// elements]; kept per (pool, nkv, hd).  The number of rows a pool holds is not known
// here: the map is given more than any pool has, and the rows asked for come from the
// page table.
int make_pool_map(CUtensorMap* out, const void* pool, int nkv, int hd) {
    typedef std::tuple<const void*, int, int> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key(pool, nkv, hd);
    {
        std::lock_guard<std::mutex> gl(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *out = it->second;
            return 0;
        }
    }
    tc5::EncodeTiledFn fn = tc5::encode_fn();
    if (!fn) return agv_fail(-4, "attention_decode: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nkv, (cuuint64_t)1 << 31};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)nkv * hd * 2};
    cuuint32_t box[3] = {64, 1, (cuuint32_t)DM_KEYS};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(pool), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return agv_fail(-4, "attention_decode: cuTensorMapEncodeTiled failed with code %d (kv heads "
                        "%d, head_dim %d)", (int)r, nkv, hd);
    std::lock_guard<std::mutex> gl(mu);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

// Which way the tensor-core form brings its tiles: 0 chosen from the sizes, 1 always 16-byte
// copies, 2 TMA wherever its sizes allow (AGAVE_B200_DECODE_TILES=copies|tma, or
// agv_attention_decode_set_tiles; for tests and measurements).
int g_decode_tiles = -1;
int decode_tiles_form() {
    if (g_decode_tiles < 0) {
        const char* e = getenv("AGAVE_B200_DECODE_TILES");
        g_decode_tiles = !e ? 0 : !strcmp(e, "copies") ? 1 : !strcmp(e, "tma") ? 2 : 0;
    }
    return g_decode_tiles;
}

int decode_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sms = 148;
    }
    return sms;
}

// CTAs per sequence: as many as stay resident together over the whole batch, at most one
// per tile of the longest sequence a launch may see; up to eight form a cluster, more
// clusters leave one partial result each.
void ctas_per_sequence(int resident, int pairs, int most, int* cs, int* clusters) {
    int per_seq = resident / pairs;
    if (per_seq > most) per_seq = most;
    if (per_seq < 1) per_seq = 1;
    *cs = 1;
    while (*cs < 8 && *cs * 2 <= per_seq) *cs *= 2;
    *clusters = per_seq / *cs;
    if (*clusters < 1) *clusters = 1;
    if (*clusters > 16) *clusters = 16;
}

// The tiles of the longest sequence a launch may see (a.n_splits on entry): as pages, a
// window that does not start on one touches one page more, unless it is a ring of its own
// size.
int most_tiles(const DecodeArgs& a, bool pages) {
    return a.n_splits + (pages && a.window > 0 && a.cap != a.window ? 1 : 0);
}

template <int HDP, bool TMA>
int launch_decode_mma(const DecodeArgs& a0, int B, cudaStream_t stream, const FuseQK& fq) {
    auto kern = attention_decode_mma_kernel<HDP, TMA>;
    constexpr int DM_THREADS = DmShape<HDP>::NT;
    constexpr int NBUF = TMA ? DmShape<HDP>::NBUF_TMA : DmShape<HDP>::NBUF;
    constexpr int smem = (2 * NBUF * DM_KEYS + DM_HEADS) * HDP * 2 + DM_HEADS * DM_KEYS * (2 + 4) +
                         DM_HEADS * 3 * 4 + 2 * DM_KEYS * 4 + (TMA ? 1024 : 0);
    static bool configured = false;
    static int resident = 0;
    if (!configured) {
        AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        int dev = 0, sms = 0, per_sm = 0;
        AGV_CUDA_OK(cudaGetDevice(&dev));
        AGV_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        AGV_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, DM_THREADS, smem));
        resident = sms * (per_sm > 0 ? per_sm : 1);
        configured = true;
    }
    DecodeArgs a = a0;
    PoolMaps<TMA> maps;
    if constexpr (TMA) {
        if (int rc = make_pool_map(&maps.k, a.k_pool, a.nkv, a.hd)) return rc;
        if (int rc = make_pool_map(&maps.v, a.v_pool, a.nkv, a.hd)) return rc;
    }
    const int G = a.nh / a.nkv;
    const int groups = a.nkv * ((G + DM_HEADS - 1) / DM_HEADS);
    int cs, clusters;
    ctas_per_sequence(resident, groups * B, most_tiles(a, TMA), &cs, &clusters);
    a.n_splits = clusters;                         // partial results per (sequence, head)
    dim3 grid(clusters * cs, groups, B);
    if (cs > 1)
        agv_launch_cluster(kern, grid, DM_THREADS, smem, stream, dim3(cs, 1, 1), a, cs, fq, maps);
    else
        agv_launch(kern, grid, DM_THREADS, smem, stream, a, 1, fq, maps);
    AGV_LAUNCH_OK("attention_decode_mma_kernel");
    return 0;
}

// The tensor-core form for a head size, its tiles by TMA where the cache's geometry is the
// tiles' (pages of 64 positions, a ring of whole pages, a head as wide as its tile).
template <int HDP>
int launch_decode_form(const DecodeArgs& a, int B, cudaStream_t stream, const FuseQK& fq) {
    const bool can = a.page == DM_KEYS && a.cap % DM_KEYS == 0 && a.hd == HDP &&
                     agv_aligned(a.k_pool, 128) && agv_aligned(a.v_pool, 128);
    const int form = decode_tiles_form();
    // A request by TMA saves its time per tile, and a window that does not start on a page
    // costs a page more than it has tiles: taken where a CTA may walk four tiles or more
    // (six with heads of 256, where 8 sequences of a 1B step, four tiles a CTA at most and in
    // the measured case one, lose 0.9 % of the step to it although the kernel alone is as
    // fast; two where a window is a ring of its own size, whose pages are its tiles exactly).
    // Measured alone, 16-byte copies against TMA: 16 sequences with the 27B model's heads
    // and a window of 1,024, one CTA a pair, 34.8 -> 26.5 us; 64 sequences of up to 2,048
    // with heads of 256, four CTAs a sequence, 32.3 -> 23.7, and 125 -> 77 at 4,096 to
    // 8,000 positions; 8 sequences of 256 to 4,096 with four kv heads of 256 32.6 -> 23.6;
    // 64 sequences with a ring of 512 12.5 -> 11.2; but one tile per CTA (8 sequences with
    // a ring of 512) 5.7 -> 6.1, which stays with the copies.
    bool tma = can && form == 2;
    if (can && form == 0) {
        const int G = a.nh / a.nkv, groups = a.nkv * ((G + DM_HEADS - 1) / DM_HEADS);
        int cs, clusters;
        const int most = most_tiles(a, true);
        ctas_per_sequence(decode_sms() * (DmShape<HDP>::NT == 256 ? 2 : 3), groups * B, most, &cs,
                          &clusters);
        const bool ring = a.window > 0 && a.cap == a.window;
        tma = most >= (ring ? 2 : DmShape<HDP>::NBUF_TMA == 3 ? 4 : 6) * cs * clusters;
    }
    if (tma) return launch_decode_mma<HDP, true>(a, B, stream, fq);
    return launch_decode_mma<HDP, false>(a, B, stream, fq);
}

int pick_chunk(int hd, int elem) {
    int ch = 64;
    while (ch > 8 && (size_t)2 * ch * hd * elem > 128 * 1024) ch /= 2;
    return ch;
}

size_t split_smem(int hd, int ch, int elem) {
    return (size_t)2 * ch * hd * elem + (size_t)AD_GC * hd * 4 + (size_t)AD_GC * ch * 4 +
           AD_GC * 2 * 4 + (size_t)ch * 4;
}

}  // namespace

// How the decode attention cuts a key range of at most max_keys positions:
// chunk length and number of chunks.  The scratch it needs is
// B * nh * n_splits * (hd + 2) floats, and B * nkv * ceil(nh / nkv / 4) counters.
AGV_API int agv_attention_decode_plan(int hd, int dtype, int max_keys, int* chunk,
                                      int* n_splits) {
    AGV_REQUIRE(hd > 0 && max_keys > 0, "attention_decode_plan: bad sizes");
    const int ch = pick_chunk(hd, dtype == AGV_F32 ? 4 : 2);
    *chunk = ch;
    *n_splits = (max_keys + ch - 1) / ch;
    return 0;
}

// One query token per batch entry against the paged cache (its own key is
// stored already).  q: [B, nh * hd] with row stride q_stride; out: [B, nh * hd]
// dense.  max_keys bounds the number of keys any entry sees in this launch
// (min(window, greatest length)): it sizes the grid, so it must be at least
// position - window start + 1 of every entry, else that entry's output is not written
// and its arrival counter stays non-zero; part_acc / part_ml are scratch of the sizes
// agv_attention_decode_plan implies; counters are B * nkv * ceil(nh / nkv / 4)
// ints that are zero before the call (the call leaves them zero).  A negative
// slot yields zeros.
static int attention_decode_impl(const void* q, long long q_stride, void* out, int dtype,
                                 const void* k_pool, const void* v_pool, const int* page_table,
                                 const int* slots, const int* positions, int max_pages, int page,
                                 int cap, int B, int nh, int nkv, int hd, float scale, int window,
                                 int max_keys, float* part_acc, float* part_ml, int* counters,
                                 cudaStream_t stream, const FuseQK& fq) {
    AGV_REQUIRE(B >= 0 && nh > 0 && nkv > 0 && hd > 0, "attention_decode: bad sizes");
    AGV_REQUIRE(nh % nkv == 0, "attention_decode: %d heads are not a multiple of %d kv heads", nh,
                nkv);
    const int elem = dtype == AGV_F32 ? 4 : 2;
    AGV_REQUIRE(dtype == AGV_F32 || dtype == AGV_BF16, "attention_decode: unknown dtype %d", dtype);
    AGV_REQUIRE(hd % 16 == 0 && hd <= AD_MAX_HD, "attention_decode: head_dim %d must be a multiple "
                "of 16 and at most %d", hd, AD_MAX_HD);
    AGV_REQUIRE(page > 0 && cap > 0 && max_pages > 0 && max_keys > 0,
                "attention_decode: bad cache geometry");
    AGV_REQUIRE(window >= 0 && (window == 0 || window <= cap),
                "attention_decode: window %d exceeds the ring of %d rows", window, cap);
    AGV_REQUIRE(agv_aligned(k_pool, 16) && agv_aligned(v_pool, 16),
                "attention_decode: cache pools must be 16-byte aligned");
    AGV_REQUIRE(B <= 65535, "attention_decode: batch %d exceeds the grid limit", B);
    AGV_REQUIRE(part_acc && part_ml && counters, "attention_decode: scratch pointers are null");
    if (B == 0) return 0;
    const int ch = pick_chunk(hd, elem);
    const int n_splits = (max_keys + ch - 1) / ch;
    const size_t smem = split_smem(hd, ch, elem);
    AGV_REQUIRE(smem <= (size_t)AD_MAX_SMEM, "attention_decode: %zu bytes of shared memory needed",
                smem);
    DecodeArgs a{q, q_stride, out, k_pool, v_pool, page_table, slots, positions, part_acc, part_ml,
                 counters, max_pages, page, cap, nh, nkv, hd, window, n_splits, ch, scale};
    if (dtype == AGV_BF16 && hd % 8 == 0 && hd <= 256 && ch == DM_KEYS &&
        (fq.part || (q_stride % 8 == 0 && agv_aligned(q, 16)))) {
        if (hd <= 64) return launch_decode_form<64>(a, B, stream, fq);
        if (hd <= 128) return launch_decode_form<128>(a, B, stream, fq);
        return launch_decode_form<256>(a, B, stream, fq);
    }
    AGV_REQUIRE(!fq.part, "attention_decode: the fused form needs the tensor-core kernel");
    const int G = nh / nkv;
    dim3 grid(n_splits, nkv * ((G + AD_GC - 1) / AD_GC), B);
    if (dtype == AGV_F32) {
        auto kern = attention_decode_split_kernel<float>;
        static bool configured = false;
        if (!configured) {
            AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             AD_MAX_SMEM));
            configured = true;
        }
        agv_launch(kern, grid, AD_THREADS, smem, stream, a);
    } else {
        auto kern = attention_decode_split_kernel<__nv_bfloat16>;
        static bool configured = false;
        if (!configured) {
            AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             AD_MAX_SMEM));
            configured = true;
        }
        agv_launch(kern, grid, AD_THREADS, smem, stream, a);
    }
    AGV_LAUNCH_OK("attention_decode_split_kernel");
    return 0;
}

AGV_API int agv_attention_decode(const void* q, long long q_stride, void* out, int dtype,
                                 const void* k_pool, const void* v_pool, const int* page_table,
                                 const int* slots, const int* positions, int max_pages, int page,
                                 int cap, int B, int nh, int nkv, int hd, float scale, int window,
                                 int max_keys, float* part_acc, float* part_ml, int* counters,
                                 cudaStream_t stream) {
    return attention_decode_impl(q, q_stride, out, dtype, k_pool, v_pool, page_table, slots,
                                 positions, max_pages, page, cap, B, nh, nkv, hd, scale, window,
                                 max_keys, part_acc, part_ml, counters, stream, FuseQK{});
}

// Whether agv_attention_decode_fused takes these sizes: bfloat16, head sizes 64, 128,
// 256, the whole head rotated (or none of it).
AGV_API int agv_attention_decode_fused_supported(int dtype, int hd, int rotary_dim) {
    return (dtype == AGV_BF16 && (hd == 64 || hd == 128 || hd == 256) &&
            (rotary_dim == 0 || rotary_dim == hd)) ? 1 : 0;
}

// agv_attention_decode with the q/k norm, the rotation and the cache store of the new
// position inside (see FuseQK): part [G, B, (nh + 2 nkv) * hd] are the projection's
// 32-bit partial sums; wq, wk [hd] or null; cos, sin [B, hd / 2] or null; store_kv 0
// for a layer that reads another layer's cache entry (then only q is formed here and
// the new position's key and value must be in the cache already).  The pools are
// written, so they are not const.
AGV_API int agv_attention_decode_fused(const float* part, int G, const float* wq, const float* wk,
                                       float eps, const float* cosv, const float* sinv,
                                       int store_kv, void* out, void* k_pool, void* v_pool,
                                       const int* page_table, const int* slots,
                                       const int* positions, int max_pages, int page, int cap,
                                       int B, int nh, int nkv, int hd, float scale, int window,
                                       int max_keys, float* part_acc, float* part_ml,
                                       int* counters, cudaStream_t stream) {
    AGV_REQUIRE(part && G >= 1, "attention_decode_fused: no partial sums");
    AGV_REQUIRE(agv_attention_decode_fused_supported(AGV_BF16, hd, cosv ? hd : 0),
                "attention_decode_fused: head_dim %d is not 64, 128 or 256", hd);
    AGV_REQUIRE(!cosv || sinv, "attention_decode_fused: cos without sin");
    AGV_REQUIRE(agv_aligned(part, 16), "attention_decode_fused: partial sums must be aligned");
    FuseQK fq{part, G, wq, wk, eps, cosv, sinv, store_kv};
    return attention_decode_impl(nullptr, 0, out, AGV_BF16, k_pool, v_pool, page_table, slots,
                                 positions, max_pages, page, cap, B, nh, nkv, hd, scale, window,
                                 max_keys, part_acc, part_ml, counters, stream, fq);
}

// ------------------------------------------------------- no-allocation variant
// See agave_b200_no_alloc.h.  The scratch of the split kernels sits in this
// file-scope device array.  In host code the array's name is only a stand-in:
// its device address comes from cudaGetSymbolAddress, looked up once per device.
#include "agave_b200_no_alloc.h"
#include <mutex>

static __device__ __align__(256) float g_static_scratch[AGV_NO_ALLOC_SCRATCH_FLOATS];
// Arrival counters of the split kernel: zero when the library is loaded, and every
// launch returns them to zero.
static __device__ __align__(256) int g_static_counters[AGV_NO_ALLOC_COUNTERS];

namespace {
constexpr int NO_ALLOC_MAX_DEVICES = 64;
float* g_static_scratch_addr[NO_ALLOC_MAX_DEVICES] = {};
int* g_static_counters_addr[NO_ALLOC_MAX_DEVICES] = {};
std::mutex g_static_scratch_mu;
}  // namespace

AGV_API int agv_attention_decode_static(const void* q, long long q_stride, void* out, int dtype,
                                        const void* k_pool, const void* v_pool,
                                        const int* page_table, const int* slots,
                                        const int* positions, int max_pages, int page, int cap,
                                        int B, int nh, int nkv, int hd, float scale, int window,
                                        int max_keys, cudaStream_t stream) {
    AGV_REQUIRE(B >= 0 && nh > 0 && hd > 0 && max_keys > 0, "attention_decode_static: bad sizes");
    int chunk = 0, n_splits = 0;
    if (int rc = agv_attention_decode_plan(hd, dtype, max_keys, &chunk, &n_splits)) return rc;
    const long long acc_floats = (long long)B * nh * n_splits * hd;
    const long long need = acc_floats + (long long)B * nh * n_splits * 2;
    AGV_REQUIRE(need <= (long long)AGV_NO_ALLOC_SCRATCH_FLOATS,
                "attention_decode_static: B=%d heads=%d chunks=%d head_dim=%d need %lld scratch "
                "values, the built-in array holds %d; use agv_attention_decode with your own "
                "scratch, or a smaller batch or max_keys",
                B, nh, n_splits, hd, need, (int)AGV_NO_ALLOC_SCRATCH_FLOATS);
    const int groups = nkv > 0 ? nkv * ((nh / nkv + AD_GC - 1) / AD_GC) : 0;
    AGV_REQUIRE((long long)B * groups <= (long long)AGV_NO_ALLOC_COUNTERS,
                "attention_decode_static: B=%d times %d head groups exceed the %d built-in counters",
                B, groups, (int)AGV_NO_ALLOC_COUNTERS);
    int dev = 0;
    AGV_CUDA_OK(cudaGetDevice(&dev));
    AGV_REQUIRE(dev >= 0 && dev < NO_ALLOC_MAX_DEVICES, "attention_decode_static: device %d", dev);
    float* base = nullptr;
    int* counters = nullptr;
    {
        std::lock_guard<std::mutex> g(g_static_scratch_mu);
        if (!g_static_scratch_addr[dev]) {
            float* p = nullptr;
            int* c = nullptr;
            AGV_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_static_scratch));
            AGV_CUDA_OK(cudaGetSymbolAddress((void**)&c, g_static_counters));
            g_static_scratch_addr[dev] = p;
            g_static_counters_addr[dev] = c;
        }
        base = g_static_scratch_addr[dev];
        counters = g_static_counters_addr[dev];
    }
    // The counters this call uses start from zero whatever an earlier call left: a call
    // whose max_keys was smaller than a sequence's key count never completes its count,
    // and these counters are not the caller's to clear.  (A memset allocates nothing.)
    AGV_CUDA_OK(cudaMemsetAsync(counters, 0, sizeof(int) * (size_t)B * (size_t)groups, stream));
    // partial sums first, then the (maximum, normaliser) pairs; both start 16-byte aligned
    return agv_attention_decode(q, q_stride, out, dtype, k_pool, v_pool, page_table, slots,
                                positions, max_pages, page, cap, B, nh, nkv, hd, scale, window,
                                max_keys, base, base + acc_floats, counters, stream);
}

// 0, or 1 + the tile at which a bounded wait of the TMA form for a key / value tile gave up
// first since the last call (this call synchronises the device and clears the word).
AGV_API int agv_attention_decode_status() {
    int v = 0, zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
    return v;
}

// 0: the way the tiles come is chosen from the sizes; 1: always 16-byte copies; 2: TMA
// wherever the cache's geometry allows it.  Returns the setting before.
AGV_API int agv_attention_decode_set_tiles(int form) {
    AGV_REQUIRE(form >= 0 && form <= 2, "attention_decode_set_tiles: 0, 1 or 2");
    const int before = decode_tiles_form();
    g_decode_tiles = form;
    return before;
}
