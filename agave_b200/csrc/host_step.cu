// The host side of a step in C++: one call runs a whole step of a decoder whose blocks
// are the standard arrangement (RMS norms around a softmax-attention mixer and a gated
// feed-forward), from the embedding to the logits or the chosen tokens.
//
// The Python layer describes the model once (agv_model_create, _add_rope, _add_block,
// _set_cache, _add_call: plain pointers and sizes, nothing is copied) and then hands each
// step's arrays and a workspace to agv_model_step, which makes every decision a step needs
// (which product kernel, how K is cut, which attention kernel, what scratch) and launches
// the kernels through the same exported launchers the Python layer calls one by one.  A
// step thus costs the host microseconds instead of one interpreter round trip per launch,
// which is what bounds a prompt step whose sizes were never seen (nothing recorded yet)
// and every step of the stepping interface.  Models with other parts (a mixer, feed-
// forward, norm, block or position encoding registered from outside) keep the Python path.
//
// The workspace is carved by a bump allocator; agv_model_workspace_bytes runs the same
// code without launching and reports the peak, so sizing and running cannot disagree.
// Buffers of one layer are reused by the next: kernels of a step run in stream order, and
// every kernel reads what its predecessors wrote only after its dependency wait.
//
// Reference: the per-token host loop over layers, src/models/gemma3.zig:331-368 (one
// token) and :413-442 (a prompt chunk); the launch decisions there are per-op backend
// calls (src/backend/cuda.zig).
#include "common.cuh"
#include <stdlib.h>
#include <string.h>
#include <utility>
#include <vector>

// ---- the launchers of the other files (all return 0 or a negative code)
extern "C" {
int agv_embed(const int*, const void*, int, float*, int, int, int, float, cudaStream_t);
int agv_rope_table(const int*, float*, float*, int, int, double, double, cudaStream_t);
int agv_norm_residual(float*, const void*, int, int, long long, const float*, const float*, void*,
                      int, const int*, int, int, float, float, int, cudaStream_t);
int agv_linear_simt(const void*, const void*, const void*, void*, int, int, int, long long,
                    long long, int, int, int, cudaStream_t);
int agv_linear_tc(const void*, const void*, const void*, void*, int, int, int, long long, long long,
                  int, int, int, int, int, cudaStream_t);
int agv_linear_tc_splits(int, int);
int agv_gemv_few_supported(int, int, int, long long, int);
int agv_gemv_few(const void*, const void*, int, int, int, const void*, long long, const float*, float*,
                 const float*, const float*, const float*, float, float, void*, long long, int,
                 cudaStream_t);
int agv_linear_tc_argmax(const void*, const void*, int*, int, int, int, long long, cudaStream_t);
int agv_qkv_prefill_tc_supported(int, int, int, long long, long long);
int agv_qkv_prefill_tc(const void*, const void*, int, int, long long, void*, long long, int, int,
                       int, const float*, const float*, float, const float*, const float*,
                       const int*, void*, void*, const int*, const int*, const int*, const int*,
                       int, int, int, void*, long long, const int*, cudaStream_t);
int agv_qk_norm_rope_store(void*, int, long long, const float*, int, int, int, int, int,
                           const float*, const float*, float, const float*, const float*, int,
                           const int*, void*, void*, const int*, const int*, const int*,
                           const int*, int, int, int, void*, long long, const int*, int, int,
                           cudaStream_t);
long long agv_attention_prefill_tc_vt_cols(int, int);
int agv_attention_prefill_tc(const void*, long long, const void*, const void*, long long, void*,
                             void*, long long, int, const int*, int, int, int, int, int, int, float,
                             int, cudaStream_t);
int agv_attention_prefill_mma(const void*, long long, const void*, const void*, long long, void*,
                              const int*, int, int, int, int, int, float, int, cudaStream_t);
int agv_attention_prefill_simt(const void*, long long, const void*, const void*, long long, void*,
                               int, const int*, const int*, const int*, int, int, int, int, float,
                               int, cudaStream_t);
int agv_attention_paged_simt(const void*, long long, void*, int, const void*, const void*,
                             const int*, const int*, const int*, const int*, int, int, int, int, int,
                             int, int, float, int, cudaStream_t);
int agv_attention_decode_plan(int, int, int, int*, int*);
int agv_attention_decode(const void*, long long, void*, int, const void*, const void*, const int*,
                         const int*, const int*, int, int, int, int, int, int, int, float, int, int,
                         float*, float*, int*, cudaStream_t);
int agv_attention_decode_fused_supported(int, int, int);
int agv_attention_decode_fused(const float*, int, const float*, const float*, float, const float*,
                               const float*, int, void*, void*, void*, const int*, const int*,
                               const int*, int, int, int, int, int, int, int, float, int, int,
                               float*, float*, int*, cudaStream_t);
}

// What the Python layer fills in (ctypes structures with the same fields, in this order).
struct AgvBlockDesc {
    const float* w_pre_mixer;      // norm weights, 32-bit, 1 + w already formed; null: no such norm
    const float* w_post_mixer;
    const float* w_pre_ffn;
    const float* w_post_ffn;
    const void* w_qkv;             // [(nh + 2 nkv) * hd, H], rows q | k | v
    const void* w_out;             // [H, nh * hd]
    const float* wq_norm;          // [hd] or null
    const float* wk_norm;
    const void* w_gate;            // [ff, H]
    const void* w_up;
    const void* w_down;            // [H, ff]
    float eps, qk_eps, scale;
    int nh, nkv, hd, window, rotary_dim, rope_slot, ff, act;
};

struct AgvCacheDesc {
    void* k_pool;
    void* v_pool;
    const int* page_table;
    int max_pages, page, cap, pool_pages;
};

struct AgvStepDesc {
    const int* tokens;
    const int* positions;
    const int* seq_index;
    const int* cu_seqlens;
    const int* slots;
    const int* lens;
    void* workspace;
    const int* rows;               // stream rows whose logits (or choices) are wanted
    float* logits;                 // [n_rows, V] 32-bit, or null
    int* argmax_out;               // [n_rows], or null: the greatest logit's index instead
    int* decode_counters;          // zeroed ints for the split decode attention
    long long workspace_bytes;
    int mode;                      // 0: whole prompts from position 0; 1: one token each
    int T, B, max_len, max_new, n_rows;
};

namespace {

struct Rope { double theta, factor; int rotary_dim; };

struct Model {
    int dtype, H, V;
    float embed_scale, final_eps;
    const void* embed;
    const float* final_w;
    const void* head_w;
    std::vector<AgvBlockDesc> blocks;
    std::vector<Rope> ropes;
    std::vector<AgvCacheDesc> caches;
    std::vector<int> call_block, call_cache;
};

// a prompt step of at most this many tokens runs the mma.sync attention (a short prompt gives
// the tcgen05 kernel, 128 query rows a CTA, a handful of CTAs with a long set-up each)
constexpr int PREFILL_TC_MIN_TOKENS = 192;

struct Arena {
    char* base;
    size_t cap, top = 0, peak = 0;
    bool dry, overflow = false;
    void* take(size_t bytes) {
        top = (top + 255) & ~(size_t)255;
        void* p = base + top;
        top += bytes;
        if (top > peak) peak = top;
        if (!dry && top > cap) overflow = true;
        return p;
    }
};

struct Partial {
    void* ptr;
    int groups;       // > 0: 32-bit partial sums [groups, T, N]; 0: [T, N] in the compute dtype
};

bool env_on(const char* name, bool dflt) {
    const char* v = getenv(name);
    return v ? v[0] != '0' : dflt;
}

struct Run {
    const Model& m;
    const AgvStepDesc& s;
    Arena& ar;
    cudaStream_t stream;
    int sms;
    int launches = 0;
    int rc = 0;
    int esz() const { return m.dtype == AGV_F32 ? 4 : 2; }
    bool dry() const { return ar.dry; }
    void did(int r) {
        ++launches;
        if (r && !rc) rc = r;
    }
    bool tc_ok(const void* x, long long lda, const void* w, int K) const {
        return m.dtype == AGV_BF16 && K % 8 == 0 && lda % 8 == 0 && agv_aligned(x, 16) &&
               agv_aligned(w, 16);
    }

    // (groups, cluster size) of the ranges K is cut into: about one CTA per SM when the
    // weight has few row tiles; the CTAs of a cluster add in the kernel, the groups are left
    // to the consumer; prompts are cut in two only over a long K with few tiles
    void plan_splits(int T, int N, int K, bool cheap, int* groups, int* csize) const {
        *groups = 1;
        *csize = 0;
        if (T > 64) {
            const int tile = T <= 128 ? 128 : 256;
            const long long ctas = (long long)((N + 127) / 128) * ((T + tile - 1) / tile);
            const int kb = (K + 63) / 64;
            if (T <= 512) {
                // short prompts: one or two token tiles, so a narrow weight is cut into
                // ranges of K whose partial sums the consumer adds
                const int most = T <= 128 ? 16 : T <= 256 ? 8 : 4;
                long long want = kb / 2;
                if (sms / ctas < want) want = sms / ctas;
                if (most < want) want = most;
                if (want >= 2) *groups = agv_linear_tc_splits(K, (int)want);
                return;
            }
            if (ctas <= sms / 2 + 6 && kb >= 32) *groups = 2;
            return;
        }
        const int tile = T <= 16 ? 16 : T <= 32 ? 32 : 64;
        const long long ctas = (long long)((N + 127) / 128) * ((T + tile - 1) / tile);
        const int kb = (K + 63) / 64;
        const long long per = (sms + ctas - 1) / ctas;
        const int want = (int)(kb < per ? kb : per);
        if (ctas >= 100 || want < 2) return;
        if (T > 16) {
            *groups = agv_linear_tc_splits(K, want < 16 ? want : 16);
        } else if (cheap) {
            *groups = agv_linear_tc_splits(K, want < 8 ? want : 8);
        } else if (want <= 8 || kb < 64) {
            *csize = want < 8 ? want : 8;
        } else {
            *groups = agv_linear_tc_splits(K, want < 16 ? want : 16);
        }
    }

    Partial linear_partial(const void* x, long long lda, const void* w, int N, int K, int T,
                           bool cheap) {
        if (tc_ok(x, lda, w, K)) {
            int groups, c;
            plan_splits(T, N, K, cheap, &groups, &c);
            void* out = ar.take((size_t)groups * T * N * 4);
            if (!dry())
                did(agv_linear_tc(x, w, nullptr, out, T, N, K, lda, N, AGV_F32, 0,
                                  groups * (c > 1 ? c : 1), c, 0, stream));
            return {out, groups};
        }
        void* out = ar.take((size_t)T * N * esz());
        if (!dry())
            did(agv_linear_simt(x, w, nullptr, out, T, N, K, lda, N, m.dtype, m.dtype, 0, stream));
        return {out, 0};
    }

    // h += post(y) (or y); x_out = next(h) if w_next
    void join(float* h, const Partial& y, const float* w_post, float eps_post, const float* w_next,
              float eps_next, void* x_out) {
        if (dry()) return;
        did(agv_norm_residual(h, y.ptr, y.groups ? AGV_F32 : m.dtype, y.groups ? y.groups : 1,
                              y.groups ? (long long)s.T * m.H : 0, w_post, w_next,
                              w_next ? x_out : nullptr, m.dtype, nullptr, s.T, m.H,
                              w_post ? eps_post : 0.f, w_next ? eps_next : 0.f, 1, stream));
    }

    Partial attend_prompt(const AgvBlockDesc& b, void* qkv, void* vt, long long vt_cols) {
        const int e = esz(), T = s.T;
        const long long width = (long long)(b.nh + 2 * b.nkv) * b.hd;
        char* q = (char*)qkv;
        char* k = q + (size_t)b.nh * b.hd * e;
        char* v = q + (size_t)(b.nh + b.nkv) * b.hd * e;
        void* out = ar.take((size_t)T * b.nh * b.hd * e);
        const bool aligned = m.dtype == AGV_BF16 && b.hd <= 256 && width % 8 == 0 &&
                             agv_aligned(q, 16) && agv_aligned(k, 16) && agv_aligned(v, 16);
        static const bool prefill_tc = [] {
            const char* v2 = getenv("AGAVE_B200_PREFILL_ATTENTION");
            return !(v2 && strcmp(v2, "mma") == 0);
        }();
        if (!dry()) {
            if (aligned && b.hd % 16 == 0 && prefill_tc && T > PREFILL_TC_MIN_TOKENS)
                did(agv_attention_prefill_tc(q, width, k, v, width, out, vt, vt_cols, 1, s.cu_seqlens,
                                             s.B, T, s.max_new, b.nh, b.nkv, b.hd, b.scale,
                                             b.window, stream));
            else if (aligned && b.hd % 8 == 0)
                did(agv_attention_prefill_mma(q, width, k, v, width, out, s.cu_seqlens, s.B,
                                              s.max_new, b.nh, b.nkv, b.hd, b.scale, b.window,
                                              stream));
            else
                did(agv_attention_prefill_simt(q, width, k, v, width, out, m.dtype, s.positions,
                                               s.seq_index, s.cu_seqlens, T, b.nh, b.nkv, b.hd,
                                               b.scale, b.window, stream));
        }
        return linear_partial(out, (long long)b.nh * b.hd, b.w_out, m.H, b.nh * b.hd, T, false);
    }

    // whether a prompt step's attention will read the values transposed (the tcgen05 kernel)
    bool wants_vt(const AgvBlockDesc& b, const void* qkv) const {
        static const bool prefill_tc = [] {
            const char* v2 = getenv("AGAVE_B200_PREFILL_ATTENTION");
            return !(v2 && strcmp(v2, "mma") == 0);
        }();
        const long long width = (long long)(b.nh + 2 * b.nkv) * b.hd;
        return prefill_tc && s.T > PREFILL_TC_MIN_TOKENS && m.dtype == AGV_BF16 && b.hd % 16 == 0 &&
               b.hd <= 256 &&
               width % 8 == 0 && agv_aligned(qkv, 16);
    }

    Partial mixer(const AgvBlockDesc& b, const AgvCacheDesc& c, const void* x,
                  float* const* cosv, float* const* sinv) {
        const int e = esz(), T = s.T, H = m.H;
        const int width = (b.nh + 2 * b.nkv) * b.hd;
        const float* cs = b.rope_slot >= 0 ? cosv[b.rope_slot] : nullptr;
        const float* sn = b.rope_slot >= 0 ? sinv[b.rope_slot] : nullptr;
        const int rotary_dim = b.rope_slot >= 0 ? b.rotary_dim : 0;
        static const int fused_qkv = [] {
            const char* v = getenv("AGAVE_B200_FUSED_QKV_PREFILL");
            return v ? atoi(v) : 1;
        }();
        if (s.mode == 0 && fused_qkv != 0 && T > 128 && tc_ok(x, H, b.w_qkv, H)) {
            const long long tiles = (long long)((width + 255) / 256) * ((T + 127) / 128);
            if ((tiles * 2 >= 3LL * sms || fused_qkv == 2) &&
                agv_qkv_prefill_tc_supported(b.hd, rotary_dim, H, H, width)) {
                // norm, rotation, the cache store and the transposed values are the epilogue
                // of the q/k/v product
                void* qkv = ar.take((size_t)T * width * e);
                void* vt = nullptr;
                long long vt_cols = 0;
                if (wants_vt(b, qkv)) {
                    vt_cols = agv_attention_prefill_tc_vt_cols(T, s.B);
                    vt = ar.take((size_t)b.nkv * b.hd * vt_cols * 2);
                }
                if (!dry())
                    did(agv_qkv_prefill_tc(x, b.w_qkv, T, H, H, qkv, width, b.nh, b.nkv, b.hd,
                                           b.wq_norm, b.wk_norm, b.qk_eps, cs, sn, s.positions,
                                           c.k_pool, c.v_pool, c.page_table, s.slots, s.lens,
                                           s.seq_index, c.max_pages, c.page, c.cap, vt, vt_cols,
                                           s.cu_seqlens, stream));
                return attend_prompt(b, qkv, vt, vt_cols);
            }
        }
        Partial proj = linear_partial(x, H, b.w_qkv, width, H, T, true);
        static const bool fused_decode = env_on("AGAVE_B200_FUSED_DECODE_ATTENTION", true);
        const int max_keys_raw = b.window ? (b.window < s.max_len ? b.window : s.max_len) : s.max_len;
        const int max_keys = max_keys_raw > 1 ? max_keys_raw : 1;
        if (s.mode == 1 && proj.groups > 0 && fused_decode && m.dtype == AGV_BF16 &&
            agv_attention_decode_fused_supported(AGV_BF16, b.hd, rotary_dim)) {
            // decoding: norm, rotation and the store of the new key and value happen inside
            // the attention kernel, on the projection's partial sums
            void* out = ar.take((size_t)T * b.nh * b.hd * e);
            int chunk = 0, n_splits = 0;
            agv_attention_decode_plan(b.hd, AGV_BF16, max_keys, &chunk, &n_splits);
            if (n_splits > 16) n_splits = 16;
            float* acc = (float*)ar.take((size_t)s.B * b.nh * n_splits * b.hd * 4);
            float* ml = (float*)ar.take((size_t)s.B * b.nh * n_splits * 2 * 4);
            if (!dry())
                did(agv_attention_decode_fused((const float*)proj.ptr, proj.groups, b.wq_norm,
                                               b.wk_norm, b.qk_eps, cs, sn, 1, out, c.k_pool,
                                               c.v_pool, c.page_table, s.slots, s.positions,
                                               c.max_pages, c.page, c.cap, s.B, b.nh, b.nkv, b.hd,
                                               b.scale, b.window, max_keys, acc, ml,
                                               s.decode_counters, stream));
            return linear_partial(out, (long long)b.nh * b.hd, b.w_out, H, b.nh * b.hd, T, false);
        }
        void* qkv = proj.groups == 0 ? proj.ptr : ar.take((size_t)T * width * e);
        void* vt = nullptr;
        long long vt_cols = 0;
        if (s.mode == 0 && wants_vt(b, qkv)) {
            vt_cols = agv_attention_prefill_tc_vt_cols(T, s.B);
            vt = ar.take((size_t)b.nkv * b.hd * vt_cols * 2);
        }
        if (!dry())
            did(agv_qk_norm_rope_store(qkv, m.dtype, width,
                                       proj.groups ? (const float*)proj.ptr : nullptr, proj.groups,
                                       T, b.nh, b.nkv, b.hd, b.wq_norm, b.wk_norm, b.qk_eps, cs, sn,
                                       rotary_dim, s.positions, c.k_pool, c.v_pool, c.page_table,
                                       s.slots, s.lens, s.seq_index, c.max_pages, c.page, c.cap, vt,
                                       vt_cols, s.cu_seqlens, vt ? s.B : 0, s.max_new, stream));
        if (s.mode == 0) return attend_prompt(b, qkv, vt, vt_cols);
        void* out = ar.take((size_t)T * b.nh * b.hd * e);
        if (b.hd % 16 == 0 && b.hd <= 512) {
            int chunk = 0, n_splits = 0;
            agv_attention_decode_plan(b.hd, m.dtype, max_keys, &chunk, &n_splits);
            float* acc = (float*)ar.take((size_t)s.B * b.nh * n_splits * b.hd * 4);
            float* ml = (float*)ar.take((size_t)s.B * b.nh * n_splits * 2 * 4);
            if (!dry())
                did(agv_attention_decode(qkv, width, out, m.dtype, c.k_pool, c.v_pool, c.page_table,
                                         s.slots, s.positions, c.max_pages, c.page, c.cap, s.B,
                                         b.nh, b.nkv, b.hd, b.scale, b.window, max_keys, acc, ml,
                                         s.decode_counters, stream));
        } else if (!dry()) {
            did(agv_attention_paged_simt(qkv, width, out, m.dtype, c.k_pool, c.v_pool, c.page_table,
                                         s.slots, s.positions, s.seq_index, c.max_pages, c.page,
                                         c.cap, T, b.nh, b.nkv, b.hd, b.scale, b.window, stream));
        }
        return linear_partial(out, (long long)b.nh * b.hd, b.w_out, H, b.nh * b.hd, T, false);
    }

    Partial feed_forward(const AgvBlockDesc& b, const void* x) {
        const int T = s.T, H = m.H;
        void* z = ar.take((size_t)T * b.ff * esz());
        if (!dry()) {
            if (tc_ok(x, H, b.w_gate, H)) {
                int c = 0;
                if (T <= 64) {
                    // decoding through a gated layer with few 64-feature tiles: two or four
                    // CTAs per tile, each on a range of K, joined by a cluster
                    const int tiles = (b.ff + 63) / 64, kb = (H + 63) / 64;
                    c = (tiles * 4 <= sms && kb >= 8) ? 4 : (tiles * 2 <= 2 * sms && kb >= 4) ? 2 : 0;
                }
                did(agv_linear_tc(x, b.w_gate, b.w_up, z, T, b.ff, H, H, b.ff, AGV_BF16, b.act,
                                  c > 1 ? c : 1, c, 0, stream));
            } else {
                did(agv_linear_simt(x, b.w_gate, b.w_up, z, T, b.ff, H, H, b.ff, m.dtype, m.dtype,
                                    b.act, stream));
            }
        }
        return linear_partial(z, b.ff, b.w_down, H, b.ff, T, false);
    }

    // Whether a decode step of this few tokens runs as dot products with the joins in the
    // projections' prologues (gemv_few.cu): five kernels a layer instead of seven.
    bool few_tokens() const {
        static const int most = [] {
            const char* v = getenv("AGAVE_B200_FEW_TOKENS");
            return v ? atoi(v) : 2;
        }();
        static const bool fused_decode = env_on("AGAVE_B200_FUSED_DECODE_ATTENTION", true);
        if (s.mode != 1 || s.T > most || s.T < 1 || m.dtype != AGV_BF16 || !fused_decode) return false;
        for (int ci : m.call_block) {
            const AgvBlockDesc& b = m.blocks[ci];
            const int width = (b.nh + 2 * b.nkv) * b.hd;
            const int rotary_dim = b.rope_slot >= 0 ? b.rotary_dim : 0;
            if (!b.w_pre_mixer || !b.w_pre_ffn) return false;
            // (a layer of more than 96 MB is bound by how fast its weights stream, and there
            // the tensor-core products, fed by TMA, are ahead: measured at the 4B and 27B sizes)
            const long long weights = 2LL * ((long long)width * m.H + (long long)m.H * b.nh * b.hd +
                                             3LL * b.ff * m.H);
            if (weights > 96LL * 1024 * 1024) return false;
            if (!agv_attention_decode_fused_supported(AGV_BF16, b.hd, rotary_dim)) return false;
            if (!agv_gemv_few_supported(s.T, width, m.H, 8, 1) ||
                !agv_gemv_few_supported(s.T, m.H, b.nh * b.hd, b.nh * b.hd, 0) ||
                !agv_gemv_few_supported(s.T, b.ff, m.H, 8, 1) ||
                !agv_gemv_few_supported(s.T, m.H, b.ff, b.ff, 0))
                return false;
        }
        return !m.call_block.empty();
    }

    // The blocks of such a step.  The stream alternates between two buffers, because the
    // CTAs of a projection all read it while one of them writes the joined stream.  Returns
    // the buffer that holds the stream after the last block.
    float* few_blocks(float* h, float* const* cosv, float* const* sinv) {
        const int T = s.T, H = m.H;
        const int n_calls = (int)m.call_block.size();
        float* cur = h;
        float* other = (float*)ar.take((size_t)T * H * 4);
        float* y_down = (float*)ar.take((size_t)T * H * 4);
        const float* pend_y = nullptr;           // the branch the next join adds
        const float* pend_w = nullptr;
        float pend_eps = 0.f;
        const size_t mark = ar.top;
        for (int ci = 0; ci < n_calls; ++ci) {
            ar.top = mark;
            const AgvBlockDesc& b = m.blocks[m.call_block[ci]];
            const AgvCacheDesc& c = m.caches[m.call_cache[ci]];
            const int width = (b.nh + 2 * b.nkv) * b.hd;
            const float* cs = b.rope_slot >= 0 ? cosv[b.rope_slot] : nullptr;
            const float* sn = b.rope_slot >= 0 ? sinv[b.rope_slot] : nullptr;
            float* qkv = (float*)ar.take((size_t)T * width * 4);
            void* att = ar.take((size_t)T * b.nh * b.hd * 2);
            float* y_out = (float*)ar.take((size_t)T * H * 4);
            void* z = ar.take((size_t)T * b.ff * 2);
            const int max_keys_raw = b.window ? (b.window < s.max_len ? b.window : s.max_len) : s.max_len;
            const int max_keys = max_keys_raw > 1 ? max_keys_raw : 1;
            int chunk = 0, n_splits = 0;
            agv_attention_decode_plan(b.hd, AGV_BF16, max_keys, &chunk, &n_splits);
            if (n_splits > 16) n_splits = 16;
            float* acc = (float*)ar.take((size_t)s.B * b.nh * n_splits * b.hd * 4);
            float* ml = (float*)ar.take((size_t)s.B * b.nh * n_splits * 2 * 4);
            if (dry()) continue;
            // q/k/v of the stream joined with the block before (or the stream as embedded)
            did(agv_gemv_few(b.w_qkv, nullptr, width, H, T, nullptr, 0, cur, pend_y ? other : nullptr,
                             pend_y, pend_w, b.w_pre_mixer, pend_eps, b.eps, qkv, width, 0, stream));
            if (pend_y) std::swap(cur, other);
            did(agv_attention_decode_fused(qkv, 1, b.wq_norm, b.wk_norm, b.qk_eps, cs, sn, 1, att,
                                           c.k_pool, c.v_pool, c.page_table, s.slots, s.positions,
                                           c.max_pages, c.page, c.cap, s.B, b.nh, b.nkv, b.hd, b.scale,
                                           b.window, max_keys, acc, ml, s.decode_counters, stream));
            did(agv_gemv_few(b.w_out, nullptr, H, b.nh * b.hd, T, att, (long long)b.nh * b.hd, nullptr,
                             nullptr, nullptr, nullptr, nullptr, 0.f, 0.f, y_out, H, 0, stream));
            did(agv_gemv_few(b.w_gate, b.w_up, b.ff, H, T, nullptr, 0, cur, other, y_out,
                             b.w_post_mixer, b.w_pre_ffn, b.eps, b.eps, z, b.ff, b.act, stream));
            std::swap(cur, other);
            did(agv_gemv_few(b.w_down, nullptr, H, b.ff, T, z, b.ff, nullptr, nullptr, nullptr, nullptr,
                             nullptr, 0.f, 0.f, y_down, H, 0, stream));
            pend_y = y_down;
            pend_w = b.w_post_ffn;
            pend_eps = b.eps;
        }
        ar.top = mark;
        if (!dry() && pend_y)                    // the last block's branch joins the stream
            did(agv_norm_residual(cur, pend_y, AGV_F32, 1, 0, pend_w, nullptr, nullptr, m.dtype, nullptr,
                                  T, H, pend_w ? pend_eps : 0.f, 0.f, 1, stream));
        return cur;
    }

    int step() {
        const int T = s.T, H = m.H, e = esz();
        const int n_calls = (int)m.call_block.size();
        float* h = (float*)ar.take((size_t)T * H * 4);
        void* xa = ar.take((size_t)T * H * e);
        void* xb = ar.take((size_t)T * H * e);
        // the rotation tables of the step, one pair per distinct (base, factor, width)
        std::vector<float*> cosv(m.ropes.size(), nullptr), sinv(m.ropes.size(), nullptr);
        if (!dry()) did(agv_embed(s.tokens, m.embed, m.dtype, h, T, H, m.V, m.embed_scale, stream));
        for (int ci = 0; ci < n_calls; ++ci) {
            const int slot = m.blocks[m.call_block[ci]].rope_slot;
            if (slot >= 0 && !cosv[slot]) {
                const Rope& r = m.ropes[slot];
                cosv[slot] = (float*)ar.take((size_t)T * (r.rotary_dim / 2) * 4);
                sinv[slot] = (float*)ar.take((size_t)T * (r.rotary_dim / 2) * 4);
                if (!dry())
                    did(agv_rope_table(s.positions, cosv[slot], sinv[slot], T, r.rotary_dim, r.theta,
                                       r.factor, stream));
            }
        }
        const bool few = few_tokens();
        if (few) h = few_blocks(h, cosv.data(), sinv.data());
        if (!few && n_calls > 0 && !dry()) {
            const AgvBlockDesc& b0 = m.blocks[m.call_block[0]];
            did(agv_norm_residual(h, nullptr, AGV_F32, 1, 0, nullptr, b0.w_pre_mixer, xa, m.dtype,
                                  nullptr, T, H, 0.f, b0.eps, 0, stream));
        }
        const size_t mark = ar.top;
        for (int ci = 0; !few && ci < n_calls; ++ci) {
            ar.top = mark;                    // a layer's buffers are reused by the next
            const AgvBlockDesc& b = m.blocks[m.call_block[ci]];
            const AgvCacheDesc& c = m.caches[m.call_cache[ci]];
            const AgvBlockDesc* nb = ci + 1 < n_calls ? &m.blocks[m.call_block[ci + 1]] : nullptr;
            Partial y = mixer(b, c, xa, cosv.data(), sinv.data());
            join(h, y, b.w_post_mixer, b.eps, b.w_pre_ffn, b.eps, xb);
            Partial d = feed_forward(b, xb);
            join(h, d, b.w_post_ffn, b.eps, nb ? nb->w_pre_mixer : nullptr, nb ? nb->eps : 0.f, xa);
        }
        ar.top = mark;
        if (s.n_rows > 0) {
            void* xn = ar.take((size_t)s.n_rows * H * e);
            if (!dry()) {
                did(agv_norm_residual(h, nullptr, AGV_F32, 1, 0, nullptr, m.final_w, xn, m.dtype,
                                      s.rows, s.n_rows, H, 0.f, m.final_eps, 0, stream));
                if (s.argmax_out) {
                    did(agv_linear_tc_argmax(xn, m.head_w, s.argmax_out, s.n_rows, m.V, H, H, stream));
                    ++launches;               // the product and the kernel that reads its keys out
                } else if (tc_ok(xn, H, m.head_w, H)) {
                    did(agv_linear_tc(xn, m.head_w, nullptr, s.logits, s.n_rows, m.V, H, H, m.V,
                                      AGV_F32, 0, 1, 0, 0, stream));
                } else {
                    did(agv_linear_simt(xn, m.head_w, nullptr, s.logits, s.n_rows, m.V, H, H, m.V,
                                        m.dtype, AGV_F32, 0, stream));
                }
            }
        }
        return rc;
    }
};

int device_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sms = 148;
    }
    return sms;
}

int check_step(const Model& m, const AgvStepDesc& s) {
    AGV_REQUIRE(s.T > 0 && s.B > 0 && s.n_rows >= 0, "model_step: bad sizes T=%d B=%d", s.T, s.B);
    AGV_REQUIRE(s.mode == 0 || (s.mode == 1 && s.T == s.B),
                "model_step: a decode step brings one token per sequence");
    AGV_REQUIRE(!(s.logits && s.argmax_out), "model_step: logits or choices, not both");
    AGV_REQUIRE(s.n_rows == 0 || s.logits || s.argmax_out, "model_step: no place for the results");
    AGV_REQUIRE(!s.argmax_out || (m.dtype == AGV_BF16 && s.n_rows <= 128 && m.H % 8 == 0),
                "model_step: the arg max epilogue takes bfloat16 and at most 128 rows");
    for (size_t i = 0; i < m.call_cache.size(); ++i)
        AGV_REQUIRE(m.call_cache[i] >= 0 && (size_t)m.call_cache[i] < m.caches.size() &&
                        m.caches[m.call_cache[i]].k_pool,
                    "model_step: call %d has no cache entry", (int)i);
    return 0;
}

}  // namespace

// A model whose blocks are the standard arrangement.  dtype: the compute dtype (AgvDtype);
// embed [V, H] and head_w [V, H] in it (head_w may be embed); final_w [H] 32-bit.  The
// handle is a pointer; nothing it points to is copied, so the tensors must outlive it.
AGV_API void* agv_model_create(int dtype, int H, int V, float embed_scale, const void* embed,
                               const float* final_w, float final_eps, const void* head_w) {
    if ((dtype != AGV_F32 && dtype != AGV_BF16) || H <= 0 || V <= 0 || !embed || !final_w || !head_w) {
        agv_fail(-1, "model_create: bad arguments");
        return nullptr;
    }
    Model* m = new Model();
    m->dtype = dtype, m->H = H, m->V = V;
    m->embed_scale = embed_scale, m->final_eps = final_eps;
    m->embed = embed, m->final_w = final_w, m->head_w = head_w;
    return m;
}

AGV_API void agv_model_destroy(void* handle) { delete (Model*)handle; }

// A rotation table kind; returns its slot (blocks name it in rope_slot).
AGV_API int agv_model_add_rope(void* handle, double theta, double factor, int rotary_dim) {
    Model* m = (Model*)handle;
    AGV_REQUIRE(m && theta > 0 && factor > 0 && rotary_dim > 0 && rotary_dim % 2 == 0,
                "model_add_rope: bad arguments");
    m->ropes.push_back({theta, factor, rotary_dim});
    return (int)m->ropes.size() - 1;
}

AGV_API int agv_model_add_block(void* handle, const AgvBlockDesc* b) {
    Model* m = (Model*)handle;
    AGV_REQUIRE(m && b, "model_add_block: null");
    AGV_REQUIRE(b->w_pre_mixer && b->w_pre_ffn && b->w_qkv && b->w_out && b->w_gate && b->w_up &&
                    b->w_down, "model_add_block: a weight is missing");
    AGV_REQUIRE(b->nh > 0 && b->nkv > 0 && b->nh % b->nkv == 0 && b->hd > 0 && b->ff > 0,
                "model_add_block: bad sizes");
    AGV_REQUIRE(b->rope_slot < (int)m->ropes.size(), "model_add_block: unknown rope slot %d",
                b->rope_slot);
    m->blocks.push_back(*b);
    return (int)m->blocks.size() - 1;
}

AGV_API int agv_model_set_cache(void* handle, int entry, const AgvCacheDesc* c) {
    Model* m = (Model*)handle;
    AGV_REQUIRE(m && c && entry >= 0 && entry < 65536, "model_set_cache: bad arguments");
    if ((size_t)entry >= m->caches.size()) m->caches.resize(entry + 1, AgvCacheDesc{});
    m->caches[entry] = *c;
    return 0;
}

// The run order: call after call, which block runs on which cache entry (each call writes
// its entry).
AGV_API int agv_model_add_call(void* handle, int block, int cache) {
    Model* m = (Model*)handle;
    AGV_REQUIRE(m && block >= 0 && (size_t)block < m->blocks.size() && cache >= 0,
                "model_add_call: unknown block %d", block);
    m->call_block.push_back(block);
    m->call_cache.push_back(cache);
    return 0;
}

// Bytes of workspace agv_model_step needs for a step of these sizes (max_len and max_new as
// in the step).  Negative: an error.
AGV_API long long agv_model_workspace_bytes(void* handle, int mode, int T, int B, int max_len,
                                            int max_new, int n_rows, int want_argmax) {
    Model* m = (Model*)handle;
    if (!m || T <= 0 || B <= 0) return agv_fail(-1, "model_workspace_bytes: bad arguments");
    AgvStepDesc s{};
    s.mode = mode, s.T = T, s.B = B, s.max_len = max_len, s.max_new = max_new, s.n_rows = n_rows;
    s.argmax_out = want_argmax ? (int*)256 : nullptr;
    Arena ar{(char*)4096, 0};
    ar.dry = true;
    Run run{*m, s, ar, nullptr, device_sms()};
    run.step();
    return (long long)ar.peak + 256;
}

// One step: every kernel from the embedding to the logits (or the chosen tokens) is
// launched on `stream`.  n_launches receives the number of launcher calls made.
AGV_API int agv_model_step(void* handle, const AgvStepDesc* s, int* n_launches, cudaStream_t stream) {
    Model* m = (Model*)handle;
    AGV_REQUIRE(m && s && s->workspace, "model_step: null");
    if (int rc = check_step(*m, *s)) return rc;
    char* base = (char*)(((uintptr_t)s->workspace + 255) & ~(uintptr_t)255);
    const size_t lost = (size_t)(base - (char*)s->workspace);
    AGV_REQUIRE((size_t)s->workspace_bytes > lost, "model_step: the workspace is too small");
    Arena ar{base, (size_t)s->workspace_bytes - lost};
    ar.dry = false;
    // sizes first, without launching: a workspace that is too small must not be half used
    {
        Arena probe{(char*)4096, 0};
        probe.dry = true;
        Run dry_run{*m, *s, probe, nullptr, device_sms()};
        dry_run.step();
        AGV_REQUIRE(probe.peak <= ar.cap, "model_step: the step needs %zu bytes of workspace, %zu given",
                    probe.peak, ar.cap);
    }
    Run run{*m, *s, ar, stream, device_sms()};
    const int rc = run.step();
    if (n_launches) *n_launches = run.launches;
    return rc;
}
