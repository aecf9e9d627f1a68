// Attention with a sliding window that keeps the sequence's first tokens, key and value heads
// of different sizes, and softmax weights that are mixed between the heads.
//
// Three kernels:
//  * qkv_prepare: per token, adds the projections' biases, turns the queries and keys by the
//    step's rotation table, divides each head by its root mean square (optional), writes the
//    queries to their buffer and the keys and values into the paged cache.  Values can be mixed
//    with the values an earlier layer made for the same token: v <- (1 - l) v + l v_first.
//  * attention_sink: one block per (token, query head).  Query at position p sees key s if
//    s <= p and (p - s < window or s < keep_first); window 0 means every earlier key.  Softmax
//    in float32 with a running maximum.  With all_values the weights of a head are applied to
//    the values of EVERY key/value head (the mixing of weights between heads needs them), else
//    to the head's own.  The results are float32.
//  * head_mix: out[t, h] = sum_g mix[h, g] * partial[t, g, kv(h)]: a mix of the heads' softmax
//    weights, applied to the values, is the same mix of their weighted value sums.
#include "api.h"
#include "common.cuh"
#include "mma.cuh"

#define QP_THREADS 128
#define QP_MAX_HD 512

// blocks (token, slot): slots 0..nh-1 query heads, nh..nh+nkv-1 key heads, then nkv value heads
template <typename TP, typename TQ, typename TC>
__global__ void __launch_bounds__(QP_THREADS)
qkv_prepare_kernel(const TP* __restrict__ proj, long long ldp, const float* __restrict__ bias, const float2* __restrict__ table,
                   int rot, int nh, int nkv, int hd, int vd, int unit_norm, const float* __restrict__ q_norm_w,
                   const float* __restrict__ k_norm_w, float eps, TQ* __restrict__ q_out, long long ldq,
                   TC* __restrict__ k_cache, TC* __restrict__ v_cache, const int* __restrict__ page_table, int pt_width,
                   const int* __restrict__ tok_seq, const int* __restrict__ positions, int n_pages, int append,
                   const float* __restrict__ v_lambda, float* __restrict__ v_first, int v_mode, int interleaved, int v_from_k,
                   int* status) {
    pdl_trigger();
    __shared__ float xs[QP_MAX_HD];
    __shared__ float scratch[33];
    const int t = blockIdx.x, slot = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    const bool is_q = slot < nh, is_k = !is_q && slot < nh + nkv;
    int page = -1;
    if (!is_q) {
        const int lp = pos / HB_PAGE_TOKENS;
        page = lp < pt_width ? page_table[(size_t)tok_seq[t] * pt_width + lp] : -1;
        if (page < 0 || page >= n_pages) {
            if (append && tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + tok_seq[t]);
            page = -1;
        }
    }
    pdl_wait();
    proj = pdl_fresh(proj);
    table = pdl_fresh(table);
    if (is_q || is_k) {
        const int col0 = is_q ? slot * hd : nh * hd + (slot - nh) * hd;
        const TP* row = proj + (size_t)t * ldp + col0;
        for (int d = tid; d < hd; d += QP_THREADS) xs[d] = to_f32(row[d]) + (bias ? bias[col0 + d] : 0.0f);
        __syncthreads();
        if (unit_norm == 2) {
            // the head divided by its root mean square and multiplied by a weight BEFORE the rotation
            const float* nw = is_q ? q_norm_w : k_norm_w;
            float s0 = 0.0f;
            for (int d = tid; d < hd; d += QP_THREADS) s0 = fmaf(xs[d], xs[d], s0);
            s0 = block_sum(s0, scratch);
            const float inv0 = 1.0f / sqrtf(s0 / (float)hd + eps);
            for (int d = tid; d < hd; d += QP_THREADS) xs[d] = xs[d] * inv0 * nw[d];
            __syncthreads();
        }
        const int half = rot >> 1;
        float ss = 0.0f;
        for (int d = tid; d < hd; d += QP_THREADS) {
            float y = xs[d];
            if (d < rot) {
                // pair i is (i, i + rot/2), or with `interleaved` (2i, 2i + 1)
                const int i = interleaved ? d >> 1 : (d < half ? d : d - half);
                const float2 cs = table[(size_t)t * half + i];
                float y1, y2;
                rope_pair(xs[interleaved ? 2 * i : i], xs[interleaved ? 2 * i + 1 : i + half], cs.x, cs.y, y1, y2);
                y = (interleaved ? (d & 1) == 0 : d < half) ? y1 : y2;
            }
            ss = fmaf(y, y, ss);
        }
        // second pass with the factor (recomputes the rotation: xs still holds the inputs)
        float inv = 1.0f;
        if (unit_norm == 1) {
            ss = block_sum(ss, scratch);
            inv = 1.0f / sqrtf(ss / (float)hd + eps);
        }
        for (int d = tid; d < hd; d += QP_THREADS) {
            float y = xs[d];
            if (d < rot) {
                // pair i is (i, i + rot/2), or with `interleaved` (2i, 2i + 1)
                const int i = interleaved ? d >> 1 : (d < half ? d : d - half);
                const float2 cs = table[(size_t)t * half + i];
                float y1, y2;
                rope_pair(xs[interleaved ? 2 * i : i], xs[interleaved ? 2 * i + 1 : i + half], cs.x, cs.y, y1, y2);
                y = (interleaved ? (d & 1) == 0 : d < half) ? y1 : y2;
            }
            y *= inv;
            if (is_q) q_out[(size_t)t * ldq + col0 + d] = from_f32<TQ>(y);
            else if (append && page >= 0) k_cache[cache_offset(page, slot - nh, pos, nkv, hd) + d] = from_f32<TC>(y);
        }
    } else {
        // the values: a projection of their own, or (`v_from_k`) the keys as projected, before their norm and rotation
        const int g = slot - nh - nkv;
        const int col0 = v_from_k ? nh * hd + g * hd : (nh + nkv) * hd + g * vd;
        const TP* row = proj + (size_t)t * ldp + col0;
        const float lam = v_mode == 2 ? v_lambda[0] : 0.0f;
        float* vf = v_first ? pdl_fresh(v_first) + (size_t)t * nkv * vd + (size_t)g * vd : nullptr;
        for (int d = tid; d < vd; d += QP_THREADS) {
            float v = to_f32(row[d]) + (bias ? bias[col0 + d] : 0.0f);
            if (v_mode == 1) vf[d] = v;
            else if (v_mode == 2) v = (1.0f - lam) * v + lam * vf[d];
            if (append && page >= 0) v_cache[cache_offset(page, g, pos, nkv, vd) + d] = from_f32<TC>(v);
        }
    }
}

extern "C" int hb_qkv_prepare(const void* proj, int proj_dtype, long long ldp, const float* bias, const float* table, int rot,
                              int n_heads, int n_kv_heads, int head_dim, int v_dim, int unit_norm, const float* q_norm_w,
                              const float* k_norm_w, float eps, void* q_out, int q_dtype, long long ldq, void* k_cache, void* v_cache, int cache_dtype, const int* page_table,
                              int pt_width, const int* tok_seq, const int* positions, int n_tokens, int n_pages, int append,
                              const float* v_lambda, float* v_first, int v_mode, int interleaved, int v_from_k, int* status,
                              void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && v_dim > 0, "qkv_prepare: bad sizes");
    HB_REQUIRE(!v_from_k || v_dim == head_dim, "qkv_prepare: values that are the keys have the keys' size");
    HB_REQUIRE(head_dim <= QP_MAX_HD, "qkv_prepare: head size %d is larger than %d", head_dim, QP_MAX_HD);
    HB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= head_dim, "qkv_prepare: %d rotated dimensions of %d", rot, head_dim);
    HB_REQUIRE(rot == 0 || table != nullptr, "qkv_prepare: no rotation table");
    HB_REQUIRE(unit_norm >= 0 && unit_norm <= 2 && (unit_norm != 2 || (q_norm_w != nullptr && k_norm_w != nullptr)),
               "qkv_prepare: norm mode %d (0 none, 1 unit norm behind the rotation, 2 weighted norm in front of it)", unit_norm);
    HB_REQUIRE(v_mode >= 0 && v_mode <= 2 && (v_mode == 0 || v_first != nullptr) && (v_mode != 2 || v_lambda != nullptr),
               "qkv_prepare: value mixing needs its buffers");
    HB_REQUIRE(n_heads + 2 * n_kv_heads <= 65535, "qkv_prepare: too many heads");
    const bool cache_same = (q_dtype == cache_dtype);
    HB_REQUIRE(cache_same, "qkv_prepare: queries and cache must have one dtype");
    dim3 grid(n_tokens, n_heads + (append ? 2 * n_kv_heads : 0));
    cudaStream_t s = (cudaStream_t)stream;
#define HB_QP_LAUNCH(TP, TQ)                                                                                                   \
    hb_launch(qkv_prepare_kernel<TP, TQ, TQ>, dim3(grid), dim3(QP_THREADS), 0, s, (const TP*)proj, ldp, bias, (const float2*)table, rot,  \
              n_heads, n_kv_heads, head_dim, v_dim, unit_norm, q_norm_w, k_norm_w, eps, (TQ*)q_out, ldq, (TQ*)k_cache, (TQ*)v_cache, page_table,       \
              pt_width, tok_seq, positions, n_pages, append, v_lambda, v_first, v_mode, interleaved, v_from_k, status)
    if (proj_dtype == HB_F32 && q_dtype == HB_F32) HB_QP_LAUNCH(float, float);
    else if (proj_dtype == HB_F32 && q_dtype == HB_BF16) HB_QP_LAUNCH(float, bf16);
    else if (proj_dtype == HB_BF16 && q_dtype == HB_BF16) HB_QP_LAUNCH(bf16, bf16);
    else return hb_fail("qkv_prepare: unsupported dtypes %d -> %d", proj_dtype, q_dtype);
#undef HB_QP_LAUNCH
    return hb_check_launch("qkv_prepare");
}

// ---------------------------------------------------------------------------------------------
#define AS_THREADS 128
#define AS_MAX_HD 1024
#define AS_MAX_ACC 16         // value columns per thread: (value heads served) * v_dim <= 128 * 16

template <typename TQ, typename TC>
__global__ void __launch_bounds__(AS_THREADS)
attention_sink_kernel(const TQ* __restrict__ q, long long ldq, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                      const int* __restrict__ page_table, int pt_width, const int* __restrict__ tok_seq,
                      const int* __restrict__ positions, float* __restrict__ out, int nh, int nkv, int hd, int vd, float scale,
                      int window, int keep_first, int chunk, const float* __restrict__ sink, int all_values, int n_pages, int* status) {
    pdl_trigger();
    pdl_wait();
    q = pdl_fresh(q);
    k_cache = pdl_fresh(k_cache);
    v_cache = pdl_fresh(v_cache);
    __shared__ float qs[AS_MAX_HD];
    __shared__ float ps[AS_THREADS];
    __shared__ int key_of[AS_THREADS];
    __shared__ int page_of[AS_THREADS];
    __shared__ float scratch[33];
    const int t = blockIdx.x, j = blockIdx.y, tid = threadIdx.x;
    const int g = j / (nh / nkv);
    const int p = positions[t];
    const int* pt = page_table + (size_t)tok_seq[t] * pt_width;
    // the keys this query sees: [0, kept) and [lo, p]
    const int lo_w = hb_oldest_visible(p, window, chunk);
    const int kept = min(min(keep_first, lo_w), p + 1);
    const int lo = max(lo_w, kept);
    const int total = kept + (p - lo + 1);
    const TQ* qr = q + (size_t)t * ldq + (size_t)j * hd;
    for (int d = tid; d < hd; d += AS_THREADS) qs[d] = to_f32(qr[d]);
    __syncthreads();

    const int n_val = all_values ? nkv : 1;
    const int n_out = n_val * vd;
    // a sink is one more term exp(sink[j]) of the softmax's sum, with no value: the running maximum and sum start from it
    float m = sink ? sink[j] : -INFINITY, l = sink ? 1.0f : 0.0f;
    float acc[AS_MAX_ACC];
#pragma unroll
    for (int i = 0; i < AS_MAX_ACC; i++) acc[i] = 0.0f;

    for (int v0 = 0; v0 < total; v0 += AS_THREADS) {
        const int vi = v0 + tid;
        const bool valid = vi < total;
        float sc = -INFINITY;
        int s = 0, page = -1;
        if (valid) {
            s = vi < kept ? vi : lo + (vi - kept);
            const int lp = s / HB_PAGE_TOKENS;
            page = lp < pt_width ? pt[lp] : -1;
            if (page >= n_pages) page = -1;
            if (page < 0) hb_note(status, HB_STATUS_PAGE, 1 + tok_seq[t]);
            if (page >= 0) {
                const TC* kr = k_cache + cache_offset(page, g, s, nkv, hd);
                float dot = 0.0f;
                for (int d = 0; d < hd; d++) dot = fmaf(qs[d], to_f32(kr[d]), dot);
                sc = dot * scale;
            }
        }
        key_of[tid] = s;
        page_of[tid] = page;
        const float tmax = block_max(sc, scratch);
        const float m_new = fmaxf(m, tmax);
        const float pr = (sc == -INFINITY) ? 0.0f : expf(sc - m_new);
        ps[tid] = pr;
        const float tsum = block_sum(pr, scratch);          // also orders the writes above before the reads below
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + tsum;
        const int n_in_tile = min(AS_THREADS, total - v0);
#pragma unroll
        for (int i = 0; i < AS_MAX_ACC; i++) {
            const int e = tid + i * AS_THREADS;
            if (e < n_out) {
                const int c = all_values ? e / vd : g, d = all_values ? e - (e / vd) * vd : e;
                float a = acc[i] * corr;
                for (int x = 0; x < n_in_tile; x++) {
                    const float pe = ps[x];
                    if (pe != 0.0f) a = fmaf(pe, to_f32(v_cache[cache_offset(page_of[x], c, key_of[x], nkv, vd) + d]), a);
                }
                acc[i] = a;
            }
        }
        m = m_new;
        __syncthreads();
    }
    float* o = out + ((size_t)t * nh + j) * n_out;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < AS_MAX_ACC; i++) {
        const int e = tid + i * AS_THREADS;
        if (e < n_out) o[e] = acc[i] * inv;
    }
}

extern "C" int hb_attention_sink(const void* q, int q_dtype, long long ldq, const void* k_cache, const void* v_cache,
                                 int cache_dtype, const int* page_table, int pt_width, const int* tok_seq,
                                 const int* positions, float* out, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                 int v_dim, float scale, int window, int keep_first, int chunk, const float* sink, int all_values,
                                 int n_pages, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && v_dim > 0 && n_pages > 0, "attention: bad sizes");
    HB_REQUIRE(n_heads % n_kv_heads == 0, "attention: %d heads are no multiple of %d kv heads", n_heads, n_kv_heads);
    HB_REQUIRE(head_dim <= AS_MAX_HD, "attention: head size %d is larger than %d", head_dim, AS_MAX_HD);
    HB_REQUIRE((all_values ? n_kv_heads : 1) * v_dim <= AS_THREADS * AS_MAX_ACC,
               "attention: %d value columns per query head are more than %d", (all_values ? n_kv_heads : 1) * v_dim, AS_THREADS * AS_MAX_ACC);
    HB_REQUIRE(n_heads <= 65535 && window >= 0 && keep_first >= 0 && chunk >= 0, "attention: bad head count, window or kept tokens");
    HB_REQUIRE(chunk == 0 || (window == 0 && keep_first == 0), "attention: chunks come without a window and kept first tokens");
    dim3 grid(n_tokens, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_AS_LAUNCH(TQ, TC)                                                                                                  \
    hb_launch(attention_sink_kernel<TQ, TC>, dim3(grid), dim3(AS_THREADS), 0, s, (const TQ*)q, ldq, (const TC*)k_cache, (const TC*)v_cache, \
              page_table, pt_width, tok_seq, positions, out, n_heads, n_kv_heads, head_dim, v_dim, scale, window, keep_first,      \
              chunk, sink, all_values, n_pages, status)
    if (q_dtype == HB_F32 && cache_dtype == HB_F32) HB_AS_LAUNCH(float, float);
    else if (q_dtype == HB_BF16 && cache_dtype == HB_BF16) HB_AS_LAUNCH(bf16, bf16);
    else return hb_fail("attention: unsupported dtypes q %d cache %d", q_dtype, cache_dtype);
#undef HB_AS_LAUNCH
    return hb_check_launch("attention_sink");
}

// out[t, h*vd + d] = sum_g mix[h, g] * partial[t, g, c(h), d], c(h) = h / (nh / nkv) when the partial
// results hold all value heads (n_val == nkv), else partial[t, g, 0, d] is taken as it is (no mixing
// possible: mix must be null).  `ones` more columns follow the heads: a one and zeros, by which the
// product behind adds its bias as one more column of its weight.
template <typename TO>
__global__ void __launch_bounds__(256)
head_mix_kernel(const float* __restrict__ partial, const float* __restrict__ mix, TO* __restrict__ out, long long ldo, int nh,
                int nkv, int vd, int n_val, int ones, const float* __restrict__ gate, long long ldg) {
    pdl_trigger();
    pdl_wait();
    partial = pdl_fresh(partial);
    gate = pdl_fresh(gate);
    const int t = blockIdx.x;
    const float* pr = partial + (size_t)t * nh * n_val * vd;
    TO* o = out + (size_t)t * ldo;
    const int group = nh / nkv;
    for (int e = threadIdx.x; e < nh * vd; e += blockDim.x) {
        const int h = e / vd, d = e - h * vd;
        float a;
        if (mix != nullptr) {
            const int c = n_val == nkv ? h / group : 0;
            a = 0.0f;
            for (int g = 0; g < nh; g++) a = fmaf(mix[h * nh + g], pr[((size_t)g * n_val + c) * vd + d], a);
        } else {
            a = pr[(size_t)h * n_val * vd + d];
        }
        if (gate != nullptr) a *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));     // one gate per (token, head)
        o[e] = from_f32<TO>(a);
    }
    for (int e = threadIdx.x; e < ones; e += blockDim.x) o[nh * vd + e] = from_f32<TO>(e == 0 ? 1.0f : 0.0f);
}

extern "C" int hb_head_mix(const float* partial, const float* mix, void* out, int out_dtype, long long ldo, int n_tokens,
                           int n_heads, int n_kv_heads, int v_dim, int n_val, int ones, const float* gate, long long ldg, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && v_dim > 0 && ones >= 0, "head_mix: bad sizes");
    HB_REQUIRE(n_val == 1 || n_val == n_kv_heads, "head_mix: partial results hold %d value heads, 1 or %d expected", n_val, n_kv_heads);
    HB_REQUIRE(mix == nullptr || n_val == n_kv_heads, "head_mix: mixing needs the partial results of every value head");
    HB_REQUIRE(ldo >= (long long)n_heads * v_dim + ones, "head_mix: output rows are too short");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16)
        hb_launch(head_mix_kernel<bf16>, dim3(n_tokens), dim3(256), 0, s, partial, mix, (bf16*)out, ldo, n_heads, n_kv_heads, v_dim, n_val, ones, gate, ldg);
    else if (out_dtype == HB_F32)
        hb_launch(head_mix_kernel<float>, dim3(n_tokens), dim3(256), 0, s, partial, mix, (float*)out, ldo, n_heads, n_kv_heads, v_dim, n_val, ones, gate, ldg);
    else return hb_fail("head_mix: unsupported output dtype %d", out_dtype);
    return hb_check_launch("head_mix");
}

// ---------------------------------------------------------------------------------------------
// attention_heads: the same attention, one block per (token, key split) for ALL query heads, so
// that a tile of keys and values is brought into shared memory once and serves every head:
// with mixed heads each head's weights meet the values of every key/value head, which makes
// the weighted value sums a product [heads x keys] x [keys x (kv heads * v_dim)] per token.
// Per tile of KT keys: scores by one thread per (kv head, key) for the heads of that group;
// softmax bookkeeping by one warp per head (running maximum m, sum l, in float32); then every
// thread adds the tile to its accumulators: 2 value columns for each of its heads, four keys at a time.
// With one split and all heads of a column in one thread the block also mixes the heads and
// writes the attention output; otherwise it writes unnormalised sums with (m, l) per head and
// split, and head_mix combines splits and heads.
// MMA variant (bfloat16 cache, 16 or 32 heads, up to 1024 value columns): the product of the tile's weights
// [heads x keys] with its values [keys x columns] runs on the tensor cores (mma.sync m16n8k16).  The weights
// are 32-bit; each is handed over as TWO bfloat16 terms, hi = bf16(p) and lo = bf16(p - hi), and the two
// products are added in the 32-bit accumulator: p is then exact to 16 mantissa bits (relative 2^-17), far
// below the rounding of the bfloat16 values it multiplies.  Scores, maxima, sums and mixing stay FP32 code.
#define AH_THREADS 512
#define AH_CPT 2

template <typename TQ, typename TC, typename TO, int HPT, int KT, bool MMA>
__global__ void __launch_bounds__(AH_THREADS)
attention_heads_kernel(const TQ* __restrict__ q, long long ldq, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                       const int* __restrict__ page_table, int pt_width, const int* __restrict__ tok_seq,
                       const int* __restrict__ positions, float* __restrict__ partial, float* __restrict__ ml,
                       const float* __restrict__ mix, TO* __restrict__ out, long long ldo, int ones, int nh, int nkv, int hd,
                       int vd, float scale, int window, int keep_first, int chunk, const float* __restrict__ sink, int splits,
                       int n_pages, int* status) {
    pdl_trigger();
    constexpr int CE = 16 / (int)sizeof(TC);            // cache elements per 16-byte piece
    extern __shared__ __align__(16) unsigned char ah_smem[];
    const int NC = nkv * vd, kst = nkv * hd + CE, vst = NC + CE;   // rows are padded by 16 bytes against bank conflicts
    float* qs = reinterpret_cast<float*>(ah_smem);      // [nh][hd]
    float* Ss = qs + nh * hd;                           // [nh][KT]
    float* m_s = Ss + nh * KT;                          // [nh]
    float* l_s = m_s + nh;
    float* c_s = l_s + nh;
    int* key_of = reinterpret_cast<int*>(c_s + nh);     // [KT]
    int* page_of = key_of + KT;
    TC* Ks = reinterpret_cast<TC*>(page_of + KT + ((4 - ((nh * hd + nh * KT + 3 * nh + 2 * KT) & 3)) & 3));
    TC* Vs = Ks + (size_t)KT * kst;
    constexpr int PST = KT + 8;                         // row stride of the weights' two bfloat16 terms
    bf16* Ph = reinterpret_cast<bf16*>(Vs + (size_t)KT * vst);      // [nh][PST] (MMA only)
    bf16* Pl = Ph + nh * PST;

    const int t = blockIdx.x, split = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int p = positions[t];
    const int* pt = page_table + (size_t)tok_seq[t] * pt_width;
    const int lo_w = hb_oldest_visible(p, window, chunk);
    const int kept = min(min(keep_first, lo_w), p + 1);
    const int lo = max(lo_w, kept);
    const int total = kept + (p - lo + 1);
    const int per = (total + splits - 1) / splits;
    const int v_begin = split * per, v_end = min(total, v_begin + per);
    const int group = nh / nkv;
    // this thread's value columns and heads
    const int col_threads = (NC + AH_CPT - 1) / AH_CPT;
    const int hg = min(AH_THREADS / col_threads, nh);
    const int my_cg = tid % col_threads, my_hg = tid / col_threads;
    const bool works = my_hg < hg;
    const int col = my_cg * AH_CPT;
    float acc[HPT][AH_CPT];
#pragma unroll
    for (int i = 0; i < HPT; i++)
#pragma unroll
        for (int j = 0; j < AH_CPT; j++) acc[i][j] = 0.0f;
    // MMA: warp w owns the pairs of 8-column tiles w, w + 16, ... (up to 4); [row tile of 16 heads][pair][tile][fragment]
    float cacc[2][4][2][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b2 = 0; b2 < 4; b2++)
#pragma unroll
            for (int c2 = 0; c2 < 2; c2++)
#pragma unroll
                for (int e = 0; e < 4; e++) cacc[a][b2][c2][e] = 0.0f;
    const int MT = nh >> 4, n_pairs = NC >> 4, r0 = lane >> 2;

    pdl_wait();
    q = pdl_fresh(q);
    k_cache = pdl_fresh(k_cache);
    v_cache = pdl_fresh(v_cache);
    for (int i = tid; i < nh * hd; i += AH_THREADS) qs[i] = to_f32(q[(size_t)t * ldq + i]);
    for (int i = tid; i < nh; i += AH_THREADS) {
        // a sink (one more term exp(sink[i]) of the sum, with no value) is where the first split's running maximum and sum start
        const bool with_sink = sink != nullptr && split == 0;
        m_s[i] = with_sink ? sink[i] : -INFINITY;
        l_s[i] = with_sink ? 1.0f : 0.0f;
    }
    const int kcpr = hd / CE, vcpr = vd / CE;            // 16-byte pieces per key row and per value row
    for (int v0 = v_begin; v0 < v_end; v0 += KT) {
        __syncthreads();                                 // the tile before has been used up
        if (tid < KT) {
            const int vi = v0 + tid;
            int s = 0, page = -1;
            if (vi < v_end) {
                s = vi < kept ? vi : lo + (vi - kept);
                const int lp = s / HB_PAGE_TOKENS;
                page = lp < pt_width ? pt[lp] : -1;
                if (page >= n_pages) page = -1;
                if (page < 0) hb_note(status, HB_STATUS_PAGE, 1 + tok_seq[t]);
            }
            key_of[tid] = s;
            page_of[tid] = page;
        }
        __syncthreads();
        // the tile's keys and values: eight 16-byte loads in flight per thread (issued before any is stored: a
        // store to shared memory between them would keep the next load's address, read from shared memory, behind it)
        auto copy_rows = [&](const TC* cache, TC* dst, int row_elems, int dst_stride, int cpr) {
            const int n = KT * nkv * cpr;
            for (int base = tid; base < n; base += AH_THREADS * 8) {
                uint4 vals[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int i = base + u * AH_THREADS;
                    vals[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (i < n) {
                        const int piece = i % cpr, pair = i / cpr, g = pair % nkv, r = pair / nkv;
                        const int page = page_of[r];
                        if (page >= 0) vals[u] = *reinterpret_cast<const uint4*>(cache + cache_offset(page, g, key_of[r], nkv, row_elems) + piece * CE);
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int i = base + u * AH_THREADS;
                    if (i < n) {
                        const int piece = i % cpr, pair = i / cpr, g = pair % nkv, r = pair / nkv;
                        *reinterpret_cast<uint4*>(dst + (size_t)r * dst_stride + g * row_elems + piece * CE) = vals[u];
                    }
                }
            }
        };
        copy_rows(k_cache, Ks, hd, kst, kcpr);
        copy_rows(v_cache, Vs, vd, vst, vcpr);
        __syncthreads();
        // scores.  Few key/value heads (their keys of a tile would occupy less than half of the threads): thread
        // (head, key), the key row read once per head; the sum runs over the dimensions in the same order either way
        if (nkv * KT * 2 <= AH_THREADS) {
            for (int i = tid; i < nh * KT; i += AH_THREADS) {
                const int h = i / KT, r = i - h * KT;
                const TC* kr = Ks + (size_t)r * kst + (h / group) * hd;
                const float4* qh = reinterpret_cast<const float4*>(qs + h * hd);
                float dot = 0.0f;
                for (int d0 = 0; d0 < hd; d0 += CE) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(kr + d0);
                    const TC* kv = reinterpret_cast<const TC*>(&raw);
#pragma unroll
                    for (int e = 0; e < CE; e += 4) {
                        const float4 qv = qh[(d0 + e) >> 2];
                        dot = fmaf(qv.x, to_f32(kv[e]), dot);
                        dot = fmaf(qv.y, to_f32(kv[e + 1]), dot);
                        dot = fmaf(qv.z, to_f32(kv[e + 2]), dot);
                        dot = fmaf(qv.w, to_f32(kv[e + 3]), dot);
                    }
                }
                Ss[h * KT + r] = (v0 + r < v_end && page_of[r] >= 0) ? dot * scale : -INFINITY;
            }
        } else
        // many key/value heads: thread (kv head, key), the heads of the group one after the other
        for (int i = tid; i < nkv * KT; i += AH_THREADS) {
            const int g = i / KT, r = i - g * KT;
            const TC* kr = Ks + (size_t)r * kst + g * hd;
            const bool valid = v0 + r < v_end && page_of[r] >= 0;
            for (int hh = 0; hh < group; hh++) {
                const float* qh = qs + (g * group + hh) * hd;
                float dot = 0.0f;
                for (int d0 = 0; d0 < hd; d0 += CE) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(kr + d0);
                    const TC* kv = reinterpret_cast<const TC*>(&raw);
#pragma unroll
                    for (int e = 0; e < CE; e++) dot = fmaf(qh[d0 + e], to_f32(kv[e]), dot);
                }
                Ss[(g * group + hh) * KT + r] = valid ? dot * scale : -INFINITY;
            }
        }
        __syncthreads();
        // running maximum and sum: one warp per head, one lane per key
        for (int h = warp; h < nh; h += AH_THREADS / 32) {
            const float s = lane < KT ? Ss[h * KT + lane] : -INFINITY;
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float pr = (s == -INFINITY) ? 0.0f : expf(s - m_new);
            const float sum = warp_sum(pr);
            if (lane < KT) {
                Ss[h * KT + lane] = pr;
                if (MMA) {
                    const bf16 hi = __float2bfloat16_rn(pr);
                    Ph[h * PST + lane] = hi;
                    Pl[h * PST + lane] = __float2bfloat16_rn(pr - __bfloat162float(hi));
                }
            }
            if (lane == 0) {
                const float corr = (m_old == -INFINITY) ? 0.0f : expf(m_old - m_new);
                m_s[h] = m_new;
                l_s[h] = l_s[h] * corr + sum;
                c_s[h] = corr;
            }
        }
        __syncthreads();
        if (MMA) {
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                if (mt < MT) {
                    const float c0 = c_s[mt * 16 + r0], c1 = c_s[mt * 16 + r0 + 8];
#pragma unroll
                    for (int i = 0; i < 4; i++)
#pragma unroll
                        for (int hf = 0; hf < 2; hf++) {
                            cacc[mt][i][hf][0] *= c0;
                            cacc[mt][i][hf][1] *= c0;
                            cacc[mt][i][hf][2] *= c1;
                            cacc[mt][i][hf][3] *= c1;
                        }
                }
            }
            const uint32_t ph_base = (uint32_t)__cvta_generic_to_shared(Ph), pl_base = (uint32_t)__cvta_generic_to_shared(Pl);
            const uint32_t v_base = (uint32_t)__cvta_generic_to_shared(Vs);
            const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
            const int v_row = ((lane >> 3) & 1) * 8 + (lane & 7), v_chunk = lane >> 4;
#pragma unroll
            for (int ks = 0; ks < KT / 16; ks++) {
                uint32_t ah[2][4], al[2][4];
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    if (mt < MT) {
                        const uint32_t off = (uint32_t)(((mt * 16 + a_row) * PST + ks * 16 + a_col) * 2);
                        ldmatrix_x4(ah[mt], ph_base + off);
                        ldmatrix_x4(al[mt], pl_base + off);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int pr2 = warp + 16 * i;
                    if (pr2 < n_pairs) {
                        uint32_t vf[4];
                        ldmatrix_x4_trans(vf, v_base + (uint32_t)(((ks * 16 + v_row) * vst + pr2 * 16 + v_chunk * 8) * 2));
#pragma unroll
                        for (int mt = 0; mt < 2; mt++) {
                            if (mt < MT) {
                                mma_bf16_16816(cacc[mt][i][0], ah[mt], vf[0], vf[1]);
                                mma_bf16_16816(cacc[mt][i][0], al[mt], vf[0], vf[1]);
                                mma_bf16_16816(cacc[mt][i][1], ah[mt], vf[2], vf[3]);
                                mma_bf16_16816(cacc[mt][i][1], al[mt], vf[2], vf[3]);
                            }
                        }
                    }
                }
            }
        } else if (works && col < NC) {
#pragma unroll
            for (int i = 0; i < HPT; i++) {
                const int h = my_hg + i * hg;
                if (h < nh) {
                    const float c = c_s[h];
#pragma unroll
                    for (int j = 0; j < AH_CPT; j++) acc[i][j] *= c;
                }
            }
            // rows beyond the split's last key hold zero weights and zero values: whole groups of four keys
            const int n_keys = (min(KT, v_end - v0) + 3) & ~3;
            for (int r = 0; r < n_keys; r += 4) {
                float v[4][AH_CPT];
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const TC* vr = Vs + (size_t)(r + x) * vst + col;
#pragma unroll
                    for (int j = 0; j < AH_CPT; j++) v[x][j] = to_f32(vr[j]);
                }
#pragma unroll
                for (int i = 0; i < HPT; i++) {
                    const int h = my_hg + i * hg;
                    if (h < nh) {
                        const float4 pe = *reinterpret_cast<const float4*>(Ss + h * KT + r);
#pragma unroll
                        for (int j = 0; j < AH_CPT; j++)
                            acc[i][j] = fmaf(pe.w, v[3][j], fmaf(pe.z, v[2][j], fmaf(pe.y, v[1][j], fmaf(pe.x, v[0][j], acc[i][j]))));
                    }
                }
            }
        }
    }
    __syncthreads();
    if (MMA) {
        // the accumulators: rows (heads) r0, r0 + 8 of each row tile, columns (lane & 3) * 2 + {0, 1} of each 8-column tile
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int pr2 = warp + 16 * i;
            if (pr2 >= n_pairs) continue;                   // the same for the whole warp
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                const int n0 = pr2 * 16 + hf * 8, cc = (lane & 3) * 2;
                if (out != nullptr) {
                    const int cv = n0 / vd, d0 = n0 - cv * vd + cc;     // an 8-column tile lies inside one value head
                    for (int h2 = cv * group; h2 < (cv + 1) * group; h2++) {
                        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
                        for (int mt = 0; mt < 2; mt++) {
                            if (mt < MT) {
                                const int g0 = mt * 16 + r0, g1 = g0 + 8;
                                const float w0 = (mix ? mix[h2 * nh + g0] : (g0 == h2 ? 1.0f : 0.0f)) / l_s[g0];
                                const float w1 = (mix ? mix[h2 * nh + g1] : (g1 == h2 ? 1.0f : 0.0f)) / l_s[g1];
                                s0 = fmaf(w1, cacc[mt][i][hf][2], fmaf(w0, cacc[mt][i][hf][0], s0));
                                s1 = fmaf(w1, cacc[mt][i][hf][3], fmaf(w0, cacc[mt][i][hf][1], s1));
                            }
                        }
#pragma unroll
                        for (int o = 4; o < 32; o <<= 1) {
                            s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                            s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                        }
                        if (r0 == 0) {
                            out[(size_t)t * ldo + h2 * vd + d0] = from_f32<TO>(s0);
                            out[(size_t)t * ldo + h2 * vd + d0 + 1] = from_f32<TO>(s1);
                        }
                    }
                } else {
#pragma unroll
                    for (int mt = 0; mt < 2; mt++) {
                        if (mt < MT) {
                            const int g0 = mt * 16 + r0, g1 = g0 + 8;
                            float* o0 = partial + (((size_t)t * nh + g0) * splits + split) * NC + n0 + cc;
                            float* o1 = partial + (((size_t)t * nh + g1) * splits + split) * NC + n0 + cc;
                            *reinterpret_cast<float2*>(o0) = make_float2(cacc[mt][i][hf][0], cacc[mt][i][hf][1]);
                            *reinterpret_cast<float2*>(o1) = make_float2(cacc[mt][i][hf][2], cacc[mt][i][hf][3]);
                        }
                    }
                }
            }
        }
        if (out != nullptr) {
            for (int e = tid; e < ones; e += AH_THREADS) out[(size_t)t * ldo + nh * vd + e] = from_f32<TO>(e == 0 ? 1.0f : 0.0f);
        } else {
            for (int h = tid; h < nh; h += AH_THREADS) {
                float* o = ml + (((size_t)t * nh + h) * splits + split) * 2;
                o[0] = m_s[h];
                o[1] = l_s[h];
            }
        }
        return;
    }
    if (out != nullptr) {
        // one split, every head of these columns in this thread: normalise, mix the heads, write the output
        if (works && col < NC) {
            const int c = col / vd, d = col - c * vd;
            for (int h2 = c * group; h2 < (c + 1) * group; h2++) {
                float o[AH_CPT];
#pragma unroll
                for (int j = 0; j < AH_CPT; j++) o[j] = 0.0f;
#pragma unroll
                for (int i = 0; i < HPT; i++) {
                    if (i < nh) {
                        const float w = (mix ? mix[h2 * nh + i] : (i == h2 ? 1.0f : 0.0f)) / l_s[i];
#pragma unroll
                        for (int j = 0; j < AH_CPT; j++) o[j] = fmaf(w, acc[i][j], o[j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < AH_CPT; j++) out[(size_t)t * ldo + h2 * vd + d + j] = from_f32<TO>(o[j]);
            }
        }
        for (int e = tid; e < ones; e += AH_THREADS) out[(size_t)t * ldo + nh * vd + e] = from_f32<TO>(e == 0 ? 1.0f : 0.0f);
        return;
    }
    if (works && col < NC) {
#pragma unroll
        for (int i = 0; i < HPT; i++) {
            const int h = my_hg + i * hg;
            if (h < nh) {
                float* o = partial + (((size_t)t * nh + h) * splits + split) * NC + col;
#pragma unroll
                for (int j = 0; j < AH_CPT; j++) o[j] = acc[i][j];
            }
        }
    }
    for (int h = tid; h < nh; h += AH_THREADS) {
        float* o = ml + (((size_t)t * nh + h) * splits + split) * 2;
        o[0] = m_s[h];
        o[1] = l_s[h];
    }
}

static size_t ah_smem_bytes(int nh, int nkv, int hd, int vd, int kt, int cache_elem, bool mma) {
    const int ce = 16 / cache_elem;
    size_t words = (size_t)nh * hd + (size_t)nh * kt + 3 * (size_t)nh + 2 * (size_t)kt;
    words = (words + 3) & ~(size_t)3;
    return words * 4 + ((size_t)kt * (nkv * hd + ce) + (size_t)kt * (nkv * vd + ce)) * cache_elem + (mma ? 2 * (size_t)nh * (kt + 8) * 2 : 0);
}

#define AH_VARIANT_MMA 64

// Whether attention_heads takes these sizes (else the caller uses attention_sink and head_mix):
// returns the heads-per-thread variant (4 or 32), 0 if none fits.
// `allow_mma` 0 keeps the tensor-core variant out (the tests compare the two).
extern "C" int hb_attention_heads_variant(int n_heads, int n_kv_heads, int head_dim, int v_dim, int cache_dtype, int allow_mma) {
    const int elem = cache_dtype == HB_BF16 ? 2 : 4, ce = 16 / elem, kt = cache_dtype == HB_BF16 ? 32 : 16;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || head_dim % ce || v_dim % ce || v_dim % AH_CPT) return 0;
    const int nc = n_kv_heads * v_dim, col_threads = (nc + AH_CPT - 1) / AH_CPT;
    if (allow_mma && cache_dtype == HB_BF16 && (n_heads == 16 || n_heads == 32) && nc % 16 == 0 && nc <= 1024
        && ah_smem_bytes(n_heads, n_kv_heads, head_dim, v_dim, kt, elem, true) <= 200 * 1024)
        return AH_VARIANT_MMA;
    if (col_threads > AH_THREADS) return 0;
    if (ah_smem_bytes(n_heads, n_kv_heads, head_dim, v_dim, kt, elem, false) > 200 * 1024) return 0;
    const int hg = min(AH_THREADS / col_threads, n_heads), hpt = (n_heads + hg - 1) / hg;
    return hpt <= 4 ? 4 : hpt <= 32 ? 32 : 0;
}

// Whether a step of one split gets its output (heads mixed, normalised) from the block itself.
extern "C" int hb_attention_heads_writes_output(int n_heads, int n_kv_heads, int head_dim, int v_dim, int cache_dtype, int allow_mma) {
    const int variant = hb_attention_heads_variant(n_heads, n_kv_heads, head_dim, v_dim, cache_dtype, allow_mma);
    if (variant == AH_VARIANT_MMA) return 1;
    if (variant == 0) return 0;
    const int col_threads = (n_kv_heads * v_dim + AH_CPT - 1) / AH_CPT;
    return min(AH_THREADS / col_threads, n_heads) == 1 ? 1 : 0;
}

template <typename TQ, typename TC, typename TO, int HPT, int KT, bool MMA>
static int ah_launch(dim3 grid, size_t smem, cudaStream_t s, const void* q, long long ldq, const void* k_cache, const void* v_cache,
                     const int* page_table, int pt_width, const int* tok_seq, const int* positions, float* partial, float* ml,
                     const float* mix, void* out, long long ldo, int ones, int nh, int nkv, int hd, int vd, float scale, int window,
                     int keep_first, int chunk, const float* sink, int splits, int n_pages, int* status) {
    static bool done[HB_MAX_DEVICES];
    if (!done[hb_device_slot()]) {
        cudaError_t e = cudaFuncSetAttribute(attention_heads_kernel<TQ, TC, TO, HPT, KT, MMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return hb_fail("attention_heads: %s", cudaGetErrorString(e));
        done[hb_device_slot()] = true;
    }
    hb_launch(attention_heads_kernel<TQ, TC, TO, HPT, KT, MMA>, dim3(grid), dim3(AH_THREADS), smem, s, (const TQ*)q, ldq, (const TC*)k_cache,
              (const TC*)v_cache, page_table, pt_width, tok_seq, positions, partial, ml, mix, (TO*)out, ldo, ones, nh, nkv, hd, vd, scale,
              window, keep_first, chunk, sink, splits, n_pages, status);
    return hb_check_launch("attention_heads");
}

// out non-null (one split, the variant holds every head in one thread): the mixed, normalised output [tokens][ldo];
// else partial [tokens][heads][splits][kv heads * v_dim] unnormalised and ml [tokens][heads][splits][2].
extern "C" int hb_attention_heads(const void* q, int q_dtype, long long ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                                  const int* page_table, int pt_width, const int* tok_seq, const int* positions, float* partial,
                                  float* ml, const float* mix, void* out, long long ldo, int ones, int n_tokens, int n_heads,
                                  int n_kv_heads, int head_dim, int v_dim, float scale, int window, int keep_first, int chunk,
                                  const float* sink, int splits, int n_pages, int allow_mma, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    const int variant = hb_attention_heads_variant(n_heads, n_kv_heads, head_dim, v_dim, cache_dtype, allow_mma);
    HB_REQUIRE(variant != 0, "attention_heads: these head sizes are not built");
    HB_REQUIRE(q_dtype == cache_dtype, "attention_heads: queries and cache must have one dtype");
    HB_REQUIRE(splits >= 1 && splits <= 65535 && window >= 0 && keep_first >= 0 && chunk >= 0 && n_pages > 0, "attention_heads: bad sizes");
    HB_REQUIRE(chunk == 0 || (window == 0 && keep_first == 0), "attention_heads: chunks come without a window and kept first tokens");
    const bool whole = hb_attention_heads_writes_output(n_heads, n_kv_heads, head_dim, v_dim, cache_dtype, allow_mma) != 0;
    HB_REQUIRE(out == nullptr || (splits == 1 && whole), "attention_heads: the block writes the output only with one split and every head in one thread");
    HB_REQUIRE(out != nullptr || (partial != nullptr && ml != nullptr), "attention_heads: no place for the partial results");
    const bool bf = cache_dtype == HB_BF16;
    const size_t smem = ah_smem_bytes(n_heads, n_kv_heads, head_dim, v_dim, bf ? 32 : 16, bf ? 2 : 4, variant == AH_VARIANT_MMA);
    dim3 grid(n_tokens, splits);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_AH(TQ, TO, HPT, KT, MMA)                                                                                                \
    return ah_launch<TQ, TQ, TO, HPT, KT, MMA>(grid, smem, s, q, ldq, k_cache, v_cache, page_table, pt_width, tok_seq, positions, partial, ml,  \
                                          mix, out, ldo, ones, n_heads, n_kv_heads, head_dim, v_dim, scale, window, keep_first, chunk, sink, splits,  \
                                          n_pages, status)
    if (bf) { if (variant == AH_VARIANT_MMA) HB_AH(bf16, bf16, 1, 32, true); else if (variant == 4) HB_AH(bf16, bf16, 4, 32, false); else HB_AH(bf16, bf16, 32, 32, false); }
    else { if (variant == 4) HB_AH(float, float, 4, 16, false); else HB_AH(float, float, 32, 16, false); }
#undef HB_AH
}

// ml null: one split whose sums are normalised already (the results of attention_sink_prefill for every value head).
// Combines key splits and mixes heads: out[t, h*vd + d] = sum_g mix[h, g] * (sum_s w_gs acc[t, g, s, c(h), d]) / (sum_s w_gs l_gs),
// w_gs = exp(m_gs - max_s m_gs); mix null: the head's own.
#define HM_COLS 32
template <typename TO>
__global__ void __launch_bounds__(256)
head_mix_splits_kernel(const float* __restrict__ partial, const float* __restrict__ ml, const float* __restrict__ mix,
                       TO* __restrict__ out, long long ldo, int nh, int nkv, int vd, int splits, int ones,
                       const float* __restrict__ gate, long long ldg) {
    // one block per (token, value head c, run of HM_COLS columns of c): first the splits of every head are combined
    // for these columns (shared memory [nh][HM_COLS]), then the heads that use c mix them
    pdl_trigger();
    pdl_wait();
    partial = pdl_fresh(partial);
    ml = pdl_fresh(ml);
    gate = pdl_fresh(gate);
    extern __shared__ float hm_smem[];
    float* wts = hm_smem;                               // [nh][splits]: w_gs / (sum_s w_gs l_gs)
    float* comb = hm_smem + nh * splits;                // [nh][HM_COLS]
    const int t = blockIdx.x, c = blockIdx.y, NC = nkv * vd, group = nh / nkv;
    const int d_begin = blockIdx.z * HM_COLS, dw = min(HM_COLS, vd - d_begin);
    for (int g = threadIdx.x; g < nh; g += blockDim.x) {
        if (ml == nullptr) {                            // one split, already normalised
            wts[g * splits] = 1.0f;
            continue;
        }
        const float* r = ml + ((size_t)t * nh + g) * splits * 2;
        float M = -INFINITY, den = 0.0f;
        for (int s = 0; s < splits; s++) M = fmaxf(M, r[2 * s]);
        for (int s = 0; s < splits; s++) den += (r[2 * s] == -INFINITY ? 0.0f : expf(r[2 * s] - M)) * r[2 * s + 1];
        for (int s = 0; s < splits; s++) wts[g * splits + s] = den > 0.0f ? (r[2 * s] == -INFINITY ? 0.0f : expf(r[2 * s] - M)) / den : 0.0f;
    }
    __syncthreads();
    const float* pr = partial + (size_t)t * nh * splits * NC + (size_t)c * vd + d_begin;
    for (int e = threadIdx.x; e < nh * dw; e += blockDim.x) {
        const int g = e / dw, d = e - g * dw;
        float v = 0.0f;
        for (int s = 0; s < splits; s++) v = fmaf(wts[g * splits + s], pr[((size_t)g * splits + s) * NC + d], v);
        comb[g * HM_COLS + d] = v;
    }
    __syncthreads();
    TO* o = out + (size_t)t * ldo;
    for (int e = threadIdx.x; e < group * dw; e += blockDim.x) {
        const int h = c * group + e / dw, d = e % dw;
        float a;
        if (mix != nullptr) {
            a = 0.0f;
            for (int g = 0; g < nh; g++) a = fmaf(mix[h * nh + g], comb[g * HM_COLS + d], a);
        } else {
            a = comb[h * HM_COLS + d];
        }
        if (gate != nullptr) a *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
        o[h * vd + d_begin + d] = from_f32<TO>(a);
    }
    if (c == 0 && blockIdx.z == 0)
        for (int e = threadIdx.x; e < ones; e += blockDim.x) o[nh * vd + e] = from_f32<TO>(e == 0 ? 1.0f : 0.0f);
}

extern "C" int hb_head_mix_splits(const float* partial, const float* ml, const float* mix, void* out, int out_dtype, long long ldo,
                                  int n_tokens, int n_heads, int n_kv_heads, int v_dim, int splits, int ones, const float* gate,
                                  long long ldg, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && v_dim > 0 && ones >= 0 && splits >= 1, "head_mix: bad sizes");
    HB_REQUIRE(ldo >= (long long)n_heads * v_dim + ones, "head_mix: output rows are too short");
    HB_REQUIRE(ml != nullptr || splits == 1, "head_mix: several splits need their maxima and sums");
    const size_t smem = ((size_t)n_heads * splits + (size_t)n_heads * HM_COLS) * sizeof(float);
    HB_REQUIRE(smem <= 48 * 1024 && n_kv_heads <= 65535, "head_mix: too many heads times (splits + value size)");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16)
        hb_launch(head_mix_splits_kernel<bf16>, dim3(n_tokens, n_kv_heads, (v_dim + HM_COLS - 1) / HM_COLS), dim3(256), smem, s, partial, ml, mix, (bf16*)out, ldo, n_heads, n_kv_heads, v_dim, splits, ones, gate, ldg);
    else if (out_dtype == HB_F32)
        hb_launch(head_mix_splits_kernel<float>, dim3(n_tokens, n_kv_heads, (v_dim + HM_COLS - 1) / HM_COLS), dim3(256), smem, s, partial, ml, mix, (float*)out, ldo, n_heads, n_kv_heads, v_dim, splits, ones, gate, ldg);
    else return hb_fail("head_mix: unsupported output dtype %d", out_dtype);
    return hb_check_launch("head_mix_splits");
}
