// Attention whose keys and values are all made from one small latent per token (low-rank keys and
// values): per token the cache holds the normed latent c [rank] and one rotated key part k_r [dr]
// that every head shares.  Head h's key is [Wuk_h c | k_r], its value Wuv_h c, so with
//   q'_h = [Wuk_h^T q_h(unrotated) | rot(q_h(rotated))]          (rank + dr numbers)
// the score is q'_h . [c | k_r] and the head's result is Wuv_h (sum_s p_s c_s): attention with ONE
// key/value head whose key is [c | k_r] and whose value is c, between two small products per head.
//
//  * latent_prepare: per token, the latent part of the down projection divided by its root mean
//    square and multiplied by a weight, the shared key part turned by the step's rotation table, both
//    written to the cache (key row [c | k_r], value row c); every head's rotated query part turned
//    and written behind the place of its q'.  The rotation pairs dimensions (2i, 2i + 1).
//  * head_linear: out[t, h, :] = W_h in[t, h, :] for every head, W given as [heads][n_in][n_out]
//    (the output index contiguous), 32-bit accumulation on the FP32 pipe; optionally times
//    sigmoid(gate[t, h]).  Serves both q' (W = Wuk as stored) and the values (W = Wuv transposed).
#include "api.h"
#include "common.cuh"

#define LP_THREADS 128

template <typename TQ>
__global__ void __launch_bounds__(LP_THREADS)
latent_prepare_kernel(const float* __restrict__ proj, long long ldp, int nh, int d, int dr, int rank, int down_at,
                      const float* __restrict__ c_weight, float eps, const float2* __restrict__ table, int rot,
                      TQ* __restrict__ q_out, long long ldq, TQ* __restrict__ k_cache, TQ* __restrict__ v_cache,
                      const int* __restrict__ page_table, int pt_width, const int* __restrict__ tok_seq,
                      const int* __restrict__ positions, int n_pages, int append, int* status) {
    pdl_trigger();
    __shared__ float scratch[33];
    const int t = blockIdx.x, slot = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t], half = rot >> 1;
    int page = -1;
    if (slot == nh) {
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
    const float* row = proj + (size_t)t * ldp;
    if (slot < nh) {
        // the rotated part of head `slot`'s query, behind the rank numbers that head_linear fills
        const float* src = row + (size_t)slot * (d + dr) + d;
        TQ* dst = q_out + (size_t)t * ldq + (size_t)slot * (rank + dr) + rank;
        for (int i = tid; i < half; i += LP_THREADS) {
            const float2 cs = table[(size_t)t * half + i];
            float y1, y2;
            rope_pair(src[2 * i], src[2 * i + 1], cs.x, cs.y, y1, y2);
            dst[2 * i] = from_f32<TQ>(y1);
            dst[2 * i + 1] = from_f32<TQ>(y2);
        }
        for (int i = rot + tid; i < dr; i += LP_THREADS) dst[i] = from_f32<TQ>(src[i]);
        return;
    }
    const float* src = row + down_at;
    float ss = 0.0f;
    for (int i = tid; i < rank; i += LP_THREADS) ss = fmaf(src[i], src[i], ss);
    ss = block_sum(ss, scratch);
    if (!append || page < 0) return;
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    TQ* kr = k_cache + cache_offset(page, 0, pos, 1, rank + dr);
    TQ* vr = v_cache + cache_offset(page, 0, pos, 1, rank);
    for (int i = tid; i < rank; i += LP_THREADS) {
        const TQ c = from_f32<TQ>(src[i] * inv * c_weight[i]);
        kr[i] = c;
        vr[i] = c;
    }
    for (int i = tid; i < half; i += LP_THREADS) {
        const float2 cs = table[(size_t)t * half + i];
        float y1, y2;
        rope_pair(src[rank + 2 * i], src[rank + 2 * i + 1], cs.x, cs.y, y1, y2);
        kr[rank + 2 * i] = from_f32<TQ>(y1);
        kr[rank + 2 * i + 1] = from_f32<TQ>(y2);
    }
    for (int i = rot + tid; i < dr; i += LP_THREADS) kr[rank + i] = from_f32<TQ>(src[rank + i]);
}

extern "C" int hb_latent_prepare(const float* proj, long long ldp, int n_heads, int d, int dr, int rank, int down_at,
                                 const float* c_weight, float eps, const float* table, int rot, void* q_out, int q_dtype, long long ldq,
                                 void* k_cache, void* v_cache, int cache_dtype, const int* page_table, int pt_width, const int* tok_seq,
                                 const int* positions, int n_tokens, int n_pages, int append, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_heads < 65535 && d > 0 && dr >= 0 && rank > 0, "latent_prepare: bad sizes");
    HB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dr && (rot == 0 || table != nullptr), "latent_prepare: %d rotated dimensions of %d", rot, dr);
    HB_REQUIRE(ldp >= (long long)down_at + rank + dr && down_at >= n_heads * (d + dr) && ldq >= (long long)n_heads * (rank + dr),
               "latent_prepare: rows are too short");
    HB_REQUIRE(q_dtype == cache_dtype, "latent_prepare: queries and cache must have one dtype");
    dim3 grid(n_tokens, n_heads + 1);
    cudaStream_t s = (cudaStream_t)stream;
    if (q_dtype == HB_BF16)
        hb_launch(latent_prepare_kernel<bf16>, dim3(grid), dim3(LP_THREADS), 0, s, proj, ldp, n_heads, d, dr, rank, down_at, c_weight, eps,
                  (const float2*)table, rot, (bf16*)q_out, ldq, (bf16*)k_cache, (bf16*)v_cache, page_table, pt_width, tok_seq, positions,
                  n_pages, append, status);
    else if (q_dtype == HB_F32)
        hb_launch(latent_prepare_kernel<float>, dim3(grid), dim3(LP_THREADS), 0, s, proj, ldp, n_heads, d, dr, rank, down_at, c_weight, eps,
                  (const float2*)table, rot, (float*)q_out, ldq, (float*)k_cache, (float*)v_cache, page_table, pt_width, tok_seq, positions,
                  n_pages, append, status);
    else return hb_fail("latent_prepare: unsupported dtype %d", q_dtype);
    return hb_check_launch("latent_prepare");
}

// ------------------------------------------------------------------------------------------------ head_linear
#define HL_TOKENS 16
#define HL_COLS 64
#define HL_KC 256            // input features staged at a time
#define HL_THREADS 256       // HL_COLS output columns x 4 groups of HL_TOKENS / 4 tokens

template <typename TW, typename TO>
__global__ void __launch_bounds__(HL_THREADS)
head_linear_kernel(const float* __restrict__ in, long long ldi, long long in_head, const TW* __restrict__ w, TO* __restrict__ out,
                   long long ldo, long long out_head, const float* __restrict__ gate, long long ldg, int n_tokens, int n_in, int n_out) {
    pdl_trigger();
    __shared__ float xs[HL_TOKENS][HL_KC + 1];
    const int t0 = blockIdx.x * HL_TOKENS, h = blockIdx.y, tid = threadIdx.x;
    const int col = blockIdx.z * HL_COLS + (tid % HL_COLS), tg = tid / HL_COLS;
    const bool live = col < n_out;
    const TW* wh = w + (size_t)h * n_in * n_out;
    pdl_wait();
    in = pdl_fresh(in);
    gate = pdl_fresh(gate);
    float acc[HL_TOKENS / 4];
#pragma unroll
    for (int j = 0; j < HL_TOKENS / 4; j++) acc[j] = 0.0f;
    for (int k0 = 0; k0 < n_in; k0 += HL_KC) {
        const int kc = min(HL_KC, n_in - k0);
        __syncthreads();
        for (int i = tid; i < HL_TOKENS * kc; i += HL_THREADS) {
            const int j = i / kc, k = i - j * kc;
            xs[j][k] = (t0 + j < n_tokens) ? in[(size_t)(t0 + j) * ldi + (size_t)h * in_head + k0 + k] : 0.0f;
        }
        __syncthreads();
        if (live) {
            for (int k = 0; k < kc; k++) {
                const float wv = to_f32(wh[(size_t)(k0 + k) * n_out + col]);
#pragma unroll
                for (int j = 0; j < HL_TOKENS / 4; j++) acc[j] = fmaf(xs[tg * (HL_TOKENS / 4) + j][k], wv, acc[j]);
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int j = 0; j < HL_TOKENS / 4; j++) {
        const int t = t0 + tg * (HL_TOKENS / 4) + j;
        if (t >= n_tokens) continue;
        float v = acc[j];
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
        out[(size_t)t * ldo + (size_t)h * out_head + col] = from_f32<TO>(v);
    }
}

extern "C" int hb_head_linear(const float* in, long long ldi, long long in_head, const void* w, int w_dtype, void* out, int out_dtype,
                              long long ldo, long long out_head, const float* gate, long long ldg, int n_tokens, int n_heads, int n_in,
                              int n_out, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_heads <= 65535 && n_in > 0 && n_out > 0, "head_linear: bad sizes");
    HB_REQUIRE((n_out + HL_COLS - 1) / HL_COLS <= 65535, "head_linear: too many output columns");
    dim3 grid((n_tokens + HL_TOKENS - 1) / HL_TOKENS, n_heads, (n_out + HL_COLS - 1) / HL_COLS);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_HL(TW, TO)                                                                                                              \
    hb_launch(head_linear_kernel<TW, TO>, dim3(grid), dim3(HL_THREADS), 0, s, in, ldi, in_head, (const TW*)w, (TO*)out, ldo, out_head, gate, \
              ldg, n_tokens, n_in, n_out)
    if (w_dtype == HB_BF16 && out_dtype == HB_BF16) HB_HL(bf16, bf16);
    else if (w_dtype == HB_BF16 && out_dtype == HB_F32) HB_HL(bf16, float);
    else if (w_dtype == HB_F32 && out_dtype == HB_F32) HB_HL(float, float);
    else if (w_dtype == HB_F32 && out_dtype == HB_BF16) HB_HL(float, bf16);
    else return hb_fail("head_linear: unsupported dtypes %d -> %d", w_dtype, out_dtype);
#undef HB_HL
    return hb_check_launch("head_linear");
}
