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
//  * latent_gather, latent_scatter: keys and values of every head written out for steps of many tokens (see there).
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
                      TQ* __restrict__ q_out, long long ldq, int q_head, int q_rot_at, int q_copy, TQ* __restrict__ k_cache, TQ* __restrict__ v_cache,
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
        // the rotated part of head `slot`'s query at column q_rot_at of the head's q_head columns: behind the rank numbers
        // that head_linear fills (q_copy 0), or behind the head's own unrotated part, copied here, with zeros up to q_head
        const float* src = row + (size_t)slot * (d + dr) + d;
        TQ* head = q_out + (size_t)t * ldq + (size_t)slot * q_head;
        TQ* dst = head + q_rot_at;
        if (q_copy > 0) {
            for (int i = tid; i < q_copy; i += LP_THREADS) head[i] = from_f32<TQ>(src[i - d]);
            for (int i = q_rot_at + dr + tid; i < q_head; i += LP_THREADS) head[i] = from_f32<TQ>(0.0f);
        }
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
                                 int q_head, int q_rot_at, int q_copy, void* k_cache, void* v_cache, int cache_dtype, const int* page_table, int pt_width, const int* tok_seq,
                                 const int* positions, int n_tokens, int n_pages, int append, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_heads < 65535 && d > 0 && dr >= 0 && rank > 0, "latent_prepare: bad sizes");
    HB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dr && (rot == 0 || table != nullptr), "latent_prepare: %d rotated dimensions of %d", rot, dr);
    HB_REQUIRE(ldp >= (long long)down_at + rank + dr && down_at >= n_heads * (d + dr) && ldq >= (long long)n_heads * q_head,
               "latent_prepare: rows are too short");
    HB_REQUIRE(q_rot_at >= 0 && q_rot_at + dr <= q_head && (q_copy == 0 || (q_copy == d && q_rot_at == d)),
               "latent_prepare: the rotated part at %d of %d columns per head (%d copied) does not fit", q_rot_at, q_head, q_copy);
    HB_REQUIRE(q_dtype == cache_dtype, "latent_prepare: queries and cache must have one dtype");
    dim3 grid(n_tokens, n_heads + 1);
    cudaStream_t s = (cudaStream_t)stream;
    if (q_dtype == HB_BF16)
        hb_launch(latent_prepare_kernel<bf16>, dim3(grid), dim3(LP_THREADS), 0, s, proj, ldp, n_heads, d, dr, rank, down_at, c_weight, eps,
                  (const float2*)table, rot, (bf16*)q_out, ldq, q_head, q_rot_at, q_copy, (bf16*)k_cache, (bf16*)v_cache, page_table, pt_width, tok_seq, positions,
                  n_pages, append, status);
    else if (q_dtype == HB_F32)
        hb_launch(latent_prepare_kernel<float>, dim3(grid), dim3(LP_THREADS), 0, s, proj, ldp, n_heads, d, dr, rank, down_at, c_weight, eps,
                  (const float2*)table, rot, (float*)q_out, ldq, q_head, q_rot_at, q_copy, (float*)k_cache, (float*)v_cache, page_table, pt_width, tok_seq, positions,
                  n_pages, append, status);
    else return hb_fail("latent_prepare: unsupported dtype %d", q_dtype);
    return hb_check_launch("latent_prepare");
}

// ------------------------------------------------------------------------------------------------ keys and values written out
// For steps that bring many tokens the keys and values of every head are written out for the step's sequences, from the
// first token on, into a scratch cache of the ordinary paged layout (as many key/value heads as heads), which the
// tensor-core prompt kernel reads: with K_h = [Wuk_h c | k_r] of d + dr numbers the products are several times smaller
// than with the rank + dr numbers of the folded form.  Three steps: latent_gather copies the sequences' latents, page by
// page, into rows [scratch page * 64 + slot] (rows behind a sequence's end are zeros) and writes the scratch page table
// (sequence b owns the pages base_b .. base_b + pages_b - 1, base_b the pages of the sequences in front); one matrix
// product with [Wuk; Wuv] makes [k_u (heads x d) | v (heads x dv)] per row; latent_scatter lays them out head by head,
// appends the shared rotated key part from the cache and pads keys and values with zeros to the kernel's head sizes.
#define LE_THREADS 256

__device__ __forceinline__ int le_base_page(const int* __restrict__ seq_len, int b) {
    int base = 0;
    for (int i = 0; i < b; i++) base += (seq_len[i] + HB_PAGE_TOKENS - 1) / HB_PAGE_TOKENS;
    return base;
}

__global__ void __launch_bounds__(LE_THREADS)
latent_gather_kernel(const bf16* __restrict__ v_cache, const int* __restrict__ page_table, int pt_width, const int* __restrict__ seq_len,
                     int rank, bf16* __restrict__ rows, int* __restrict__ scratch_table, int scratch_width, int n_pages, int* status) {
    pdl_trigger();
    pdl_wait();
    v_cache = pdl_fresh(v_cache);
    const int j = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int len = seq_len[b], pages = (len + HB_PAGE_TOKENS - 1) / HB_PAGE_TOKENS;
    if (j >= pages) {
        if (tid == 0 && j < scratch_width) scratch_table[(size_t)b * scratch_width + j] = -1;
        return;
    }
    const int sp = le_base_page(seq_len, b) + j;
    if (tid == 0) scratch_table[(size_t)b * scratch_width + j] = sp;
    int page = j < pt_width ? page_table[(size_t)b * pt_width + j] : -1;
    if (page < 0 || page >= n_pages) {
        if (tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + b);
        page = -1;
    }
    const int valid = page < 0 ? 0 : min(HB_PAGE_TOKENS, len - j * HB_PAGE_TOKENS);
    const bf16* src = v_cache + (size_t)(page < 0 ? 0 : page) * HB_PAGE_TOKENS * rank;
    bf16* dst = rows + (size_t)sp * HB_PAGE_TOKENS * rank;
    const int live = valid * rank, all = HB_PAGE_TOKENS * rank;
    if ((rank & 7) == 0) {
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        for (int i = tid * 8; i < all; i += LE_THREADS * 8)
            *reinterpret_cast<uint4*>(dst + i) = i < live ? *reinterpret_cast<const uint4*>(src + i) : zero;
    } else {
        for (int i = tid; i < all; i += LE_THREADS) dst[i] = i < live ? src[i] : __float2bfloat16(0.0f);
    }
}

__global__ void __launch_bounds__(LE_THREADS)
latent_scatter_kernel(const bf16* __restrict__ kv, long long ldkv, const bf16* __restrict__ k_cache, const int* __restrict__ page_table,
                      int pt_width, const int* __restrict__ seq_len, int nh, int d, int dr, int dv, int rank, int hd_out, int vd_out,
                      bf16* __restrict__ k_out, bf16* __restrict__ v_out, int n_pages) {
    pdl_trigger();
    pdl_wait();
    kv = pdl_fresh(kv);
    k_cache = pdl_fresh(k_cache);
    const int j = blockIdx.x, b = blockIdx.y, h = blockIdx.z, tid = threadIdx.x;
    const int len = seq_len[b], pages = (len + HB_PAGE_TOKENS - 1) / HB_PAGE_TOKENS;
    if (j >= pages) return;
    const int sp = le_base_page(seq_len, b) + j;
    int page = j < pt_width ? page_table[(size_t)b * pt_width + j] : -1;
    if (page < 0 || page >= n_pages) page = -1;                 // latent_gather has noted it
    const int valid = page < 0 ? 0 : min(HB_PAGE_TOKENS, len - j * HB_PAGE_TOKENS);
    const bf16 zero = __float2bfloat16(0.0f);
    const bf16* krot = k_cache + (size_t)(page < 0 ? 0 : page) * HB_PAGE_TOKENS * (rank + dr) + rank;
    const bf16* src = kv + (size_t)sp * HB_PAGE_TOKENS * ldkv;
    bf16* kd = k_out + ((size_t)sp * nh + h) * HB_PAGE_TOKENS * hd_out;
    bf16* vd = v_out + ((size_t)sp * nh + h) * HB_PAGE_TOKENS * vd_out;
    for (int i = tid; i < HB_PAGE_TOKENS * hd_out; i += LE_THREADS) {
        const int r = i / hd_out, c = i - r * hd_out;
        bf16 x = zero;
        if (r < valid) {
            if (c < d) x = src[(size_t)r * ldkv + (size_t)h * d + c];
            else if (c < d + dr) x = krot[(size_t)r * (rank + dr) + (c - d)];
        }
        kd[i] = x;
    }
    for (int i = tid; i < HB_PAGE_TOKENS * vd_out; i += LE_THREADS) {
        const int r = i / vd_out, c = i - r * vd_out;
        vd[i] = (r < valid && c < dv) ? src[(size_t)r * ldkv + (size_t)nh * d + (size_t)h * dv + c] : zero;
    }
}

// rows: bfloat16 [scratch pages * 64, rank]; scratch_table int32 [n_seqs, scratch_width]; max_pages: the most pages a sequence has.
extern "C" int hb_latent_gather(const void* v_cache, const int* page_table, int pt_width, const int* seq_len, int n_seqs, int max_pages,
                                int rank, void* rows, int* scratch_table, int scratch_width, int n_pages, int* status, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && max_pages > 0 && rank > 0 && scratch_width >= max_pages, "latent_gather: bad sizes");
    HB_REQUIRE(((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)rows & 15) == 0, "latent_gather: the cache and the rows must be 16-byte aligned");
    hb_launch(latent_gather_kernel, dim3(scratch_width, n_seqs), dim3(LE_THREADS), 0, (cudaStream_t)stream, (const bf16*)v_cache, page_table,
              pt_width, seq_len, rank, (bf16*)rows, scratch_table, scratch_width, n_pages, status);
    return hb_check_launch("latent_gather");
}

// kv: bfloat16 [scratch pages * 64, ldkv] = [k_u (heads x d) | v (heads x dv) | ...]; k_out [scratch pages, heads, 64, hd_out],
// v_out [scratch pages, heads, 64, vd_out].
extern "C" int hb_latent_scatter(const void* kv, long long ldkv, const void* k_cache, const int* page_table, int pt_width, const int* seq_len,
                                 int n_seqs, int max_pages, int n_heads, int d, int dr, int dv, int rank, int hd_out, int vd_out, void* k_out,
                                 void* v_out, int n_pages, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_heads > 0 && n_heads <= 65535 && max_pages > 0, "latent_scatter: bad sizes");
    HB_REQUIRE(d > 0 && dr >= 0 && dv > 0 && hd_out >= d + dr && vd_out >= dv && ldkv >= (long long)n_heads * (d + dv), "latent_scatter: rows are too short");
    hb_launch(latent_scatter_kernel, dim3(max_pages, n_seqs, n_heads), dim3(LE_THREADS), 0, (cudaStream_t)stream, (const bf16*)kv, ldkv,
              (const bf16*)k_cache, page_table, pt_width, seq_len, n_heads, d, dr, dv, rank, hd_out, vd_out, (bf16*)k_out, (bf16*)v_out, n_pages);
    return hb_check_launch("latent_scatter");
}

// ------------------------------------------------------------------------------------------------ head_linear
// One block: 16 tokens x COLS output columns of one head (COLS 64, or 32 where 64 would leave most SMs without a block).
// A thread owns two neighbouring columns (one 4- or 8-byte weight load serves both) and every SLICES-th input feature,
// for all 16 tokens; the SLICES partial sums of an output are then added in a fixed order.  A decode step, whose few
// tokens give few blocks, so has many threads reading different weight rows at once instead of one thread walking all
// of a column's rows.  COLS is chosen from the sizes of the product alone, never from the number of tokens, so that a
// token's result does not depend on what else the step brings.
#define HL_TOKENS 16
#define HL_KC 256            // input features staged at a time
#define HL_THREADS 256       // COLS / 2 column pairs x SLICES slices of the input features

template <typename TW> struct hl_pair;
template <> struct hl_pair<bf16> {
    static __device__ __forceinline__ float2 load(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
};
template <> struct hl_pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
};

template <typename TW, typename TO, int HL_COLS>
__global__ void __launch_bounds__(HL_THREADS)
head_linear_kernel(const float* __restrict__ in, long long ldi, long long in_head, const TW* __restrict__ w, TO* __restrict__ out,
                   long long ldo, long long out_head, const float* __restrict__ gate, long long ldg, int n_tokens, int n_in, int n_out,
                   int pairs_aligned) {
    constexpr int HL_SLICES = 2 * HL_THREADS / HL_COLS;
    pdl_trigger();
    // the staged inputs [HL_TOKENS][HL_KC + 1]; afterwards the partial sums [HL_SLICES][HL_TOKENS][HL_COLS]
    __shared__ float sh[HL_SLICES * HL_TOKENS * HL_COLS];
    float (*xs)[HL_KC + 1] = reinterpret_cast<float (*)[HL_KC + 1]>(sh);
    const int t0 = blockIdx.x * HL_TOKENS, h = blockIdx.y, tid = threadIdx.x;
    const int cp = tid % (HL_COLS / 2), slice = tid / (HL_COLS / 2);
    const int col = blockIdx.z * HL_COLS + 2 * cp;
    const bool live0 = col < n_out, live1 = col + 1 < n_out, both = live1 && pairs_aligned;
    const TW* wh = w + (size_t)h * n_in * n_out;
    pdl_wait();
    in = pdl_fresh(in);
    gate = pdl_fresh(gate);
    float acc[HL_TOKENS][2];
#pragma unroll
    for (int j = 0; j < HL_TOKENS; j++) acc[j][0] = acc[j][1] = 0.0f;
    for (int k0 = 0; k0 < n_in; k0 += HL_KC) {
        const int kc = min(HL_KC, n_in - k0);
        __syncthreads();
        for (int i = tid; i < HL_TOKENS * kc; i += HL_THREADS) {
            const int j = i / kc, k = i - j * kc;
            xs[j][k] = (t0 + j < n_tokens) ? in[(size_t)(t0 + j) * ldi + (size_t)h * in_head + k0 + k] : 0.0f;
        }
        __syncthreads();
        if (live0) {
#pragma unroll 8
            for (int k = slice; k < kc; k += HL_SLICES) {
                const TW* wr = wh + (size_t)(k0 + k) * n_out + col;
                float2 wv;
                if (both) wv = hl_pair<TW>::load(wr);
                else wv = make_float2(to_f32(wr[0]), live1 ? to_f32(wr[1]) : 0.0f);
#pragma unroll
                for (int j = 0; j < HL_TOKENS; j++) {
                    const float x = xs[j][k];
                    acc[j][0] = fmaf(x, wv.x, acc[j][0]);
                    acc[j][1] = fmaf(x, wv.y, acc[j][1]);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < HL_TOKENS; j++)
        *reinterpret_cast<float2*>(&sh[(slice * HL_TOKENS + j) * HL_COLS + 2 * cp]) = make_float2(acc[j][0], acc[j][1]);
    __syncthreads();
    for (int i = tid; i < HL_TOKENS * HL_COLS; i += HL_THREADS) {
        const int j = i / HL_COLS, c = i - j * HL_COLS;
        const int t = t0 + j, oc = blockIdx.z * HL_COLS + c;
        if (t >= n_tokens || oc >= n_out) continue;
        float v = 0.0f;
#pragma unroll
        for (int sl = 0; sl < HL_SLICES; sl++) v += sh[(sl * HL_TOKENS + j) * HL_COLS + c];
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
        out[(size_t)t * ldo + (size_t)h * out_head + oc] = from_f32<TO>(v);
    }
}

extern "C" int hb_head_linear(const float* in, long long ldi, long long in_head, const void* w, int w_dtype, void* out, int out_dtype,
                              long long ldo, long long out_head, const float* gate, long long ldg, int n_tokens, int n_heads, int n_in,
                              int n_out, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_heads <= 65535 && n_in > 0 && n_out > 0, "head_linear: bad sizes");
    HB_REQUIRE((n_out + 31) / 32 <= 65535, "head_linear: too many output columns");
    // narrow tiles where wide ones would not fill the SMs once (a matter of the product's sizes only)
    const int cols = ((long long)n_heads * ((n_out + 63) / 64) < 148) ? 32 : 64;
    dim3 grid((n_tokens + HL_TOKENS - 1) / HL_TOKENS, n_heads, (n_out + cols - 1) / cols);
    cudaStream_t s = (cudaStream_t)stream;
    // two neighbouring weights in one load: every row of every head must start on a pair's boundary
    const int pairs_aligned = (n_out % 2 == 0 && ((uintptr_t)w & 7) == 0) ? 1 : 0;
#define HB_HL(TW, TO)                                                                                                              \
    do {                                                                                                                           \
        if (cols == 32)                                                                                                            \
            hb_launch(head_linear_kernel<TW, TO, 32>, dim3(grid), dim3(HL_THREADS), 0, s, in, ldi, in_head, (const TW*)w, (TO*)out, ldo, \
                      out_head, gate, ldg, n_tokens, n_in, n_out, pairs_aligned);                                                   \
        else                                                                                                                       \
            hb_launch(head_linear_kernel<TW, TO, 64>, dim3(grid), dim3(HL_THREADS), 0, s, in, ldi, in_head, (const TW*)w, (TO*)out, ldo, \
                      out_head, gate, ldg, n_tokens, n_in, n_out, pairs_aligned);                                                   \
    } while (0)
    if (w_dtype == HB_BF16 && out_dtype == HB_BF16) HB_HL(bf16, bf16);
    else if (w_dtype == HB_BF16 && out_dtype == HB_F32) HB_HL(bf16, float);
    else if (w_dtype == HB_F32 && out_dtype == HB_F32) HB_HL(float, float);
    else if (w_dtype == HB_F32 && out_dtype == HB_BF16) HB_HL(float, bf16);
    else return hb_fail("head_linear: unsupported dtypes %d -> %d", w_dtype, out_dtype);
#undef HB_HL
    return hb_check_launch("head_linear");
}
