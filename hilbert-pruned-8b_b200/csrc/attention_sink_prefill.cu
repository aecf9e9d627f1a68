// Attention with a sliding window that keeps the first tokens, for steps that bring many tokens:
// flash-style on the tensor cores (mma.sync m16n8k16, bfloat16 cache), for batches of sequences with
// unequal numbers of new tokens.
//
// One CTA = 64 consecutive new tokens of one sequence x one query head x ONE value head; each of its
// 4 warps owns 16 query rows.  With mixed heads a head's softmax weights meet the values of every
// key/value head (head_mix then mixes the per-(head, value head) results), so the value head is a grid
// index of its own and the scores are made once per value head; without mixing the grid has one value
// head per query head, its own.  Keys are walked page by page (64 keys) through a cp.async pipeline:
// first the pages of the kept first tokens that lie before the window, then the window's pages.  Query
// row at position p sees key s if s <= p and (p - s < window or s < keep_first); with `chunk` instead, if s lies in p's
// own run of `chunk` positions.  `sink_logit` (per head): one more term of the softmax's sum.  Scores, running
// maximum and sum are float32.  The weights enter the second product as TWO bfloat16 terms, hi = bf16(w)
// and lo = bf16(w - hi), added in the float32 accumulator: exact to 16 mantissa bits.  The result is
// normalised and written in float32: out[token][head][value head (or 0)][v_dim].
//
// Sizes: key heads of 64, 128, 192 or 256, value heads of 64 or 128; any head and group counts.
#include "api.h"
#include "mma.cuh"

#define SP_THREADS 128
#define SP_ROWS 64
#define SP_STAGES 2
#define SP_LOG2E 1.4426950408889634f

__device__ __forceinline__ void split_pack(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

template <int HD, int VD>
__global__ void __launch_bounds__(SP_THREADS)
attn_sink_prefill_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                         const int* __restrict__ page_table, int pt_width, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_pos0, float* __restrict__ out, int n_seqs, int nh, int nkv, int n_val,
                         float scale_log2e, int window, int keep_first, int chunk, const float* __restrict__ sink_logit, int n_pages,
                         int* status) {
    pdl_trigger();
    pdl_wait();
    q = pdl_fresh(q);
    kc = pdl_fresh(kc);
    vc = pdl_fresh(vc);
    constexpr int K_ROW = HD * 2, V_ROW = VD * 2;
    constexpr int K_TILE = HB_PAGE_TOKENS * K_ROW, V_TILE = HB_PAGE_TOKENS * V_ROW;
    constexpr int K_CHUNKS = K_ROW / 16, V_CHUNKS = V_ROW / 16, KSTEPS = HD / 16;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.x, g = head / (nh / nkv);
    const int vh = n_val == 1 ? g : (int)blockIdx.z;            // the value head whose values this CTA weighs

    // the sequence and the block of its new tokens this CTA serves: blocks from the back, heads fastest,
    // so that the query blocks that see the most keys start first
    int b = 0, blk = gridDim.y - 1 - blockIdx.y;
    for (; b < n_seqs; b++) {
        const int nb = (seq_start[b + 1] - seq_start[b] + SP_ROWS - 1) / SP_ROWS;
        if (blk < nb) break;
        blk -= nb;
    }
    if (b >= n_seqs) return;
    const int t_begin = seq_start[b], n_new = seq_start[b + 1] - t_begin, pos0 = seq_pos0[b];
    const int row_base = blk * SP_ROWS;
    const int rows_here = min(SP_ROWS, n_new - row_base);
    const int* pt = page_table + (size_t)b * pt_width;

    const int r0 = row_base + warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int p0 = pos0 + r0, p1 = pos0 + r1;
    const bool v0 = r0 < n_new, v1 = r1 < n_new;
    uint32_t qf[KSTEPS][4];
    {
        const int c = (lane & 3) * 2;
        const bf16* q0 = q + (size_t)(t_begin + r0) * q_stride + (size_t)head * HD;
        const bf16* q1 = q + (size_t)(t_begin + r1) * q_stride + (size_t)head * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c) : 0u;
            qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c) : 0u;
            qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c + 8) : 0u;
            qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c + 8) : 0u;
        }
    }
    // pages of the CTA: the window's, from the oldest key its first row sees to its last row's own key, and
    // before them the pages of kept first tokens that the window no longer covers
    const int first_pos = pos0 + row_base, last_pos = pos0 + row_base + rows_here - 1;
    const int lo_cta = hb_oldest_visible(first_pos, window, chunk);
    const int p_begin = lo_cta / HB_PAGE_TOKENS, p_end = last_pos / HB_PAGE_TOKENS + 1;
    const int n_sink = window > 0 ? min((keep_first + HB_PAGE_TOKENS - 1) / HB_PAGE_TOKENS, p_begin) : 0;
    const int n_iter = n_sink + (p_end - p_begin);
    const int lo0 = hb_oldest_visible(p0, window, chunk);
    const int lo1 = hb_oldest_visible(p1, window, chunk);
    const int w_first = pos0 + row_base + warp * 16, w_last = w_first + 15;
    const int w_lo = hb_oldest_visible(w_first, window, chunk);

    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    bool bad_page = false;
    auto load_page = [&](int stage, int it) {
        if (it < n_iter) {
            const int page_idx = it < n_sink ? it : p_begin + (it - n_sink);
            int page = page_idx < pt_width ? pt[page_idx] : -1;
            if (page < 0 || page >= n_pages) {                  // a fault of the host's bookkeeping: noted once, behind the loop
                bad_page = true;
                page = 0;
            }
            const uint8_t* ksrc = (const uint8_t*)(kc + ((size_t)page * nkv + g) * HB_PAGE_TOKENS * HD);
            const uint8_t* vsrc = (const uint8_t*)(vc + ((size_t)page * nkv + vh) * HB_PAGE_TOKENS * VD);
            const uint32_t kdst = smem_base + stage * (K_TILE + V_TILE), vdst = kdst + K_TILE;
#pragma unroll
            for (int i = tid; i < HB_PAGE_TOKENS * K_CHUNKS; i += SP_THREADS)
                cp_async_16(kdst + swizzled<K_ROW>(i / K_CHUNKS, i % K_CHUNKS), ksrc + (size_t)i * 16);
#pragma unroll
            for (int i = tid; i < HB_PAGE_TOKENS * V_CHUNKS; i += SP_THREADS)
                cp_async_16(vdst + swizzled<V_ROW>(i / V_CHUNKS, i % V_CHUNKS), vsrc + (size_t)i * 16);
        }
        cp_async_commit();
    };

    float o[VD / 8][4];
#pragma unroll
    for (int i = 0; i < VD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    if (sink_logit != nullptr) {
        // one more term exp(sink) of every row's sum, with no value: the running maximum starts there, and one lane of the
        // four that share a row carries the term in its part of the sum
        m[0] = m[1] = sink_logit[head] * SP_LOG2E;
        l[0] = l[1] = (lane & 3) == 0 ? 1.0f : 0.0f;
    }

#pragma unroll
    for (int s = 0; s < SP_STAGES - 1; s++) load_page(s, s);

    for (int it = 0; it < n_iter; it++) {
        cp_async_wait<SP_STAGES - 2>();
        __syncthreads();
        load_page((it + SP_STAGES - 1) % SP_STAGES, it + SP_STAGES - 1);
        const bool sink = it < n_sink;
        const int pi = sink ? it : p_begin + (it - n_sink);
        const int page_first = pi * HB_PAGE_TOKENS, page_last = page_first + HB_PAGE_TOKENS - 1;
        // nothing for this warp's rows here: a page behind them, or one in front of their windows without kept first tokens
        if (!sink && (page_first > w_last || (page_last < w_lo && page_first >= keep_first))) continue;
        const uint32_t kt = smem_base + (it % SP_STAGES) * (K_TILE + V_TILE), vt = kt + K_TILE;

        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
            for (int kq = 0; kq < 4; kq++) {
                uint32_t kf[4];
                const int key_row = kq * 16 + ((lane >> 4) << 3) + (lane & 7);
                ldmatrix_x4(kf, kt + swizzled<K_ROW>(key_row, 2 * ks + ((lane >> 3) & 1)));
                mma_bf16_16816(s[2 * kq], qf[ks], kf[0], kf[1]);
                mma_bf16_16816(s[2 * kq + 1], qf[ks], kf[2], kf[3]);
            }
        }
        const bool edge = sink || page_last > w_first || page_first < hb_oldest_visible(w_last, window, chunk);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = s[nt][e] * scale_log2e;
                if (edge) {
                    const int key = page_first + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int pp = (e >> 1) ? p1 : p0, ll = (e >> 1) ? lo1 : lo0;
                    if (key > pp || (key < ll && key >= keep_first)) v = -INFINITY;
                }
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float r = mx[h];
            r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, 1));
            r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, 2));
            const float m_new = fmaxf(m[h], r);
            const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = exp2f(m[h] - m_safe);
            m[h] = m_new;
            float sum = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float p = exp2f(s[nt][2 * h + e] - m_safe);
                    s[nt][2 * h + e] = p;
                    sum += p;
                }
            l[h] = l[h] * corr + sum;
#pragma unroll
            for (int i = 0; i < VD / 8; i++) {
                o[i][2 * h] *= corr;
                o[i][2 * h + 1] *= corr;
            }
        }
#pragma unroll
        for (int kq = 0; kq < 4; kq++) {
            uint32_t ph[4], pl[4];
            split_pack(s[2 * kq][0], s[2 * kq][1], ph[0], pl[0]);
            split_pack(s[2 * kq][2], s[2 * kq][3], ph[1], pl[1]);
            split_pack(s[2 * kq + 1][0], s[2 * kq + 1][1], ph[2], pl[2]);
            split_pack(s[2 * kq + 1][2], s[2 * kq + 1][3], ph[3], pl[3]);
            const int v_row = kq * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
            for (int dn = 0; dn < VD / 16; dn++) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vt + swizzled<V_ROW>(v_row, 2 * dn + (lane >> 4)));
                mma_bf16_16816(o[2 * dn], ph, vf[0], vf[1]);
                mma_bf16_16816(o[2 * dn], pl, vf[0], vf[1]);
                mma_bf16_16816(o[2 * dn + 1], ph, vf[2], vf[3]);
                mma_bf16_16816(o[2 * dn + 1], pl, vf[2], vf[3]);
            }
        }
    }
    cp_async_wait<0>();
    if (bad_page && tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + b);

#pragma unroll
    for (int h = 0; h < 2; h++) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
    const int c = (lane & 3) * 2;
    const int slot = n_val == 1 ? 0 : vh;
    if (v0) {
        float* dst = out + (((size_t)(t_begin + r0) * nh + head) * n_val + slot) * VD + c;
#pragma unroll
        for (int i = 0; i < VD / 8; i++) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][0] * inv0, o[i][1] * inv0);
    }
    if (v1) {
        float* dst = out + (((size_t)(t_begin + r1) * nh + head) * n_val + slot) * VD + c;
#pragma unroll
        for (int i = 0; i < VD / 8; i++) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2] * inv1, o[i][3] * inv1);
    }
}

extern "C" int hb_attention_sink_prefill_supported(int n_heads, int n_kv_heads, int head_dim, int v_dim) {
    return (head_dim == 64 || head_dim == 128 || head_dim == 192 || head_dim == 256) && (v_dim == 64 || v_dim == 128) && n_kv_heads > 0
           && n_heads % n_kv_heads == 0;
}

template <int HD, int VD>
static int launch_sink_prefill(const void* q, long long q_stride, const void* kc, const void* vc, const int* page_table, int pt_width,
                               const int* seq_start, const int* seq_pos0, float* out, int n_seqs, int q_blocks, int nh, int nkv,
                               int n_val, float scale, int window, int keep_first, int chunk, const float* sink, int n_pages, int* status,
                               cudaStream_t s) {
    constexpr int SMEM = SP_STAGES * HB_PAGE_TOKENS * (HD + VD) * 2;
    static bool attr_done[HB_MAX_DEVICES] = {};
    bool& attr_set = attr_done[hb_device_slot()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_sink_prefill_kernel<HD, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("attention_sink_prefill: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    dim3 grid(nh, q_blocks, n_val);
    hb_launch(attn_sink_prefill_kernel<HD, VD>, dim3(grid), dim3(SP_THREADS), SMEM, s, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc,
              page_table, pt_width, seq_start, seq_pos0, out, n_seqs, nh, nkv, n_val, scale * SP_LOG2E, window, keep_first, chunk, sink, n_pages, status);
    return hb_check_launch("attention_sink_prefill");
}

// q: [tokens, q_stride] bfloat16; out: float32 [tokens][heads][n_val][v_dim], n_val = kv heads (every value head, for
// mixed heads) or 1 (the head's own); q_blocks = sum over sequences of ceil(new tokens / 64).
extern "C" int hb_attention_sink_prefill(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                         const int* page_table, int pt_width, const int* seq_start, const int* seq_pos0,
                                         float* out, int n_seqs, int q_blocks, int n_heads, int n_kv_heads, int head_dim, int v_dim,
                                         int n_val, float scale, int window, int keep_first, int chunk, const float* sink, int n_pages, int* status,
                                         void* stream) {
    if (n_seqs == 0 || q_blocks == 0) return 0;
    HB_REQUIRE(hb_attention_sink_prefill_supported(n_heads, n_kv_heads, head_dim, v_dim),
               "attention_sink_prefill: head sizes %d and %d are not built (keys 64 to 256 in steps of 64, values 64 or 128)", head_dim, v_dim);
    HB_REQUIRE(n_seqs > 0 && q_blocks > 0 && q_blocks <= 65535 && window >= 0 && keep_first >= 0 && chunk >= 0, "attention_sink_prefill: bad sizes");
    HB_REQUIRE(chunk == 0 || (window == 0 && keep_first == 0), "attention_sink_prefill: chunks come without a window and kept first tokens");
    HB_REQUIRE(n_val == 1 || (n_val == n_kv_heads && n_val <= 65535), "attention_sink_prefill: %d value heads per head, 1 or %d expected", n_val, n_kv_heads);
    HB_REQUIRE(q_stride % 2 == 0 && ((uintptr_t)q & 3) == 0 && ((uintptr_t)out & 7) == 0, "attention_sink_prefill: queries and output must be aligned");
    HB_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, "attention_sink_prefill: cache must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
#define HB_SP(HD, VD)                                                                                                                     \
    return launch_sink_prefill<HD, VD>(q, q_stride, k_cache, v_cache, page_table, pt_width, seq_start, seq_pos0, out, n_seqs, q_blocks, n_heads, \
                                       n_kv_heads, n_val, scale, window, keep_first, chunk, sink, n_pages, status, s)
    if (head_dim == 256 && v_dim == 128) HB_SP(256, 128);
    if (head_dim == 256 && v_dim == 64) HB_SP(256, 64);
    if (head_dim == 192 && v_dim == 128) HB_SP(192, 128);
    if (head_dim == 192 && v_dim == 64) HB_SP(192, 64);
    if (head_dim == 128 && v_dim == 128) HB_SP(128, 128);
    if (head_dim == 128 && v_dim == 64) HB_SP(128, 64);
    if (head_dim == 64 && v_dim == 128) HB_SP(64, 128);
    HB_SP(64, 64);
#undef HB_SP
}
