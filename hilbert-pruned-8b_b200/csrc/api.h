// C interface of the kernel library (loaded from Python with ctypes).
//
// Conventions: pointers are device pointers unless named host_*; `stream` is a cudaStream_t;
// dtypes are HbDtype codes (0 = float32, 1 = bfloat16); row-major matrices with explicit row
// strides in elements; every function returns 0 or sets hb_last_error().
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* hb_last_error(void);
int hb_device_info(int device, int* sm_major, int* sm_minor, int* sm_count);

// `status` (here and below): the caller's int32[4] status words (common.cuh: a bounded wait that
// ran out, non-finite logits, a bad page number, a bad token id), or null.
// `packed`: the table is stored as contiguous 128 x 64 tiles (the layout of hb_gemm_tc's packed weights);
// `scale` multiplies every embedding
int hb_embed(const int* tokens, const void* table, int table_dtype, float* out, int n_tokens, int hidden,
             int vocab, int packed, float scale, int* status, void* stream);
int hb_rmsnorm(const float* x, const float* weight, float eps, float offset, void* out, int out_dtype,
               const int* rows, int n_rows, int hidden, void* stream);
int hb_silu_mul(const void* gate_up, int in_dtype, long long in_stride, void* out, int out_dtype,
                long long out_stride, int n_rows, int inter, void* stream);
// out[t][i] = amplitude * (cos, sin)(inv_freq[i] * positions[t])
int hb_rope_table(const int* positions, const float* inv_freq, float* out, int n_tokens, int half, float amplitude,
                  void* stream);
int hb_rope_kv_append(void* qkv, int qkv_dtype, long long qkv_stride, const float* table, int rot,
                      int n_heads, int n_kv_heads, int head_dim, void* k_cache, void* v_cache, int cache_dtype,
                      const int* page_table, int pt_width, const int* tok_seq, const int* positions,
                      int n_tokens, int append, int n_pages, int* status, void* stream);
// Time marks of a timeline build (see common.cuh); other builds refuse.
int hb_timeline_set(void* marks, void* count, int capacity, int events);
int hb_gemm_general(const void* a, int a_dtype, long long lda, const void* w, int w_dtype, long long ldw,
                    void* out, int out_dtype, long long ldc, int M, int N, int K, int accumulate, void* stream);
int hb_gemm_tc_token_tile(int M);
long long hb_gemm_tc_scratch_floats(int M, int N, int K, int mode, int schedule);
long long hb_gemm_tc_tiles(int M, int N, int mode);
int hb_gemm_tc_resident_clusters(int mode, int size);
int hb_gemm_tc(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out, long long ldc,
               int M, int N, int K, int mode, int up_row0, int schedule, float* partials, long long partials_capacity,
               int* tile_counters, long long counters_capacity, int* error_flag, int packed, void* stream);
// A norm between two products, folded into them (hb_gemm_tc_fold; null pointers: that side is not used).
typedef struct {
    const float* prep_w;        // producer (mode 2): the norm's weight; the factor is prep_offset + prep_w[feature]
    float prep_offset;
    void* prep_out;             // bfloat16 [M, prep_ld]: the new residual values times the factor
    long long prep_ld;
    float* prep_sumsq;          // [M, sumsq_ld]: per token, the sums of squares of each 32 features
    const float* scale_sumsq;   // consumer (modes 0, 1, 3): such sums, written by the producer
    int scale_parts;            // how many of them per token
    float scale_inv_size;       // 1 / (features of the normed vector)
    float scale_eps;
    int sumsq_ld;
} HbNormFold;
int hb_gemm_tc_fold(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out, long long ldc,
               int M, int N, int K, int mode, int up_row0, int schedule, float* partials, long long partials_capacity,
               int* tile_counters, long long counters_capacity, int* error_flag, int packed, const HbNormFold* fold, void* stream);
int hb_gemm_tc2_wanted(int M, int N, int K);
int hb_gemm_tc2_resident_pairs(int mode);
int hb_gemm_tc2(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out, long long ldc,
                int M, int N, int K, int mode, int up_row0, int* error_flag, int packed, void* stream);
int hb_attention_general(const void* q, int q_dtype, long long q_stride, const void* k_cache, const void* v_cache,
                         int cache_dtype, const int* page_table, int pt_width, const int* tok_seq,
                         const int* positions, void* out, int out_dtype, long long out_stride, int n_tokens,
                         int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_pages, int* status,
                         void* stream);
int hb_attention_decode_supported(int n_heads, int n_kv_heads, int head_dim);
int hb_attention_decode_ctas_per_sm(int head_dim);
long long hb_attention_decode_scratch_floats(int batch, int n_heads, int head_dim, int splits);
int hb_attention_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                        const int* page_table, int pt_width, const int* positions, float* scratch, void* out,
                        long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim, float scale,
                        int window, int splits, int max_pages, int n_pages, int* status, void* stream);
int hb_attention_decode_combined(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                 const int* page_table, int pt_width, const int* positions, float* scratch, int* counters,
                                 void* out, long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim,
                                 float scale, int window, int splits, int max_pages, int n_pages, int* status,
                                 void* stream);
int hb_attention_decode_fused(const void* qkv, long long stride, const float* table, int rot, void* k_cache,
                              void* v_cache, const int* page_table, int pt_width, const int* positions, float* scratch,
                              int* counters, void* out, long long out_stride, int batch, int n_heads, int n_kv_heads,
                              int head_dim, float scale, int window, int splits, int max_pages, int n_pages, int append,
                              int* status, void* stream);
int hb_attention_prefill_supported(int n_heads, int n_kv_heads, int head_dim);
int hb_attention_prefill(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                         const int* page_table, int pt_width, const int* seq_start, const int* seq_pos0, void* out,
                         long long out_stride, int n_seqs, int q_blocks, int n_heads, int n_kv_heads, int head_dim,
                         float scale, int window, int n_pages, int* status, void* stream);
int hb_attention_prefill_tc_supported(int n_heads, int n_kv_heads, int head_dim);
int hb_attention_prefill_tc(const void* q, long long q_stride, long long n_tokens, const void* k_cache, const void* v_cache,
                            const int* page_table, int pt_width, const int* seq_start, const int* seq_pos0, void* out,
                            long long out_stride, int n_seqs, int q_blocks, int n_heads, int n_kv_heads, int head_dim,
                            float scale, int window, int n_pages, int* error_flag, void* stream);
// Dynamic tanh: out[r] = tanh(alpha[0] * x[rows[r]]) * w + b (rows null: row r)
int hb_dyt(const float* x, const float* w, const float* b, const float* alpha, void* out, int out_dtype, long long ldo,
           const int* rows, int n_rows, int C, void* stream);
// Short causal convolution over time with the last taps - 1 inputs of every sequence as state
// ([slot][taps - 1][C] floats at state + slot * state_stride): out = h + conv(h); with norm_w the
// input is the residual stream and h = dyt(x) is made on the way.
int hb_short_conv(const float* x, const float* norm_w, const float* norm_b, const float* norm_alpha, const float* conv_w,
                  int taps, float* state, long long state_stride, const int* state_slots, const int* seq_start, void* out,
                  int out_dtype, long long ldo, int n_seqs, int max_new, int C, void* stream);   // max_new: the most tokens a sequence brings
int hb_relu2(const void* in, int in_dtype, long long ldi, void* out, int out_dtype, long long ldo, int n_rows, int n,
             void* stream);
// Biases, rotation, unit norm, cache append (keys [pages][kv][64][head_dim], values [pages][kv][64][v_dim]);
// v_mode 0: values as they are; 1: also kept in v_first [tokens][kv * v_dim]; 2: mixed with v_first by v_lambda[0]
int hb_qkv_prepare(const void* proj, int proj_dtype, long long ldp, const float* bias, const float* table, int rot,
                   int n_heads, int n_kv_heads, int head_dim, int v_dim, int unit_norm, const float* q_norm_w, const float* k_norm_w,
                   float eps, void* q_out, int q_dtype, long long ldq, void* k_cache, void* v_cache, int cache_dtype, const int* page_table, int pt_width,
                   const int* tok_seq, const int* positions, int n_tokens, int n_pages, int append, const float* v_lambda,
                   float* v_first, int v_mode, int interleaved, int v_from_k, int* status, void* stream);
// out [tokens][heads][all_values ? kv heads : 1][v_dim] float32
int hb_attention_sink(const void* q, int q_dtype, long long ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                      const int* page_table, int pt_width, const int* tok_seq, const int* positions, float* out, int n_tokens,
                      int n_heads, int n_kv_heads, int head_dim, int v_dim, float scale, int window, int keep_first, int chunk,
                      const float* sink, int all_values, int n_pages, int* status, void* stream);
int hb_head_mix(const float* partial, const float* mix, void* out, int out_dtype, long long ldo, int n_tokens, int n_heads,
                int n_kv_heads, int v_dim, int n_val, int ones, const float* gate, long long ldg, void* stream);
// One block per (token, key split) for all heads; see attention_sink.cu.  hb_attention_heads_variant: 0 when the sizes are not built.
int hb_attention_heads_variant(int n_heads, int n_kv_heads, int head_dim, int v_dim, int cache_dtype, int allow_mma);
int hb_attention_heads_writes_output(int n_heads, int n_kv_heads, int head_dim, int v_dim, int cache_dtype, int allow_mma);
int hb_attention_heads(const void* q, int q_dtype, long long ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                       const int* page_table, int pt_width, const int* tok_seq, const int* positions, float* partial, float* ml,
                       const float* mix, void* out, long long ldo, int ones, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                       int v_dim, float scale, int window, int keep_first, int chunk, const float* sink, int splits, int n_pages,
                       int allow_mma, int* status, void* stream);
int hb_head_mix_splits(const float* partial, const float* ml, const float* mix, void* out, int out_dtype, long long ldo, int n_tokens,
                       int n_heads, int n_kv_heads, int v_dim, int splits, int ones, const float* gate, long long ldg, void* stream);
// Flash-style on the tensor cores for steps of many tokens (bfloat16, head sizes 64 or 128); out float32
// [tokens][heads][n_val][v_dim], n_val = kv heads (every value head) or 1 (the head's own); see attention_sink_prefill.cu.
int hb_attention_sink_prefill_supported(int n_heads, int n_kv_heads, int head_dim, int v_dim);
int hb_attention_sink_prefill(const void* q, long long q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                              int pt_width, const int* seq_start, const int* seq_pos0, float* out, int n_seqs, int q_blocks,
                              int n_heads, int n_kv_heads, int head_dim, int v_dim, int n_val, float scale, int window,
                              int keep_first, int chunk, const float* sink, int n_pages, int* status, void* stream);
// proj rows: [q heads*d | k heads*d | v heads*dv | gate heads*dv | z_i heads | z_f heads]; state per slot:
// S [heads][d][dv], n [heads][d], m [heads]; out [tokens][heads*dv] float32
int hb_mlstm_scan(const void* proj, int proj_dtype, long long ldp, const float* gate_bias, float cap, float q_scale, float* state,
                  long long state_stride, const int* state_slots, const int* seq_start, float* out, int n_seqs, int n_heads,
                  int d, int dv, void* stream);
// the same recurrence, 32 tokens at a time (steps that bring many tokens)
int hb_mlstm_chunks(const void* proj, int proj_dtype, long long ldp, const float* gate_bias, float cap, float q_scale, float* state,
                    long long state_stride, const int* state_slots, const int* seq_start, float* out, int n_seqs, int n_heads,
                    int d, int dv, void* stream);
int hb_mlstm_output(const float* o, const void* gate, int gate_dtype, long long ldg, const float* w, float eps, void* out,
                    int out_dtype, long long ldo, int n_tokens, int n_heads, int dv, void* stream);
// out[i] = mean + stdev * N(0, 1): element i of the counter-based stream `base`
int hb_random_normal(void* out, int out_dtype, long long n, unsigned long long base, float stdev, float mean,
                     void* stream);
int hb_argmax(const float* logits, long long stride, int* out, int n_rows, int vocab, int parts, void* scratch,
              int* counters, int* status, void* stream);
int hb_sample(const float* logits, long long stride, const float* temperature, const long long* seeds,
              const long long* request_ids, const long long* steps, int* out, int n_rows, int vocab, int* status,
              void* stream);

// A norm on a sublayer's output on its way into the residual stream: x += rmsnorm(y) * (offset + w); with w2 and h
// also h = rmsnorm(x) * (offset2 + w2) for the next sublayer (post_norm.cu).  out = sa a + sb b over n floats.
int hb_rmsnorm_add(const float* y, long long ldy, const float* w, float eps, float offset, float* x, long long ldx,
                   const float* w2, float eps2, float offset2, void* h, int h_dtype, long long ldh, int n_rows, int n, void* stream);
int hb_scaled_sum(const float* a, float sa, const float* b, float sb, float* out, long long n, void* stream);
// Window + pooled-block attention with sigmoid weights (attention_pool.cu).  proj rows: [q heads*d | k kv*d | v kv*dv | ...] float32.
int hb_qk_norm_append(const float* proj, long long ldp, const float* q_weight, const float* k_weight, float eps, void* q_out,
                      int q_dtype, long long ldq, void* k_cache, void* v_cache, int cache_dtype, const int* page_table, int pt_width,
                      const int* tok_seq, const int* positions, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int v_dim,
                      int n_pages, int append, int* status, void* stream);
int hb_pool_blocks(const void* k_cache, const void* v_cache, int cache_dtype, float* pk_cache, float* pv_cache, const int* pt_tok,
                   const int* pt_pool, int pt_width, const int* seq_pos0, const int* seq_len, int n_seqs, int max_new, int pool,
                   int n_kv_heads, int head_dim, int v_dim, int n_pages_tok, int n_pages_pool, int* status, void* stream);
int hb_attention_pool_supported(int head_dim, int v_dim);
// q_tiles: sum over the sequences of ceil(new tokens / 16); gate (float32, may be null) multiplies the result by its sigmoid;
// splits > 1: the keys are cut into ranges whose sums go to partial [splits][tokens][heads * v_dim] and are added by a second kernel
int hb_attention_pool(const void* q, int q_dtype, long long ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                      const float* pk_cache, const float* pv_cache, const int* pt_tok, const int* pt_pool, int pt_width,
                      const int* seq_start, const int* seq_pos0, int n_seqs, int q_tiles, const float* head_bias, const float* gate,
                      long long ldg, void* out, int out_dtype, long long ldo, float* partial, int n_tokens, int n_heads, int n_kv_heads,
                      int head_dim, int v_dim, float scale, int window, int pool, int n_pages_tok, int n_pages_pool, int splits,
                      int part, int grouped, int* status, void* stream);   // part 1: the pooled blocks alone, without the gate, into partial;
                                                                            // grouped: one token per sequence, a block's rows are a kv head's query heads
// the window part on the tensor cores (attention_pool_prefill.cu): bfloat16, head sizes 64 or 128, q_blocks = sum of ceil(new / 64);
// pooled: what hb_attention_pool made with part 1 (float32 [tokens][heads * v_dim]) or null
int hb_attention_pool_prefill_supported(int head_dim, int v_dim);
int hb_attention_pool_prefill(const void* q, long long q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                              int pt_width, const int* seq_start, const int* seq_pos0, const float* head_bias, const float* pooled,
                              const float* gate, long long ldg, void* out, long long out_stride, int n_seqs, int q_blocks, int n_heads,
                              int n_kv_heads, int head_dim, int v_dim, float scale, int window, int n_pages, int* status, void* stream);
// Matrix memory with a fixed decay per head (decay_memory.cu).  proj rows: [q heads*d | k heads*d | v heads*dv | ...] float32;
// state per slot: S [heads][d][dv]; out [tokens][heads*dv] float32; act 1: silu on q, k and v
int hb_decay_memory(const float* proj, long long ldp, const float* decay, float* state, long long state_stride, const int* state_slots,
                    const int* seq_start, float* out, long long ldo, int n_seqs, int n_heads, int d, int dv, int act, const float* table,
                    int rot, float k_scale, void* stream);
int hb_gated_norm(const float* o, long long ldi, const float* gate, long long ldg, const float* w, float eps, float out_scale, void* out,
                  int out_dtype, long long ldo, int n_rows, int n, int group, int gate_kind, void* stream);
// Layer norm with weight and bias: alone (optionally over gathered rows), and on a sublayer's output on its way into the
// residual stream (of one output, or of the weighted sum sa * y + sb * y2), with a copy of the new rows in another dtype
// (layer_norm.cu)
int hb_layernorm(const float* x, long long ldx, const float* w, const float* b, float eps, void* out, int out_dtype, long long ldo,
                 const int* rows, int n_rows, int n, void* stream);
int hb_layernorm_add(const float* y, long long ldy, const float* y2, long long ldy2, float sa, float sb, const float* w, const float* b,
                     float eps, float* x, long long ldx, void* copy, int copy_dtype, long long ldc, int n_rows, int n, void* stream);
int hb_convert(const float* x, void* out, int out_dtype, long long n, void* stream);
// Attention over one cached latent per token (latent_attention.cu): the cache rows, and the per-head products around it
int hb_latent_prepare(const float* proj, long long ldp, int n_heads, int d, int dr, int rank, int down_at, const float* c_weight, float eps,
                      const float* table, int rot, void* q_out, int q_dtype, long long ldq, int q_head, int q_rot_at, int q_copy, void* k_cache,
                      void* v_cache, int cache_dtype, const int* page_table, int pt_width, const int* tok_seq, const int* positions, int n_tokens,
                      int n_pages, int append, int* status, void* stream);
int hb_latent_gather(const void* v_cache, const int* page_table, int pt_width, const int* seq_len, int n_seqs, int max_pages, int rank,
                     void* rows, int* scratch_table, int scratch_width, int n_pages, int* status, void* stream);
int hb_latent_scatter(const void* kv, long long ldkv, const void* k_cache, const int* page_table, int pt_width, const int* seq_len, int n_seqs,
                      int max_pages, int n_heads, int d, int dr, int dv, int rank, int hd_out, int vd_out, void* k_out, void* v_out, int n_pages,
                      void* stream);
int hb_head_linear(const float* in, long long ldi, long long in_head, const void* w, int w_dtype, void* out, int out_dtype, long long ldo,
                   long long out_head, const float* gate, long long ldg, int n_tokens, int n_heads, int n_in, int n_out, void* stream);
// Short causal convolution with bias, activation and state; selective state-space scan (selective_scan.cu)
int hb_conv_act(const float* x, long long ldx, const float* conv_w, const float* conv_b, int taps, float* state, long long state_stride,
                const int* state_slots, const int* seq_start, void* out, int out_dtype, long long ldo, int n_seqs, int max_new, int C,
                int act, void* stream);
// chunk_len 0: one block walks a sequence's tokens; else chunks of chunk_len run side by side in three launches and need
// carry: n_seqs * max_chunks * inner * (2 * n_state + 1) floats (max_chunks = the most chunks a sequence has)
int hb_selective_scan(const void* u, int u_dtype, long long ldu, const float* bc, long long ldb, const float* z, long long ldz,
                      const float* dt_raw, long long lddt, const float* b_dt, const float* a_log, const float* dvec, float* state,
                      long long state_stride, const int* state_slots, const int* seq_start, void* out, int out_dtype, long long ldo,
                      int n_seqs, int inner, int n_state, int chunk_len, int max_chunks, float* carry, long long carry_floats,
                      void* stream);
// Mixture of experts (moe.cu)
int hb_moe_route(const void* h, int h_dtype, long long ldh, const float* w_router, int* experts, float* weights, int n_tokens, int width,
                 int n_experts, int top, void* stream);
// tile_rows: hb_moe_tile_rows(tensor_cores), the rows of a plan tile of the products' variant (FP32 pipe, or mma.sync for
// bfloat16 operands whose rows are multiples of 8 elements)
int hb_moe_tile_rows(int tensor_cores);
int hb_moe_plan(const int* experts, int n_entries, int n_experts, int tile_rows, int* offsets, int* order, int* tiles, void* stream);
int hb_moe_max_tiles(int n_entries, int n_experts, int tile_rows);
int hb_moe_glu(const void* h, int h_dtype, long long ldh, const void* w_gate, const void* w_up, int w_dtype, const int* offsets,
               const int* order, const int* tiles, int max_tiles, int top, void* act, int act_dtype, long long lda, int ff, int width,
               float limit, float alpha, int tensor_cores, void* stream);
int hb_moe_down(const void* act, int act_dtype, long long lda, const void* w_down, int w_dtype, const int* offsets, const int* order,
                const int* tiles, int max_tiles, int top, float* down, long long ldd, int width, int ff, int tensor_cores, void* stream);
// experts non-null: entries whose expert number is n_real or more are identity experts (their result is the row of h)
int hb_moe_combine(const float* down, long long ldd, const float* weights, int top, float* out, long long ldo, int n_tokens, int width,
                   int accumulate, const int* experts, int n_real, const void* h, int h_dtype, long long ldh, void* stream);
int hb_glu_clamp(const float* in, long long ldi, void* out, int out_dtype, long long ldo, int n_rows, int F, float limit, float alpha,
                 void* stream);
// softmax over all router outputs, choice by score + correction inside the `keep` best of `groups` runs, weights from the
// scores divided by their sum + norm_eps
int hb_moe_route_scores(const void* h, int h_dtype, long long ldh, const float* w_router, const float* correction, int* experts,
                        float* weights, int n_tokens, int width, int n_outputs, int top, int groups, int keep, float norm_eps,
                        void* stream);
// kind 0: gelu_tanh(in[:, :F]) * in[:, F:2F]; kind 1: gelu_erf(in[:, :F]) * sigmoid(in[:, row_gate]) (row_gate < 0: no gate)
int hb_gelu_unit(const float* in, long long ldi, void* out, int out_dtype, long long ldo, int n_rows, int F, int kind, int row_gate,
                 void* stream);
// Token embedding plus the hashed embedding of (previous token, token) (elementwise.cu); state: one int32 per slot
int hb_embed_pair(const int* tokens, const void* table, int table_dtype, const void* pairs, float* out, int n_tokens, int hidden,
                  int vocab, int packed, float scale, int buckets, long long mul_prev, long long mul_cur, const int* positions,
                  const int* tok_seq, const int* seq_start, const int* state_slots, int* state, long long state_stride, int* status,
                  void* stream);
// x += m * y, optionally followed by the next norm of the new rows; out (+)= norm(a) wa + norm(b) wb (post_norm.cu)
int hb_scaled_add_norm(const float* y, long long ldy, float m, float* x, long long ldx, const float* w2, float eps2, float offset2,
                       void* h, int h_dtype, long long ldh, int n_rows, int n, void* stream);
int hb_normed_sum(const float* a, long long lda, const float* wa, const float* b, long long ldb, const float* wb, float eps, float* out,
                  long long ldo, int n_rows, int n, int accumulate, void* stream);
// The recurrent memory per head with token-dependent decay (head_scan.cu): decay_mode 0 one scalar per (token, head) from a
// step size, 1 one per (token, head, state index) from a sigmoid; chunk_len 0: one block walks a sequence's tokens, else
// three launches with carry of n_seqs * max_chunks * heads * (2 * head_dim * n_state + (mode ? n_state : 1)) floats
int hb_head_scan(const float* u, long long ldu, const float* kmat, long long ldk, const float* qmat, long long ldq, const float* z,
                 long long ldz, const float* draw, long long ldd, const float* dbias, const float* a_log, float inv_tau,
                 const float* dskip, float q_scale, float* state, long long state_stride, const int* state_slots, const int* seq_start,
                 void* out, int out_dtype, long long ldo, int n_seqs, int n_heads, int n_groups, int head_dim, int n_state,
                 int decay_mode, int chunk_len, int max_chunks, float* carry, long long carry_floats, void* stream);

#ifdef __cplusplus
}
#endif
