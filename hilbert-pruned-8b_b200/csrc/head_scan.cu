// A recurrent matrix memory per head whose decay depends on the token: the state-space form with one scalar
// decay per (token, head), and the gated linear attention form with one decay per (token, head, key channel).
//
// Per sequence, head h, value channel j (of P) and state index n (of N), all in 32-bit:
//   S[j][n] <- a[t][h][n] S[j][n] + s[t][h] u[t][h][j] k[t][g(h)][n]          (evaluated as S + (a - 1) S + s u k)
//   y[t][h][j] = q_scale * sum_n S[j][n] q[t][g(h)][n] + D[h] u[t][h][j];   out = y * silu(z[t][h][j]) if z is given
// with g(h) = h / (H / G) (G groups of heads share k and q).  The decay a and the input's factor s:
//   mode 0 (scalar):  dt = softplus(dt_raw[t][h] + dt_bias[h]),  a = exp(-exp(A_log[h]) dt) for every n,  s = dt
//   mode 1 (channel): a = sigmoid(a_raw[t][h][n] + a_bias[h][n]) ^ inv_tau = exp(-softplus(-(..)) inv_tau),  s = 1
// a - 1 is made by expm1 from the decay's logarithm: with decays close to one, exp() rounded to 32 bits would be off by
// percents of the distance to one, and that error would grow with every token.
//
// A group of LANES threads owns a value channel (state index n = lane, lane + LANES, ...); a block owns CH = 256 / LANES
// channels of ONE head of one sequence and walks its tokens in order, HS_TOK tokens of inputs staged in shared memory
// at a time (what depends on the token alone, softplus, exponentials and the gate, is made while staging, once per block).
// The state [slot][H][P][N] is read once and written once per step.
//
// Steps that bring many tokens to a sequence while heads and channels are too few to fill the device cut the tokens into
// chunks and run three launches (the recurrence is linear in S): every chunk from a zero state, without outputs, leaving
// its final state L and the sum of the decays' logarithms; head_scan_carry: chunk by chunk, S_start[c + 1] =
// exp(sum log a) S_start[c] + L_c, which also leaves the sequence's new state; every chunk again from its S_start, with
// outputs.  The same sums in another order.
#include "api.h"
#include "common.cuh"

#define HS_THREADS 256
#define HS_TOK 32
#define HS_MAX_PER 8

__device__ __forceinline__ float hs_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename TO, int LANES>
__global__ void __launch_bounds__(HS_THREADS)
head_scan_kernel(const float* __restrict__ u, long long ldu, const float* __restrict__ kmat, long long ldk,
                 const float* __restrict__ qmat, long long ldq, const float* __restrict__ z, long long ldz,
                 const float* __restrict__ draw, long long ldd, const float* __restrict__ dbias, const float* __restrict__ a_log,
                 float inv_tau, const float* __restrict__ dskip, float q_scale, float* __restrict__ state, long long state_stride,
                 const int* __restrict__ state_slots, const int* __restrict__ seq_start, TO* __restrict__ out, long long ldo,
                 int H, int G, int P, int N, int decay_mode, int pass, int chunk_len, int max_chunks, float* __restrict__ carry_L,
                 float* __restrict__ carry_log, const float* __restrict__ carry_S0) {
    // pass 0: the whole step from the sequence's state; 1: chunk blockIdx.z % max_chunks from zeros, no outputs, L and
    // the decays' logarithms out; 3: that chunk from carry_S0, with outputs (head_scan_carry wrote the state)
    pdl_trigger();
    constexpr int CH = HS_THREADS / LANES;
    extern __shared__ float hs_smem[];
    float* ks = hs_smem;                       // [HS_TOK][N]: s * k
    float* qs = ks + HS_TOK * N;               // [HS_TOK][N]
    float* es = qs + HS_TOK * N;               // [HS_TOK][N] (mode 1) or [HS_TOK] (mode 0): a - 1
    float* us = es + HS_TOK * (decay_mode ? N : 1);   // [HS_TOK][CH]
    float* zs = us + HS_TOK * CH;              // [HS_TOK][CH]: silu(z), or 1
    float* ls = zs + HS_TOK * CH;              // [HS_TOK][N or 1]: the decays' logarithms (pass 1 only reads them)
    float* ds = ls + HS_TOK * (decay_mode ? N : 1);   // [HS_TOK]: the step sizes (mode 0)
    const int tid = threadIdx.x, lane = tid % LANES, ch = tid / LANES;
    const int h = blockIdx.y, g = h / (H / G);
    const int b = pass == 0 ? (int)blockIdx.z : (int)blockIdx.z / max_chunks;
    const int chunk = pass == 0 ? 0 : (int)blockIdx.z % max_chunks;
    const int j = blockIdx.x * CH + ch;
    const bool live = j < P;
    const int n_seq = seq_start[b + 1] - seq_start[b];
    const int t_lo = chunk * chunk_len;
    if (pass != 0 && t_lo >= n_seq) return;
    const int start = seq_start[b] + t_lo, n_all = pass == 0 ? n_seq : min(chunk_len, n_seq - t_lo);
    const float A = decay_mode == 0 ? -expf(a_log[h]) : 0.0f;
    const float bias0 = decay_mode == 0 ? dbias[h] : 0.0f;
    const float D = dskip != nullptr ? dskip[h] : 0.0f;
    const int LW = decay_mode ? N : 1;
    const size_t carry_at = (((size_t)b * max_chunks + chunk) * H + h) * (size_t)P + (live ? j : 0);
    const size_t carry_log_at = (((size_t)b * max_chunks + chunk) * H + h) * (size_t)LW;
    pdl_wait();
    u = pdl_fresh(u);
    kmat = pdl_fresh(kmat);
    qmat = pdl_fresh(qmat);
    z = pdl_fresh(z);
    draw = pdl_fresh(draw);
    state = pdl_fresh(state);
    carry_S0 = pdl_fresh(carry_S0);
    float* srow = state + (size_t)state_slots[b] * state_stride + ((size_t)h * P + (live ? j : 0)) * N;
    float S[HS_MAX_PER];
    float log_sum[HS_MAX_PER];                 // pass 1, mode 1: this lane's state indices; mode 0: every lane the same
#pragma unroll
    for (int k = 0; k < HS_MAX_PER; k++) {
        const int n = lane + k * LANES;
        S[k] = 0.0f;
        log_sum[k] = 0.0f;
        if (live && n < N && pass != 1) S[k] = pass == 0 ? srow[n] : carry_S0[carry_at * N + n];
    }
    for (int base = 0; base < n_all; base += HS_TOK) {
        const int nt = min(HS_TOK, n_all - base);
        __syncthreads();
        if (decay_mode == 0) {
            for (int i = tid; i < nt; i += HS_THREADS) {
                const size_t t = (size_t)(start + base + i);
                const float dt = hs_softplus(draw[t * ldd + h] + bias0);
                const float lg = A * dt;
                ds[i] = dt;
                ls[i] = lg;
                es[i] = expm1f(lg);
            }
            __syncthreads();
        }
        for (int i = tid; i < nt * N; i += HS_THREADS) {
            const int r = i / N, n = i - r * N;
            const size_t t = (size_t)(start + base + r);
            float s = 1.0f;
            if (decay_mode == 0) {
                s = ds[r];
            } else {
                const float zz = draw[t * ldd + (size_t)h * N + n] + dbias[(size_t)h * N + n];
                const float lg = -hs_softplus(-zz) * inv_tau;        // log(sigmoid(zz)) / tau
                ls[i] = lg;
                es[i] = expm1f(lg);
            }
            ks[i] = s * kmat[t * ldk + (size_t)g * N + n];
            qs[i] = qmat[t * ldq + (size_t)g * N + n];
        }
        for (int i = tid; i < nt * CH; i += HS_THREADS) {
            const int r = i / CH, c = i - r * CH, jj = blockIdx.x * CH + c;
            const size_t t = (size_t)(start + base + r);
            us[i] = jj < P ? u[t * ldu + (size_t)h * P + jj] : 0.0f;
            float gate = 1.0f;
            if (z != nullptr && jj < P) {
                const float zv = z[t * ldz + (size_t)h * P + jj];
                gate = zv / (1.0f + expf(-zv));
            }
            zs[i] = gate;
        }
        __syncthreads();
#pragma unroll 2
        for (int r = 0; r < nt; r++) {
            const float* kr = ks + r * N;
            const float* qr = qs + r * N;
            const float uv = us[r * CH + ch];
            const float e0 = decay_mode == 0 ? es[r] : 0.0f;
            float y = 0.0f;
#pragma unroll
            for (int k = 0; k < HS_MAX_PER; k++) {
                const int n = lane + k * LANES;
                if (n < N) {
                    const float e = decay_mode == 0 ? e0 : es[r * N + n];
                    S[k] = fmaf(e, S[k], fmaf(uv, kr[n], S[k]));
                    y = fmaf(S[k], qr[n], y);
                    if (pass == 1) log_sum[k] += decay_mode == 0 ? ls[r] : ls[r * N + n];
                }
            }
            if (pass == 1) continue;
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o, LANES);
            if (lane == 0 && live) out[(size_t)(start + base + r) * ldo + (size_t)h * P + j] = from_f32<TO>(fmaf(y, q_scale, D * uv) * zs[r * CH + ch]);
        }
    }
    if (live && pass != 3) {
#pragma unroll
        for (int k = 0; k < HS_MAX_PER; k++) {
            const int n = lane + k * LANES;
            if (n < N) (pass == 0 ? srow : carry_L + carry_at * N)[n] = S[k];
        }
    }
    if (pass == 1 && blockIdx.x == 0 && ch == 0) {
        // the chunk's sum of logarithms: one value per head (mode 0) or per state index (mode 1)
        if (decay_mode == 0) {
            if (lane == 0) carry_log[carry_log_at] = log_sum[0];
        } else {
#pragma unroll
            for (int k = 0; k < HS_MAX_PER; k++) {
                const int n = lane + k * LANES;
                if (n < N) carry_log[carry_log_at + n] = log_sum[k];
            }
        }
    }
}

// S_start of every chunk and the sequence's new state: one thread per (sequence, head, channel, state index)
__global__ void __launch_bounds__(256)
head_scan_carry_kernel(const float* __restrict__ carry_L, const float* __restrict__ carry_log, float* __restrict__ carry_S0,
                       float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
                       const int* __restrict__ seq_start, int H, int P, int N, int decay_mode, int chunk_len, int max_chunks) {
    pdl_trigger();
    pdl_wait();
    carry_L = pdl_fresh(carry_L);
    carry_log = pdl_fresh(carry_log);
    state = pdl_fresh(state);
    const int b = blockIdx.y;
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    const long long per = (long long)H * P * N;
    if (i >= per) return;
    const int n = (int)(i % N), h = (int)(i / ((long long)P * N));
    const int chunks = (seq_start[b + 1] - seq_start[b] + chunk_len - 1) / chunk_len;
    const int LW = decay_mode ? N : 1;
    float* sp = state + (size_t)state_slots[b] * state_stride + i;
    float S = *sp;
    for (int c = 0; c < chunks; c++) {
        const size_t at = (size_t)b * max_chunks + c;
        carry_S0[at * per + i] = S;
        const float lg = carry_log[(at * H + h) * LW + (decay_mode ? n : 0)];
        S = fmaf(expm1f(lg), S, S) + carry_L[at * per + i];
    }
    *sp = S;
}

static int hs_lanes(int N, long long blocks_at_4) {
    int full = N <= 4 ? 4 : N <= 8 ? 8 : N <= 16 ? 16 : 32;
    int lanes = full / 4 < 4 ? 4 : full / 4;
    while (lanes * HS_MAX_PER < N) lanes *= 2;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, hb_device_slot());
    // more lanes per channel (fewer channels per block, more blocks) while the grid has fewer than two blocks per SM
    while (lanes < full && blocks_at_4 * lanes / 4 < 2 * sms) lanes *= 2;
    return lanes;
}

extern "C" int hb_head_scan(const float* u, long long ldu, const float* kmat, long long ldk, const float* qmat, long long ldq,
                            const float* z, long long ldz, const float* draw, long long ldd, const float* dbias, const float* a_log,
                            float inv_tau, const float* dskip, float q_scale, float* state, long long state_stride,
                            const int* state_slots, const int* seq_start, void* out, int out_dtype, long long ldo, int n_seqs,
                            int n_heads, int n_groups, int head_dim, int n_state, int decay_mode, int chunk_len, int max_chunks,
                            float* carry, long long carry_floats, void* stream) {
    if (n_seqs == 0) return 0;
    const int H = n_heads, G = n_groups, P = head_dim, N = n_state;
    HB_REQUIRE(n_seqs > 0 && H > 0 && G > 0 && P > 0 && N > 0 && H % G == 0 && H <= 65535, "head_scan: bad sizes");
    HB_REQUIRE(N <= HS_MAX_PER * 32, "head_scan: state size %d (up to %d is built)", N, HS_MAX_PER * 32);
    HB_REQUIRE(decay_mode == 0 || decay_mode == 1, "head_scan: decay mode %d (0 scalar per head, 1 per state index)", decay_mode);
    HB_REQUIRE(draw != nullptr && dbias != nullptr && (decay_mode == 1 || a_log != nullptr), "head_scan: the decay's inputs are missing");
    HB_REQUIRE(ldu >= (long long)H * P && ldk >= (long long)G * N && ldq >= (long long)G * N && ldo >= (long long)H * P &&
               (z == nullptr || ldz >= (long long)H * P) && ldd >= (decay_mode ? (long long)H * N : (long long)H) &&
               state_stride >= (long long)H * P * N, "head_scan: rows are too short");
    HB_REQUIRE(out_dtype == HB_BF16 || out_dtype == HB_F32, "head_scan: unsupported output dtype %d", out_dtype);
    const long long per = (long long)n_seqs * max_chunks * H * P * N;
    const long long logs = (long long)n_seqs * max_chunks * H * (decay_mode ? N : 1);
    HB_REQUIRE(chunk_len == 0 || (chunk_len > 0 && max_chunks > 0 && (long long)n_seqs * max_chunks <= 65535 && carry != nullptr &&
                                  carry_floats >= 2 * per + logs), "head_scan: chunks need their carry buffer");
    float* carry_L = carry;
    float* carry_S0 = carry ? carry + per : nullptr;
    float* carry_log = carry ? carry + 2 * per : nullptr;
    const long long grids = (long long)n_seqs * (chunk_len ? max_chunks : 1) * H;
    const int lanes = hs_lanes(N, (long long)((P + HS_THREADS / 4 - 1) / (HS_THREADS / 4)) * grids), ch = HS_THREADS / lanes;
    const size_t smem = sizeof(float) * ((size_t)HS_TOK * (2 * N + 2 * (decay_mode ? N : 1) + 2 * ch + 1));
    HB_REQUIRE(smem <= 200 * 1024, "head_scan: state size %d needs too much shared memory", N);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_HS(TO, L, PASS)                                                                                                              \
    {                                                                                                                                   \
        if (smem > 48 * 1024) {                                                                                                         \
            static bool done[HB_MAX_DEVICES] = {};                                                                                      \
            const int slot = hb_device_slot();                                                                                          \
            if (!done[slot]) {                                                                                                          \
                cudaError_t e = cudaFuncSetAttribute(head_scan_kernel<TO, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);  \
                if (e != cudaSuccess) return hb_fail("head_scan: shared memory: %s", cudaGetErrorString(e));                            \
                done[slot] = true;                                                                                                      \
            }                                                                                                                           \
        }                                                                                                                               \
        hb_launch(head_scan_kernel<TO, L>, dim3((P + ch - 1) / ch, H, n_seqs * (PASS == 0 ? 1 : max_chunks)), dim3(HS_THREADS), smem, s, \
                  u, ldu, kmat, ldk, qmat, ldq, z, ldz, draw, ldd, dbias, a_log, inv_tau, dskip, q_scale, state, state_stride,           \
                  state_slots, seq_start, (TO*)out, ldo, H, G, P, N, decay_mode, PASS, chunk_len, max_chunks, carry_L, carry_log,        \
                  (const float*)carry_S0);                                                                                              \
    }
#define HB_HS_L(TO, PASS)                                \
    switch (lanes) {                                     \
        case 4: HB_HS(TO, 4, PASS) break;                \
        case 8: HB_HS(TO, 8, PASS) break;                \
        case 16: HB_HS(TO, 16, PASS) break;              \
        default: HB_HS(TO, 32, PASS) break;              \
    }
#define HB_HS_P(PASS)                                                              \
    do {                                                                           \
        if (out_dtype == HB_BF16) { HB_HS_L(bf16, PASS) } else { HB_HS_L(float, PASS) } \
    } while (0)
    if (chunk_len == 0) {
        HB_HS_P(0);
        return hb_check_launch("head_scan");
    }
    HB_HS_P(1);
    if (hb_check_launch("head_scan (chunks from zero)")) return 1;
    const long long elems = (long long)H * P * N;
    hb_launch(head_scan_carry_kernel, dim3((unsigned)((elems + 255) / 256), n_seqs), dim3(256), 0, s, (const float*)carry_L,
              (const float*)carry_log, carry_S0, state, state_stride, state_slots, seq_start, H, P, N, decay_mode, chunk_len, max_chunks);
    if (hb_check_launch("head_scan_carry")) return 1;
    HB_HS_P(3);
#undef HB_HS_P
#undef HB_HS_L
#undef HB_HS
    return hb_check_launch("head_scan (chunks with outputs)");
}
