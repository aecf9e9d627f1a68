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
// A group of LANES threads owns a value channel (each PER consecutive state indices, in registers); a block owns CH = 256 /
// LANES channels of ONE head of one sequence and walks its tokens in order, HS_TOK tokens of inputs staged in shared memory
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
#define HS_PAD 4            // floats between two lanes' runs of a staged row: the lanes' 16-byte loads then hit different banks

__device__ __forceinline__ float hs_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// LANES threads own a value channel; each holds PER consecutive state indices (n = lane * PER + k) in registers, so that the
// staged k, q and decay rows are read by 16-byte loads and the sum over n needs log2(LANES) shuffles per token.  Rows are
// staged with zeros behind index N: the walk has no bounds checks.
template <typename TO, int LANES, int PER>
__global__ void __launch_bounds__(HS_THREADS, PER <= 8 ? 4 : 2)
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
    constexpr int CH = HS_THREADS / LANES, RS = LANES * (PER + HS_PAD), NP = LANES * PER;
    constexpr int HS_STAGE = PER <= 8 ? 4 : 8;     // loads of k, q and decay inputs a thread issues before it uses the first
    extern __shared__ __align__(16) float hs_smem[];
    const int EW = decay_mode ? RS : 4;            // floats per token of the decay rows
    float* ks = hs_smem;                           // [HS_TOK][RS]: s * k
    float* qs = ks + HS_TOK * RS;                  // [HS_TOK][RS]
    float* es = qs + HS_TOK * RS;                  // [HS_TOK][EW]: a - 1 (mode 0: one value per token, at [r * 4])
    float* us = es + HS_TOK * EW;                  // [HS_TOK][CH]
    float* zs = us + HS_TOK * CH;                  // [HS_TOK][CH]: silu(z), or 1
    float* ls = zs + HS_TOK * CH;                  // [HS_TOK][NP or 1]: the decays' logarithms (pass 1 sums them)
    float* ds = ls + HS_TOK * (decay_mode ? NP : 1);   // [HS_TOK]: the step sizes (mode 0)
    float* lsum = ds + HS_TOK;                     // [NP or 1]: pass 1, the chunk's sum of logarithms
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
    const size_t carry_log_at = (((size_t)b * max_chunks + chunk) * H + h) * (size_t)LW;
    const bool sums_logs = pass == 1 && blockIdx.x == 0;
    pdl_wait();
    u = pdl_fresh(u);
    kmat = pdl_fresh(kmat);
    qmat = pdl_fresh(qmat);
    z = pdl_fresh(z);
    draw = pdl_fresh(draw);
    state = pdl_fresh(state);
    carry_S0 = pdl_fresh(carry_S0);
    // The block's channels' states are one contiguous run of memory: it is read (and at the end written) by consecutive
    // threads through shared memory (one float of padding per 32, so that the owners' reads hit different banks), since a
    // thread's own PER values lie PER floats apart from its neighbour's.
    const int j0 = blockIdx.x * CH, n_mine = min(CH, P - j0) * N;
    float* sblock = state + (size_t)state_slots[b] * state_stride + ((size_t)h * P + j0) * N;
    const size_t carry_block = ((((size_t)b * max_chunks + chunk) * H + h) * (size_t)P + j0) * N;
    float S[PER];
    if (pass != 1) {
        const float* src = pass == 0 ? sblock : carry_S0 + carry_block;
        if ((N & 3) == 0 && ((uintptr_t)src & 15) == 0) {
            // 16-byte loads, eight of a thread in flight before the first is stored
            const float4* src4 = reinterpret_cast<const float4*>(src);
            const int n4 = n_mine >> 2;
            for (int base4 = tid; base4 < n4; base4 += HS_THREADS * 8) {
                float4 v[8];
#pragma unroll
                for (int q8 = 0; q8 < 8; q8++) {
                    const int i4 = base4 + q8 * HS_THREADS;
                    v[q8] = i4 < n4 ? src4[i4] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
#pragma unroll
                for (int q8 = 0; q8 < 8; q8++) {
                    const int i4 = base4 + q8 * HS_THREADS, i = i4 << 2, at = i + (i >> 5);      // four values never straddle a pad
                    if (i4 < n4) {
                        hs_smem[at] = v[q8].x;
                        hs_smem[at + 1] = v[q8].y;
                        hs_smem[at + 2] = v[q8].z;
                        hs_smem[at + 3] = v[q8].w;
                    }
                }
            }
        } else {
            for (int i = tid; i < n_mine; i += HS_THREADS) hs_smem[i + (i >> 5)] = src[i];
        }
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < PER; k++) {
        const int n = lane * PER + k, i = ch * N + n;
        S[k] = (live && n < N && pass != 1) ? hs_smem[i + (i >> 5)] : 0.0f;
    }
    if (sums_logs)
        for (int i = tid; i < LW; i += HS_THREADS) lsum[i] = 0.0f;
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
                es[i * 4] = expm1f(lg);
            }
            __syncthreads();
        }
        // the tokens' k, q and decay inputs: HS_STAGE loads of a thread in flight before the first is used
        for (int i0 = tid; i0 < nt * NP; i0 += HS_THREADS * HS_STAGE) {
            float kv[HS_STAGE], qv[HS_STAGE], dr[HS_STAGE];
#pragma unroll
            for (int s8 = 0; s8 < HS_STAGE; s8++) {
                const int i = i0 + s8 * HS_THREADS, r = i / NP, n = i - r * NP;
                kv[s8] = qv[s8] = dr[s8] = 0.0f;
                if (i < nt * NP && n < N) {
                    const size_t t = (size_t)(start + base + r);
                    kv[s8] = kmat[t * ldk + (size_t)g * N + n];
                    qv[s8] = qmat[t * ldq + (size_t)g * N + n];
                    if (decay_mode) dr[s8] = draw[t * ldd + (size_t)h * N + n] + dbias[(size_t)h * N + n];
                }
            }
#pragma unroll
            for (int s8 = 0; s8 < HS_STAGE; s8++) {
                const int i = i0 + s8 * HS_THREADS, r = i / NP, n = i - r * NP;
                if (i >= nt * NP) break;
                const int at = r * RS + (n / PER) * (PER + HS_PAD) + n % PER;
                if (decay_mode == 0) {
                    kv[s8] *= ds[r];
                } else {
                    const float lg = n < N ? -hs_softplus(-dr[s8]) * inv_tau : 0.0f;      // log(sigmoid) / tau
                    ls[i] = lg;
                    es[at] = expm1f(lg);
                }
                ks[at] = kv[s8];
                qs[at] = qv[s8];
            }
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
        if (sums_logs)
            for (int i = tid; i < LW; i += HS_THREADS) {
                float a = lsum[i];
                for (int r = 0; r < nt; r++) a += ls[decay_mode ? r * NP + i : r];
                lsum[i] = a;
            }
        const int seg = lane * (PER + HS_PAD);
#pragma unroll(PER >= 16 ? 1 : 2)
        for (int r = 0; r < nt; r++) {
            const float4* kr = reinterpret_cast<const float4*>(ks + r * RS + seg);
            const float4* qr = reinterpret_cast<const float4*>(qs + r * RS + seg);
            const float4* er = reinterpret_cast<const float4*>(es + r * EW + (decay_mode ? seg : 0));
            const float uv = us[r * CH + ch];
            const float e0 = er[0].x;
            float y = 0.0f;
#pragma unroll
            for (int k4 = 0; k4 < PER / 4; k4++) {
                const float4 kk = kr[k4], qq = qr[k4];
                float4 ee = make_float4(e0, e0, e0, e0);
                if (decay_mode) ee = er[k4];
                S[4 * k4 + 0] = fmaf(ee.x, S[4 * k4 + 0], fmaf(uv, kk.x, S[4 * k4 + 0]));
                S[4 * k4 + 1] = fmaf(ee.y, S[4 * k4 + 1], fmaf(uv, kk.y, S[4 * k4 + 1]));
                S[4 * k4 + 2] = fmaf(ee.z, S[4 * k4 + 2], fmaf(uv, kk.z, S[4 * k4 + 2]));
                S[4 * k4 + 3] = fmaf(ee.w, S[4 * k4 + 3], fmaf(uv, kk.w, S[4 * k4 + 3]));
                y = fmaf(S[4 * k4 + 0], qq.x, y);
                y = fmaf(S[4 * k4 + 1], qq.y, y);
                y = fmaf(S[4 * k4 + 2], qq.z, y);
                y = fmaf(S[4 * k4 + 3], qq.w, y);
            }
            if (pass == 1) continue;
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o, LANES);
            if (lane == 0 && live) out[(size_t)(start + base + r) * ldo + (size_t)h * P + j] = from_f32<TO>(fmaf(y, q_scale, D * uv) * zs[r * CH + ch]);
        }
    }
    if (pass != 3) {
        __syncthreads();                               // the last tokens' staged rows have been read
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int n = lane * PER + k, i = ch * N + n;
            if (live && n < N) hs_smem[i + (i >> 5)] = S[k];
        }
        __syncthreads();
        float* dst = pass == 0 ? sblock : carry_L + carry_block;
        if ((N & 3) == 0 && ((uintptr_t)dst & 15) == 0) {
            for (int i4 = tid; i4 < (n_mine >> 2); i4 += HS_THREADS) {
                const int i = i4 << 2, at = i + (i >> 5);
                reinterpret_cast<float4*>(dst)[i4] = make_float4(hs_smem[at], hs_smem[at + 1], hs_smem[at + 2], hs_smem[at + 3]);
            }
        } else {
            for (int i = tid; i < n_mine; i += HS_THREADS) dst[i] = hs_smem[i + (i >> 5)];
        }
    }
    if (sums_logs) {
        __syncthreads();
        for (int i = tid; i < LW; i += HS_THREADS) carry_log[carry_log_at + i] = lsum[i];
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

// State indices a thread holds (PER) and threads per channel (LANES), LANES * PER >= N: as many indices per thread as the
// state allows (fewer loads and shuffles per update), but fewer (more threads and blocks) while the grid would leave SMs idle.
static void hs_shape(int N, int P, long long grids, int& lanes, int& per) {
    per = N <= 16 ? 4 : N <= 32 ? 8 : N <= 64 ? 16 : 32;
    lanes = 4;
    while (lanes * per < N) lanes *= 2;                       // N up to 256: 8 x 32
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, hb_device_slot());
    while (per > 4 && lanes < 16 && (long long)((P + HS_THREADS / lanes - 1) / (HS_THREADS / lanes)) * grids < 2 * sms) {
        per /= 2;
        lanes *= 2;
    }
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
    HB_REQUIRE(N <= 256, "head_scan: state size %d (up to 256 is built)", N);
    HB_REQUIRE(decay_mode == 0 || decay_mode == 1, "head_scan: decay mode %d (0 scalar per head, 1 per state index)", decay_mode);
    HB_REQUIRE(draw != nullptr && dbias != nullptr && (decay_mode == 1 || a_log != nullptr), "head_scan: the decay's inputs are missing");
    HB_REQUIRE(ldu >= (long long)H * P && ldk >= (long long)G * N && ldq >= (long long)G * N && ldo >= (long long)H * P &&
               (z == nullptr || ldz >= (long long)H * P) && ldd >= (decay_mode ? (long long)H * N : (long long)H) &&
               state_stride >= (long long)H * P * N, "head_scan: rows are too short");
    HB_REQUIRE(out_dtype == HB_BF16 || out_dtype == HB_F32, "head_scan: unsupported output dtype %d", out_dtype);
    const long long all_states = (long long)n_seqs * max_chunks * H * P * N;
    const long long logs = (long long)n_seqs * max_chunks * H * (decay_mode ? N : 1);
    HB_REQUIRE(chunk_len == 0 || (chunk_len > 0 && max_chunks > 0 && (long long)n_seqs * max_chunks <= 65535 && carry != nullptr &&
                                  carry_floats >= 2 * all_states + logs), "head_scan: chunks need their carry buffer");
    float* carry_L = carry;
    float* carry_S0 = carry ? carry + all_states : nullptr;
    float* carry_log = carry ? carry + 2 * all_states : nullptr;
    const long long grids = (long long)n_seqs * (chunk_len ? max_chunks : 1) * H;
    int lanes = 4, per = 4;
    hs_shape(N, P, grids, lanes, per);
    const int ch = HS_THREADS / lanes, rs = lanes * (per + HS_PAD), np = lanes * per;
    const size_t smem = sizeof(float) * ((size_t)HS_TOK * (2 * rs + (decay_mode ? rs + np : 4 + 1) + 2 * ch + 1) + (decay_mode ? np : 1));
    HB_REQUIRE(smem <= 200 * 1024, "head_scan: state size %d needs too much shared memory", N);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_HS(TO, L, PER, PASS)                                                                                                         \
    {                                                                                                                                   \
        if (smem > 48 * 1024) {                                                                                                         \
            static bool done[HB_MAX_DEVICES] = {};                                                                                      \
            const int slot = hb_device_slot();                                                                                          \
            if (!done[slot]) {                                                                                                          \
                cudaError_t e = cudaFuncSetAttribute(head_scan_kernel<TO, L, PER>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
                if (e != cudaSuccess) return hb_fail("head_scan: shared memory: %s", cudaGetErrorString(e));                            \
                done[slot] = true;                                                                                                      \
            }                                                                                                                           \
        }                                                                                                                               \
        hb_launch(head_scan_kernel<TO, L, PER>, dim3((P + ch - 1) / ch, H, n_seqs * (PASS == 0 ? 1 : max_chunks)), dim3(HS_THREADS), smem, s, \
                  u, ldu, kmat, ldk, qmat, ldq, z, ldz, draw, ldd, dbias, a_log, inv_tau, dskip, q_scale, state, state_stride,           \
                  state_slots, seq_start, (TO*)out, ldo, H, G, P, N, decay_mode, PASS, chunk_len, max_chunks, carry_L, carry_log,        \
                  (const float*)carry_S0);                                                                                              \
    }
#define HB_HS_R(TO, L, PASS)                             \
    switch (per) {                                       \
        case 4: HB_HS(TO, L, 4, PASS) break;             \
        case 8: HB_HS(TO, L, 8, PASS) break;             \
        case 16: HB_HS(TO, L, 16, PASS) break;           \
        default: HB_HS(TO, L, 32, PASS) break;           \
    }
#define HB_HS_L(TO, PASS)                                \
    switch (lanes) {                                     \
        case 4: HB_HS_R(TO, 4, PASS) break;              \
        case 8: HB_HS_R(TO, 8, PASS) break;              \
        default: HB_HS_R(TO, 16, PASS) break;            \
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
#undef HB_HS_R
#undef HB_HS
    return hb_check_launch("head_scan (chunks with outputs)");
}
