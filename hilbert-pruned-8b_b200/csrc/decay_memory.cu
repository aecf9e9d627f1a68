// A matrix memory with a fixed decay per head (linear attention with exponential forgetting):
//   S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t        (S: head size x value size, 32-bit)
// with q, k, v = act(projections), act = silu or nothing; optionally q and k are then turned by the step's
// rotation table (pairs (i, i + rot/2) of the first rot dimensions of every head) and k is multiplied by a
// constant.  The state is carried per sequence.
//
// decay_memory: DM_CHUNK tokens at a time.  Within a chunk that starts from S0 (tokens j, s = 0 ..):
//   o_j = decay^(j+1) S0^T q_j + sum_{s <= j} decay^(j-s) (q_j . k_s) v_s
//   S'  = decay^n S0 + sum_s decay^(n-1-s) k_s v_s^T                        (n tokens in the chunk)
// so one pass over the state serves up to DM_CHUNK tokens; a chunk of one token is the recurrence
// itself (decode steps).  Only non-negative powers of the decay appear, nothing is divided.  One
// block per (slice of DM_COLS value columns, head, sequence), everything in 32-bit FP32-pipe code.
//
// gated_norm: out = o / sqrt(mean(o^2) + eps) * w * f(gate) * out_scale, the mean taken over each row (all
// heads together) or over each run of `group` values of it (a head at a time); w may be absent, f is
// sigmoid or silu; rounded once for the output product.
#include "api.h"
#include "common.cuh"

#define DM_THREADS 256
#define DM_CHUNK 32
#define DM_COLS 16           // value columns a block owns: narrow slices, so that one sequence's heads fill the device
#define DM_GROUPS (DM_THREADS / DM_COLS)
#define DM_MAX_DIM 256

static size_t dm_smem_bytes(int d) {
    // q, k [chunk][d + 1]; v [chunk][cols]; a [chunk][chunk + 1]; S [d][cols]; powers [chunk + 1]
    return sizeof(float) * ((size_t)2 * DM_CHUNK * (d + 1) + DM_CHUNK * DM_COLS + DM_CHUNK * (DM_CHUNK + 1) + (size_t)d * DM_COLS + DM_CHUNK + 1);
}

__device__ __forceinline__ float dm_act(float z, int act) { return act == 1 ? z / (1.0f + expf(-z)) : z; }

__global__ void __launch_bounds__(DM_THREADS)
decay_memory_kernel(const float* __restrict__ proj, long long ldp, const float* __restrict__ decay, float* __restrict__ state,
                    long long state_stride, const int* __restrict__ state_slots, const int* __restrict__ seq_start,
                    float* __restrict__ out, long long ldo, int H, int d, int dv, int act, const float2* __restrict__ table, int rot,
                    float k_scale) {
    pdl_trigger();
    extern __shared__ float dm_smem[];
    float* Qs = dm_smem;
    float* Ks = Qs + DM_CHUNK * (d + 1);
    float* Vs = Ks + DM_CHUNK * (d + 1);
    float* As = Vs + DM_CHUNK * DM_COLS;
    float* Ss = As + DM_CHUNK * (DM_CHUNK + 1);
    float* pw = Ss + d * DM_COLS;
    const int tid = threadIdx.x, c0 = blockIdx.x * DM_COLS, h = blockIdx.y, b = blockIdx.z;
    const int lane = tid % DM_COLS, grp = tid / DM_COLS;   // column lane, DM_GROUPS groups
    const int col = c0 + lane;
    const bool live = col < dv;
    const int start = seq_start[b], n_all = seq_start[b + 1] - start;
    const double lam = (double)decay[h];
    if (tid <= DM_CHUNK) pw[tid] = (float)pow(lam, (double)tid);
    pdl_wait();
    proj = pdl_fresh(proj);
    state = pdl_fresh(state);
    table = pdl_fresh(table);
    float* S = state + (size_t)state_slots[b] * state_stride + (size_t)h * d * dv;
    for (int i = grp; i < d; i += DM_GROUPS) Ss[i * DM_COLS + lane] = live ? S[(size_t)i * dv + col] : 0.0f;
    const long long qo = (long long)h * d, ko = (long long)H * d + (long long)h * d, vo = (long long)2 * H * d + (long long)h * dv;
    for (int base = 0; base < n_all; base += DM_CHUNK) {
        const int n = min(DM_CHUNK, n_all - base);
        __syncthreads();                               // the chunk before has been read; the state is in place
        if (((d | dv | c0) & 3) == 0 && (ldp & 3) == 0 && ((qo | ko | vo) & 3) == 0 && ((uintptr_t)proj & 15) == 0) {
            // 16-byte loads, all of a thread's loads in flight before the first activation
            const int cpr = d / 4, total = 2 * n * cpr;                     // q chunks, then k chunks
            for (int base0 = 0; base0 < total; base0 += DM_THREADS * 4) {
                float4 raw[4];
                int at[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int i = base0 + u * DM_THREADS + tid;
                    at[u] = -1;
                    if (i < total) {
                        const int which = i >= n * cpr, r = i - which * n * cpr;
                        const int j = r / cpr, ch = r - j * cpr;
                        raw[u] = *reinterpret_cast<const float4*>(proj + (size_t)(start + base + j) * ldp + (which ? ko : qo) + ch * 4);
                        at[u] = which * DM_CHUNK * (d + 1) + j * (d + 1) + ch * 4;
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (at[u] < 0) continue;
                    float* dst = Qs + at[u];                                // Ks follows Qs
                    dst[0] = dm_act(raw[u].x, act);
                    dst[1] = dm_act(raw[u].y, act);
                    dst[2] = dm_act(raw[u].z, act);
                    dst[3] = dm_act(raw[u].w, act);
                }
            }
            const int wv = min(DM_COLS, dv - c0) / 4;                       // whole chunks of this slice's value columns
            for (int i = tid; i < n * (DM_COLS / 4); i += DM_THREADS) {
                const int j = i / (DM_COLS / 4), ch = i - j * (DM_COLS / 4);
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (ch < wv) v = *reinterpret_cast<const float4*>(proj + (size_t)(start + base + j) * ldp + vo + c0 + ch * 4);
                float* dst = Vs + j * DM_COLS + ch * 4;
                dst[0] = ch < wv ? dm_act(v.x, act) : 0.0f;
                dst[1] = ch < wv ? dm_act(v.y, act) : 0.0f;
                dst[2] = ch < wv ? dm_act(v.z, act) : 0.0f;
                dst[3] = ch < wv ? dm_act(v.w, act) : 0.0f;
            }
        } else {
            for (int i = tid; i < n * d; i += DM_THREADS) {
                const int j = i / d, c = i - j * d;
                const float* row = proj + (size_t)(start + base + j) * ldp;
                Qs[j * (d + 1) + c] = dm_act(row[qo + c], act);
                Ks[j * (d + 1) + c] = dm_act(row[ko + c], act);
            }
            for (int i = tid; i < n * DM_COLS; i += DM_THREADS) {
                const int j = i / DM_COLS, c = i % DM_COLS;
                Vs[i] = (c0 + c < dv) ? dm_act(proj[(size_t)(start + base + j) * ldp + vo + c0 + c], act) : 0.0f;
            }
        }
        if (rot > 0 || k_scale != 1.0f) {
            // the staged queries and keys turned in place by their tokens' angles; the keys scaled
            __syncthreads();
            const int half = rot >> 1;
            for (int i = tid; i < n * half; i += DM_THREADS) {
                const int j = i / half, c = i - j * half;
                const float2 cs = table[(size_t)(start + base + j) * half + c];
                float* qr = Qs + j * (d + 1);
                float* kr = Ks + j * (d + 1);
                float y1, y2;
                rope_pair(qr[c], qr[c + half], cs.x, cs.y, y1, y2);
                qr[c] = y1;
                qr[c + half] = y2;
                rope_pair(kr[c], kr[c + half], cs.x, cs.y, y1, y2);
                kr[c] = y1;
                kr[c + half] = y2;
            }
            if (k_scale != 1.0f) {
                __syncthreads();
                for (int i = tid; i < n * d; i += DM_THREADS) Ks[(i / d) * (d + 1) + i % d] *= k_scale;
            }
        }
        __syncthreads();
        // a[j][s] = decay^(j-s) q_j . k_s for s <= j
        for (int i = tid; i < n * n; i += DM_THREADS) {
            const int j = i / n, s = i - j * n;
            float a = 0.0f;
            if (s <= j) {
                const float* qr = Qs + j * (d + 1);
                const float* kr = Ks + s * (d + 1);
                float dot = 0.0f;
                for (int c = 0; c < d; c++) dot = fmaf(qr[c], kr[c], dot);
                a = dot * pw[j - s];
            }
            As[j * (DM_CHUNK + 1) + s] = a;
        }
        __syncthreads();
        // o[j][col]: tokens j = grp, grp + DM_GROUPS, ...
        for (int j = grp; j < n; j += DM_GROUPS) {
            const float* qr = Qs + j * (d + 1);
            float from_state = 0.0f;
            for (int i = 0; i < d; i++) from_state = fmaf(Ss[i * DM_COLS + lane], qr[i], from_state);
            float o = from_state * pw[j + 1];
            const float* ar = As + j * (DM_CHUNK + 1);
            for (int s = 0; s <= j; s++) o = fmaf(ar[s], Vs[s * DM_COLS + lane], o);
            if (live) out[(size_t)(start + base + j) * ldo + (size_t)h * dv + col] = o;
        }
        __syncthreads();                               // every reader of the old state is done
        // S[i][col] = decay^n S[i][col] + sum_s decay^(n-1-s) k_s[i] v_s[col]: rows i = grp, grp + DM_GROUPS, ...
        for (int i = grp; i < d; i += DM_GROUPS) {
            float acc = Ss[i * DM_COLS + lane] * pw[n];
            for (int s = 0; s < n; s++) acc = fmaf(Ks[s * (d + 1) + i] * pw[n - 1 - s], Vs[s * DM_COLS + lane], acc);
            Ss[i * DM_COLS + lane] = acc;
        }
    }
    __syncthreads();
    if (live)
        for (int i = grp; i < d; i += DM_GROUPS) S[(size_t)i * dv + col] = Ss[i * DM_COLS + lane];
}

extern "C" int hb_decay_memory(const float* proj, long long ldp, const float* decay, float* state, long long state_stride,
                               const int* state_slots, const int* seq_start, float* out, long long ldo, int n_seqs, int n_heads,
                               int d, int dv, int act, const float* table, int rot, float k_scale, void* stream) {
    if (n_seqs == 0) return 0;
    HB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_heads > 0 && n_heads <= 65535 && d > 0 && dv > 0, "decay_memory: bad sizes");
    HB_REQUIRE(d <= DM_MAX_DIM, "decay_memory: head size %d (up to %d is built)", d, DM_MAX_DIM);
    HB_REQUIRE(ldp >= (long long)n_heads * (2 * d + dv) && state_stride >= (long long)n_heads * d * dv, "decay_memory: rows are too short");
    HB_REQUIRE(act == 0 || act == 1, "decay_memory: activation %d (0 none, 1 silu)", act);
    HB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= d && (rot == 0 || table != nullptr), "decay_memory: %d rotated dimensions of %d", rot, d);
    static bool done[HB_MAX_DEVICES] = {};
    const int slot = hb_device_slot();
    if (!done[slot]) {
        cudaError_t e = cudaFuncSetAttribute(decay_memory_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dm_smem_bytes(DM_MAX_DIM));
        if (e != cudaSuccess) return hb_fail("decay_memory: shared memory: %s", cudaGetErrorString(e));
        done[slot] = true;
    }
    dim3 grid((dv + DM_COLS - 1) / DM_COLS, n_heads, n_seqs);
    hb_launch(decay_memory_kernel, dim3(grid), dim3(DM_THREADS), dm_smem_bytes(d), (cudaStream_t)stream, proj, ldp, decay, state, state_stride,
              state_slots, seq_start, out, ldo, n_heads, d, dv, act, (const float2*)table, rot, k_scale);
    return hb_check_launch("decay_memory");
}

// ------------------------------------------------------------------------------------------------ gated_norm
__device__ __forceinline__ float gn_gate(float z, int kind) { return kind == 1 ? z / (1.0f + expf(-z)) : 1.0f / (1.0f + expf(-z)); }

template <typename TO>
__global__ void __launch_bounds__(256)
gated_norm_kernel(const float* __restrict__ o, long long ldi, const float* __restrict__ gate, long long ldg,
                  const float* __restrict__ w, float eps, float out_scale, TO* __restrict__ out, long long ldo, int n, int group,
                  int gate_kind) {
    pdl_trigger();
    pdl_wait();
    o = pdl_fresh(o);
    gate = pdl_fresh(gate);
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* r = o + (size_t)t * ldi;
    if (group < n) {
        // a warp per run of `group` values
        const int lane = threadIdx.x & 31;
        for (int g = threadIdx.x >> 5; g * group < n; g += 8) {
            const float* rg = r + (size_t)g * group;
            float ss = 0.0f;
            for (int i = lane; i < group; i += 32) ss = fmaf(rg[i], rg[i], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)group + eps);
            for (int i = lane; i < group; i += 32) {
                const int e = g * group + i;
                float v = rg[i] * inv * (w ? w[e] : 1.0f);
                if (gate != nullptr) v *= gn_gate(gate[(size_t)t * ldg + e], gate_kind);
                out[(size_t)t * ldo + e] = from_f32<TO>(v * out_scale);
            }
        }
        return;
    }
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) ss = fmaf(r[i], r[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        float v = r[i] * inv * (w ? w[i] : 1.0f);
        if (gate != nullptr) v *= gn_gate(gate[(size_t)t * ldg + i], gate_kind);
        out[(size_t)t * ldo + i] = from_f32<TO>(v * out_scale);
    }
}

extern "C" int hb_gated_norm(const float* o, long long ldi, const float* gate, long long ldg, const float* w, float eps, float out_scale,
                             void* out, int out_dtype, long long ldo, int n_rows, int n, int group, int gate_kind, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n > 0 && ldi >= n && ldo >= n, "gated_norm: bad sizes");
    HB_REQUIRE(group > 0 && n % group == 0, "gated_norm: runs of %d values do not divide a row of %d", group, n);
    HB_REQUIRE(gate_kind == 0 || gate_kind == 1, "gated_norm: gate %d (0 sigmoid, 1 silu)", gate_kind);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16)
        hb_launch(gated_norm_kernel<bf16>, dim3(n_rows), dim3(256), 0, s, o, ldi, gate, ldg, w, eps, out_scale, (bf16*)out, ldo, n, group, gate_kind);
    else if (out_dtype == HB_F32)
        hb_launch(gated_norm_kernel<float>, dim3(n_rows), dim3(256), 0, s, o, ldi, gate, ldg, w, eps, out_scale, (float*)out, ldo, n, group, gate_kind);
    else return hb_fail("gated_norm: unsupported output dtype %d", out_dtype);
    return hb_check_launch("gated_norm");
}
