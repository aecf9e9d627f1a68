// Mixture of experts: router, plan, the experts' products over the tokens routed to them, and
// the weighted sum.
//
// moe_route:  z = Wr h in 32-bit; the `top` largest logits of a token (lowest index on ties) are
//             its experts, their weights softmax over those logits alone.
// moe_plan:   entries (token, k) ordered by expert: offsets[e] .. offsets[e + 1] index `order`, whose
//             values are entry numbers token * top + k; plus the list of (expert, first row) tiles
//             of MOE_BM rows that the two products walk.  One block; the grid of the products is
//             sized for the worst case and blocks beyond the last tile leave at once, so nothing
//             is read back by the host.
// moe_glu:    act[slot] = f(Wg_e h_token, Wu_e h_token) for the rows of an expert's tiles, with
//             f(g, u) = g' sigmoid(alpha g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit).
// moe_down:   down[entry] = Wd_e act[slot] (32-bit), written at the ENTRY's row, so that
// moe_combine: out[token] (+)= sum_k weight[token][k] down[token * top + k], in k order.
// The order of the entries inside an expert's range depends on the atomics of the plan; an entry's
// numbers do not, since every output element is one sequential sum over K.
//
// moe_route_scores: another router.  Scores s = softmax(z) over ALL router outputs; choice scores c = s + correction; the
//             outputs form `groups` equal runs of neighbours, a run's score is its largest c, and only outputs of the `keep`
//             best runs can be chosen; the `top` largest c among those are the token's experts, their weights s (without
//             the correction) divided by their sum (+ norm_eps).  Router outputs from `n_real` on are identity experts: they
//             have no matrices, the plan leaves them out, and moe_combine adds weight * h for them.
// Experts without a gate (moe_glu with w_up null): act = gelu(W_up h), the exact (erf) form.
//
// The products are tiled FP32-pipe kernels (MOE_BM rows x MOE_BN columns x MOE_BK): they serve
// both precisions, with 32-bit accumulation.  glu_clamp is the same activation for a dense
// [gate | up] matrix (a shared expert, whose products are ordinary matrix products).
#include "api.h"
#include "common.cuh"
#include "mma.cuh"

#define MOE_BM 32
#define MOE_BN 32
#define MOE_BK 32
#define MOE_THREADS 256
// the tensor-core variant (bfloat16, rows of a multiple of 8 elements): MM_BM rows x MM_BN columns x MM_BK per stage
#define MM_BM 64
#define MM_BN 64
#define MM_BK 64
#define MM_STAGES 3
#define MM_THREADS 256

// ------------------------------------------------------------------------------------------------ route
template <typename TH>
__global__ void __launch_bounds__(256)
moe_route_kernel(const TH* __restrict__ h, long long ldh, const float* __restrict__ wr, int* __restrict__ experts,
                 float* __restrict__ weights, int W, int E, int top) {
    pdl_trigger();
    pdl_wait();
    h = pdl_fresh(h);
    extern __shared__ float mr_smem[];
    float* hs = mr_smem;             // [W]
    float* zs = hs + W;              // [E]
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < W; i += 256) hs[i] = to_f32(h[(size_t)t * ldh + i]);
    __syncthreads();
    for (int e = warp; e < E; e += 8) {
        const float* w = wr + (size_t)e * W;
        float s = 0.0f;
        for (int i = lane; i < W; i += 32) s = fmaf(w[i], hs[i], s);
        s = warp_sum(s);
        if (lane == 0) zs[e] = s;
    }
    __syncthreads();
    if (warp == 0) {
        // `top` rounds of: the largest logit not yet taken, lowest index on ties
        float zmax = 0.0f, denom = 0.0f;
        for (int k = 0; k < top; k++) {
            float best = -INFINITY;
            int best_e = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float v = zs[e];
                if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
                if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
            }
            if (best_e >= E) best_e = 0;                  // a row of logits that are not numbers: any expert, the result is not finite anyway
            if (k == 0) zmax = best;
            const float p = expf(best - zmax);
            denom += p;
            if (lane == 0) {
                experts[(size_t)t * top + k] = best_e;
                weights[(size_t)t * top + k] = p;
                zs[best_e] = -INFINITY;
            }
            __syncwarp();
        }
        if (lane == 0)
            for (int k = 0; k < top; k++) weights[(size_t)t * top + k] /= denom;
    }
}

extern "C" int hb_moe_route(const void* h, int h_dtype, long long ldh, const float* w_router, int* experts, float* weights,
                            int n_tokens, int width, int n_experts, int top, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && width > 0 && n_experts > 0 && top >= 1 && top <= n_experts, "moe_route: bad sizes");
    const size_t smem = sizeof(float) * ((size_t)width + n_experts);
    HB_REQUIRE(smem <= 48 * 1024, "moe_route: width + experts = %d is too wide", width + n_experts);
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dtype == HB_BF16)
        hb_launch(moe_route_kernel<bf16>, dim3(n_tokens), dim3(256), smem, s, (const bf16*)h, ldh, w_router, experts, weights, width, n_experts, top);
    else if (h_dtype == HB_F32)
        hb_launch(moe_route_kernel<float>, dim3(n_tokens), dim3(256), smem, s, (const float*)h, ldh, w_router, experts, weights, width, n_experts, top);
    else return hb_fail("moe_route: unsupported dtype %d", h_dtype);
    return hb_check_launch("moe_route");
}

template <typename TH>
__global__ void __launch_bounds__(256)
moe_route_scores_kernel(const TH* __restrict__ h, long long ldh, const float* __restrict__ wr, const float* __restrict__ correction,
                        int* __restrict__ experts, float* __restrict__ weights, int W, int E, int top, int groups, int keep,
                        float norm_eps) {
    pdl_trigger();
    pdl_wait();
    h = pdl_fresh(h);
    extern __shared__ float mr_smem[];
    float* hs = mr_smem;             // [W]
    float* ss = hs + W;              // [E]: scores
    float* cs = ss + E;              // [E]: choice scores, minus infinity once taken or shut out
    float* gs = cs + E;              // [groups]: a run's score, minus infinity once kept
    float* kept = gs + groups;       // [groups]: 1 for the runs whose outputs can be chosen
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < W; i += 256) hs[i] = to_f32(h[(size_t)t * ldh + i]);
    __syncthreads();
    for (int e = warp; e < E; e += 8) {
        const float* w = wr + (size_t)e * W;
        float s = 0.0f;
        for (int i = lane; i < W; i += 32) s = fmaf(w[i], hs[i], s);
        s = warp_sum(s);
        if (lane == 0) ss[e] = s;
    }
    __syncthreads();
    if (warp != 0) return;
    // softmax over all outputs
    float zmax = -INFINITY;
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, ss[e]);
    zmax = warp_max(zmax);
    float den = 0.0f;
    for (int e = lane; e < E; e += 32) {
        const float p = expf(ss[e] - zmax);
        ss[e] = p;
        den += p;
    }
    den = warp_sum(den);
    for (int e = lane; e < E; e += 32) {
        ss[e] = ss[e] / den;
        cs[e] = ss[e] + (correction ? correction[e] : 0.0f);
    }
    __syncwarp();
    auto arg_best = [&](const float* v, int n, float& best, int& best_i) {       // the largest, lowest index on ties
        best = -INFINITY;
        best_i = 0x7fffffff;
        for (int e = lane; e < n; e += 32)
            if (v[e] > best || (v[e] == best && e < best_i)) { best = v[e]; best_i = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
        }
    };
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; e++) b = fmaxf(b, cs[e]);
            gs[g] = b;
            kept[g] = 0.0f;
        }
        __syncwarp();
        for (int k = 0; k < keep; k++) {
            float b;
            int bi;
            arg_best(gs, groups, b, bi);
            if (bi >= groups) bi = 0;
            if (lane == 0) { gs[bi] = -INFINITY; kept[bi] = 1.0f; }      // a kept run cannot win again
            __syncwarp();
        }
        // the other runs' outputs are shut out: minus infinity, not zero (choice scores can be negative)
        for (int e = lane; e < E; e += 32)
            if (kept[e / per] == 0.0f) cs[e] = -INFINITY;
        __syncwarp();
    }
    float sum = 0.0f;
    for (int k = 0; k < top; k++) {
        float b;
        int bi;
        arg_best(cs, E, b, bi);
        if (bi >= E) bi = 0;                              // nothing left (or scores that are not numbers): any output
        const float p = ss[bi];
        sum += p;
        if (lane == 0) {
            experts[(size_t)t * top + k] = bi;
            weights[(size_t)t * top + k] = p;
            cs[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0)
        for (int k = 0; k < top; k++) weights[(size_t)t * top + k] /= (sum + norm_eps);
}

extern "C" int hb_moe_route_scores(const void* h, int h_dtype, long long ldh, const float* w_router, const float* correction, int* experts,
                                   float* weights, int n_tokens, int width, int n_outputs, int top, int groups, int keep, float norm_eps,
                                   void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && width > 0 && n_outputs > 0 && top >= 1 && top <= n_outputs, "moe_route_scores: bad sizes");
    HB_REQUIRE(groups >= 1 && n_outputs % groups == 0 && keep >= 1 && keep <= groups,
               "moe_route_scores: %d outputs in %d groups of which %d are kept", n_outputs, groups, keep);
    HB_REQUIRE(top <= (n_outputs / groups) * keep, "moe_route_scores: the kept groups hold fewer than %d outputs", top);
    const size_t smem = sizeof(float) * ((size_t)width + 2 * n_outputs + 2 * groups);
    HB_REQUIRE(smem <= 48 * 1024, "moe_route_scores: width + outputs = %d is too wide", width + n_outputs);
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dtype == HB_BF16)
        hb_launch(moe_route_scores_kernel<bf16>, dim3(n_tokens), dim3(256), smem, s, (const bf16*)h, ldh, w_router, correction, experts, weights,
                  width, n_outputs, top, groups, keep, norm_eps);
    else if (h_dtype == HB_F32)
        hb_launch(moe_route_scores_kernel<float>, dim3(n_tokens), dim3(256), smem, s, (const float*)h, ldh, w_router, correction, experts,
                  weights, width, n_outputs, top, groups, keep, norm_eps);
    else return hb_fail("moe_route_scores: unsupported dtype %d", h_dtype);
    return hb_check_launch("moe_route_scores");
}

// ------------------------------------------------------------------------------------------------ plan
// offsets [E + 1], order [entries], tiles [1 + 2 * max_tiles]: tiles[0] = number of tiles, then (expert, first row) pairs
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ experts, int n_entries, int E, int tile_rows, int* __restrict__ offsets, int* __restrict__ order,
                int* __restrict__ tiles) {
    pdl_trigger();
    pdl_wait();
    experts = pdl_fresh(experts);
    extern __shared__ int mp_smem[];
    int* count = mp_smem;            // [E]
    int* cursor = count + E;         // [E]
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += 1024) count[e] = 0;
    __syncthreads();
    // (an entry whose expert number is E or more belongs to an identity expert: no product walks it)
    for (int i = tid; i < n_entries; i += 1024)
        if (experts[i] < E) atomicAdd(&count[experts[i]], 1);
    __syncthreads();
    if (tid == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E; e++) {
            offsets[e] = at;
            cursor[e] = at;
            for (int r = 0; r < count[e]; r += tile_rows) {
                tiles[1 + 2 * nt] = e;
                tiles[2 + 2 * nt] = at + r;
                nt++;
            }
            at += count[e];
        }
        offsets[E] = at;
        tiles[0] = nt;
    }
    __syncthreads();
    for (int i = tid; i < n_entries; i += 1024)
        if (experts[i] < E) order[atomicAdd(&cursor[experts[i]], 1)] = i;
}

extern "C" int hb_moe_tile_rows(int tensor_cores) { return tensor_cores ? MM_BM : MOE_BM; }

extern "C" int hb_moe_plan(const int* experts, int n_entries, int n_experts, int tile_rows, int* offsets, int* order, int* tiles, void* stream) {
    if (n_entries == 0) return 0;
    HB_REQUIRE(n_entries > 0 && n_experts > 0 && n_experts <= 4096, "moe_plan: bad sizes");
    HB_REQUIRE(tile_rows == MOE_BM || tile_rows == MM_BM, "moe_plan: tiles of %d rows (%d or %d are built)", tile_rows, MOE_BM, MM_BM);
    hb_launch(moe_plan_kernel, dim3(1), dim3(1024), sizeof(int) * 2 * n_experts, (cudaStream_t)stream, experts, n_entries, n_experts, tile_rows,
              offsets, order, tiles);
    return hb_check_launch("moe_plan");
}

extern "C" int hb_moe_max_tiles(int n_entries, int n_experts, int tile_rows) { return (n_entries + tile_rows - 1) / tile_rows + n_experts; }

// ------------------------------------------------------------------------------------------------ the experts' products
__device__ __forceinline__ float moe_gelu_erf(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f)); }
// the first product's epilogue: the clamped gated unit of two matrices (MODE 1), or the exact gelu of one (MODE 2)
template <int MODE>
__device__ __forceinline__ float moe_first_act(float a0, float a1, float limit, float alpha);
__device__ __forceinline__ float moe_glu(float g, float u, float limit, float alpha);
template <> __device__ __forceinline__ float moe_first_act<1>(float a0, float a1, float limit, float alpha) { return moe_glu(a0, a1, limit, alpha); }
template <> __device__ __forceinline__ float moe_first_act<2>(float a0, float a1, float limit, float alpha) { return moe_gelu_erf(a0); }
template <> __device__ __forceinline__ float moe_first_act<0>(float a0, float a1, float limit, float alpha) { return a0; }
__device__ __forceinline__ float moe_glu(float g, float u, float limit, float alpha) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
}

// GLU: a rows are h[token of the entry], two weight matrices [E][N][K], result act[slot][N] in TO.
// else: a rows are act[slot], one weight matrix, result down[entry][N] in 32-bit.
template <typename TA, typename TW, typename TO, int MODE>
__global__ void __launch_bounds__(MOE_THREADS)
moe_product_kernel(const TA* __restrict__ a, long long lda, const TW* __restrict__ w0, const TW* __restrict__ w1,
                   const int* __restrict__ offsets, const int* __restrict__ order, const int* __restrict__ tiles, int top,
                   TO* __restrict__ out, long long ldo, int N, int K, float limit, float alpha) {
    pdl_trigger();
    constexpr bool GLU = MODE == 1, FIRST = MODE != 0;        // FIRST: rows gathered by token, results at the slot
    __shared__ float As[MOE_BK][MOE_BM + 1];
    __shared__ float B0[MOE_BK][MOE_BN + 1];
    __shared__ float B1[GLU ? MOE_BK : 1][MOE_BN + 1];
    __shared__ int row_src[MOE_BM], row_dst[MOE_BM];
    pdl_wait();
    a = pdl_fresh(a);
    tiles = pdl_fresh(tiles);
    order = pdl_fresh(order);
    offsets = pdl_fresh(offsets);
    if ((int)blockIdx.x >= tiles[0]) return;
    const int e = tiles[1 + 2 * blockIdx.x], r0 = tiles[2 + 2 * blockIdx.x];
    const int rows = min(MOE_BM, offsets[e + 1] - r0);
    const int n0 = blockIdx.y * MOE_BN;
    const int tid = threadIdx.x;
    if (tid < MOE_BM) {
        const int entry = tid < rows ? order[r0 + tid] : -1;
        row_src[tid] = entry < 0 ? -1 : (FIRST ? entry / top : r0 + tid);
        row_dst[tid] = entry < 0 ? -1 : (FIRST ? r0 + tid : entry);
    }
    __syncthreads();
    const TW* we0 = w0 + (size_t)e * N * K;
    const TW* we1 = GLU ? w1 + (size_t)e * N * K : nullptr;
    // thread -> rows ty * 2 + {0, 1}, columns tx * 2 + {0, 1}
    const int tx = tid & 15, ty = tid >> 4;
    float acc0[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}}, acc1[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
        for (int i = tid; i < MOE_BM * MOE_BK; i += MOE_THREADS) {
            const int r = i / MOE_BK, k = i - r * MOE_BK;
            const int src = row_src[r];
            As[k][r] = (src >= 0 && k0 + k < K) ? to_f32(a[(size_t)src * lda + k0 + k]) : 0.0f;
        }
        for (int i = tid; i < MOE_BN * MOE_BK; i += MOE_THREADS) {
            const int n = i / MOE_BK, k = i - n * MOE_BK;
            const bool in = n0 + n < N && k0 + k < K;
            B0[k][n] = in ? to_f32(we0[(size_t)(n0 + n) * K + k0 + k]) : 0.0f;
            if (GLU) B1[k][n] = in ? to_f32(we1[(size_t)(n0 + n) * K + k0 + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < MOE_BK; k++) {
            const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
            const float b0 = B0[k][tx * 2], b1 = B0[k][tx * 2 + 1];
            acc0[0][0] = fmaf(a0, b0, acc0[0][0]);
            acc0[0][1] = fmaf(a0, b1, acc0[0][1]);
            acc0[1][0] = fmaf(a1, b0, acc0[1][0]);
            acc0[1][1] = fmaf(a1, b1, acc0[1][1]);
            if (GLU) {
                const float c0 = B1[k][tx * 2], c1 = B1[k][tx * 2 + 1];
                acc1[0][0] = fmaf(a0, c0, acc1[0][0]);
                acc1[0][1] = fmaf(a0, c1, acc1[0][1]);
                acc1[1][0] = fmaf(a1, c0, acc1[1][0]);
                acc1[1][1] = fmaf(a1, c1, acc1[1][1]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int dst = row_dst[ty * 2 + i];
        if (dst < 0) continue;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int n = n0 + tx * 2 + j;
            if (n >= N) continue;
            const float v = moe_first_act<MODE>(acc0[i][j], acc1[i][j], limit, alpha);
            out[(size_t)dst * ldo + n] = from_f32<TO>(v);
        }
    }
}


// The same two products on the tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit accumulators): a block owns a
// plan tile of MM_BM rows and MM_BN output columns; rows (gathered by the plan's order) and weight rows arrive through a
// MM_STAGES-deep cp.async pipeline into XOR-swizzled shared memory and are read with ldmatrix; eight warps as 4 (rows) x 2
// (columns), each 16 rows x 32 columns (and both matrices for the gated unit, whose activation is the epilogue).
template <int MODE, typename TO>
__global__ void __launch_bounds__(MM_THREADS)
moe_product_mma_kernel(const bf16* __restrict__ a, long long lda, const bf16* __restrict__ w0, const bf16* __restrict__ w1,
                       const int* __restrict__ offsets, const int* __restrict__ order, const int* __restrict__ tiles, int top,
                       TO* __restrict__ out, long long ldo, int N, int K, float limit, float alpha) {
    pdl_trigger();
    extern __shared__ __align__(128) unsigned char mm_smem[];
    constexpr bool GLU = MODE == 1, FIRST = MODE != 0;
    constexpr int TILE_BYTES = MM_BM * MM_BK * 2, MATS = GLU ? 3 : 2, STAGE_BYTES = TILE_BYTES * MATS;
    static_assert(MM_BM == MM_BN && MM_BK * 2 == 128, "one tile shape and 128-byte rows for rows and weights");
    __shared__ int row_src[MM_BM], row_dst[MM_BM];
    pdl_wait();
    a = pdl_fresh(a);
    tiles = pdl_fresh(tiles);
    order = pdl_fresh(order);
    offsets = pdl_fresh(offsets);
    if ((int)blockIdx.x >= tiles[0]) return;
    const int e = tiles[1 + 2 * blockIdx.x], r0 = tiles[2 + 2 * blockIdx.x];
    const int rows = min(MM_BM, offsets[e + 1] - r0);
    const int n0 = blockIdx.y * MM_BN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < MM_BM) {
        const int entry = tid < rows ? order[r0 + tid] : -1;
        row_src[tid] = entry < 0 ? -1 : (FIRST ? entry / top : r0 + tid);
        row_dst[tid] = entry < 0 ? -1 : (FIRST ? r0 + tid : entry);
    }
    __syncthreads();
    const bf16* we0 = w0 + (size_t)e * N * K;
    const bf16* we1 = GLU ? w1 + (size_t)e * N * K : nullptr;
    const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(mm_smem);
    const int nk = (K + MM_BK - 1) / MM_BK;

    auto load_stage = [&](int stage, int kb) {
        const uint32_t base = smem0 + stage * STAGE_BYTES;
        unsigned char* gbase = mm_smem + stage * STAGE_BYTES;
        for (int i = tid; i < MM_BM * 8; i += MM_THREADS) {
            const int row = i >> 3, ch = i & 7;
            const int k = kb * MM_BK + ch * 8;
            const uint32_t off = swizzled<128>(row, ch);
            const int src = row_src[row];
            if (src >= 0 && k < K) cp_async_16(base + off, a + (size_t)src * lda + k);
            else *reinterpret_cast<uint4*>(gbase + off) = make_uint4(0u, 0u, 0u, 0u);
            const int n = n0 + row;
            if (n < N && k < K) {
                cp_async_16(base + TILE_BYTES + off, we0 + (size_t)n * K + k);
                if (GLU) cp_async_16(base + 2 * TILE_BYTES + off, we1 + (size_t)n * K + k);
            } else {
                *reinterpret_cast<uint4*>(gbase + TILE_BYTES + off) = make_uint4(0u, 0u, 0u, 0u);
                if (GLU) *reinterpret_cast<uint4*>(gbase + 2 * TILE_BYTES + off) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };

    const int wm = warp & 3, wn = warp >> 2;
    float acc0[4][4], acc1[GLU ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc0[i][j] = 0.0f;
            if (GLU) acc1[i][j] = 0.0f;
        }
#pragma unroll
    for (int s = 0; s < MM_STAGES - 1; s++) {
        if (s < nk) load_stage(s, s);
        cp_async_commit();
    }
    for (int kb = 0; kb < nk; kb++) {
        cp_async_wait<MM_STAGES - 2>();
        __syncthreads();                                   // stage kb has landed for everyone; stage kb - 1 has been read by everyone
        const int nxt = kb + MM_STAGES - 1;
        if (nxt < nk) load_stage(nxt % MM_STAGES, nxt);
        cp_async_commit();
        const uint32_t sa = smem0 + (kb % MM_STAGES) * STAGE_BYTES, sb0 = sa + TILE_BYTES, sb1 = sa + 2 * TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < MM_BK / 16; ks++) {
            uint32_t af[4];
            ldmatrix_x4(af, sa + swizzled<128>(wm * 16 + (lane & 15), 2 * ks + (lane >> 4)));
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int brow = wn * 32 + half * 16 + ((lane >> 4) << 3) + (lane & 7);
                const int bch = 2 * ks + ((lane >> 3) & 1);
                uint32_t bf[4];
                ldmatrix_x4(bf, sb0 + swizzled<128>(brow, bch));
                mma_bf16_16816(acc0[2 * half], af, bf[0], bf[1]);
                mma_bf16_16816(acc0[2 * half + 1], af, bf[2], bf[3]);
                if (GLU) {
                    ldmatrix_x4(bf, sb1 + swizzled<128>(brow, bch));
                    mma_bf16_16816(acc1[2 * half], af, bf[0], bf[1]);
                    mma_bf16_16816(acc1[2 * half + 1], af, bf[2], bf[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    const int g = lane >> 2, tg = lane & 3;
#pragma unroll
    for (int hr = 0; hr < 2; hr++) {
        const int dst = row_dst[wm * 16 + g + 8 * hr];
        if (dst < 0) continue;
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int n = n0 + wn * 32 + nt * 8 + 2 * tg + j;
                if (n >= N) continue;
                const float v0 = acc0[nt][2 * hr + j];
                out[(size_t)dst * ldo + n] = from_f32<TO>(moe_first_act<MODE>(v0, acc1[GLU ? nt : 0][2 * hr + j], limit, alpha));
            }
    }
}

template <int MODE, typename TO>
static int moe_mma_launch(dim3 grid, cudaStream_t s, const bf16* a, long long lda, const bf16* w0, const bf16* w1, const int* offsets,
                          const int* order, const int* tiles, int top, TO* out, long long ldo, int N, int K, float limit, float alpha) {
    constexpr int SMEM = MM_STAGES * MM_BM * MM_BK * 2 * (MODE == 1 ? 3 : 2);
    static bool done[HB_MAX_DEVICES] = {};
    const int slot = hb_device_slot();
    if (!done[slot]) {
        cudaError_t e = cudaFuncSetAttribute(moe_product_mma_kernel<MODE, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("moe: shared memory: %s", cudaGetErrorString(e));
        done[slot] = true;
    }
    hb_launch(moe_product_mma_kernel<MODE, TO>, dim3(grid), dim3(MM_THREADS), SMEM, s, a, lda, w0, w1, offsets, order, tiles, top, out, ldo, N, K,
              limit, alpha);
    return 0;
}

extern "C" int hb_moe_glu(const void* h, int h_dtype, long long ldh, const void* w_gate, const void* w_up, int w_dtype, const int* offsets,
                          const int* order, const int* tiles, int max_tiles, int top, void* act, int act_dtype, long long lda, int ff,
                          int width, float limit, float alpha, int tensor_cores, void* stream) {
    HB_REQUIRE(max_tiles > 0 && ff > 0 && width > 0 && top >= 1, "moe_glu: bad sizes");
    HB_REQUIRE((ff + MOE_BN - 1) / MOE_BN <= 65535, "moe_glu: too many columns");
    dim3 grid(max_tiles, (ff + MOE_BN - 1) / MOE_BN);
    cudaStream_t s = (cudaStream_t)stream;
    if (tensor_cores) {
        HB_REQUIRE(h_dtype == HB_BF16 && w_dtype == HB_BF16 && act_dtype == HB_BF16 && width % 8 == 0 && ldh % 8 == 0 &&
                   (((uintptr_t)h | (uintptr_t)w_gate | (uintptr_t)w_up) & 15) == 0,   /* a null w_up: one matrix */
                   "moe_glu: the tensor-core variant needs bfloat16 operands with 16-byte aligned rows");
        grid.y = (ff + MM_BN - 1) / MM_BN;
        if (w_up == nullptr) {
            if (moe_mma_launch<2, bf16>(grid, s, (const bf16*)h, ldh, (const bf16*)w_gate, (const bf16*)nullptr, offsets, order, tiles, top,
                                        (bf16*)act, lda, ff, width, limit, alpha)) return 1;
        } else if (moe_mma_launch<1, bf16>(grid, s, (const bf16*)h, ldh, (const bf16*)w_gate, (const bf16*)w_up, offsets, order, tiles, top,
                                           (bf16*)act, lda, ff, width, limit, alpha)) return 1;
        return hb_check_launch("moe_glu");
    }
    if (w_up == nullptr) {
        // one matrix per expert (passed as w_gate) and the exact gelu
        if (h_dtype == HB_BF16 && w_dtype == HB_BF16 && act_dtype == HB_BF16)
            hb_launch(moe_product_kernel<bf16, bf16, bf16, 2>, dim3(grid), dim3(MOE_THREADS), 0, s, (const bf16*)h, ldh, (const bf16*)w_gate,
                      (const bf16*)nullptr, offsets, order, tiles, top, (bf16*)act, lda, ff, width, limit, alpha);
        else if (h_dtype == HB_F32 && w_dtype == HB_F32 && act_dtype == HB_F32)
            hb_launch(moe_product_kernel<float, float, float, 2>, dim3(grid), dim3(MOE_THREADS), 0, s, (const float*)h, ldh, (const float*)w_gate,
                      (const float*)nullptr, offsets, order, tiles, top, (float*)act, lda, ff, width, limit, alpha);
        else return hb_fail("moe_glu: unsupported dtypes h %d w %d act %d", h_dtype, w_dtype, act_dtype);
        return hb_check_launch("moe_glu");
    }
    if (h_dtype == HB_BF16 && w_dtype == HB_BF16 && act_dtype == HB_BF16)
        hb_launch(moe_product_kernel<bf16, bf16, bf16, 1>, dim3(grid), dim3(MOE_THREADS), 0, s, (const bf16*)h, ldh, (const bf16*)w_gate,
                  (const bf16*)w_up, offsets, order, tiles, top, (bf16*)act, lda, ff, width, limit, alpha);
    else if (h_dtype == HB_F32 && w_dtype == HB_F32 && act_dtype == HB_F32)
        hb_launch(moe_product_kernel<float, float, float, 1>, dim3(grid), dim3(MOE_THREADS), 0, s, (const float*)h, ldh, (const float*)w_gate,
                  (const float*)w_up, offsets, order, tiles, top, (float*)act, lda, ff, width, limit, alpha);
    else return hb_fail("moe_glu: unsupported dtypes h %d w %d act %d", h_dtype, w_dtype, act_dtype);
    return hb_check_launch("moe_glu");
}

extern "C" int hb_moe_down(const void* act, int act_dtype, long long lda, const void* w_down, int w_dtype, const int* offsets, const int* order,
                           const int* tiles, int max_tiles, int top, float* down, long long ldd, int width, int ff, int tensor_cores,
                           void* stream) {
    HB_REQUIRE(max_tiles > 0 && ff > 0 && width > 0, "moe_down: bad sizes");
    HB_REQUIRE((width + MOE_BN - 1) / MOE_BN <= 65535, "moe_down: too many columns");
    dim3 grid(max_tiles, (width + MOE_BN - 1) / MOE_BN);
    cudaStream_t s = (cudaStream_t)stream;
    if (tensor_cores) {
        HB_REQUIRE(act_dtype == HB_BF16 && w_dtype == HB_BF16 && ff % 8 == 0 && lda % 8 == 0 && (((uintptr_t)act | (uintptr_t)w_down) & 15) == 0,
                   "moe_down: the tensor-core variant needs bfloat16 operands with 16-byte aligned rows");
        grid.y = (width + MM_BN - 1) / MM_BN;
        if (moe_mma_launch<0, float>(grid, s, (const bf16*)act, lda, (const bf16*)w_down, (const bf16*)nullptr, offsets, order, tiles, top,
                                         down, ldd, width, ff, 0.0f, 0.0f)) return 1;
        return hb_check_launch("moe_down");
    }
    if (act_dtype == HB_BF16 && w_dtype == HB_BF16)
        hb_launch(moe_product_kernel<bf16, bf16, float, 0>, dim3(grid), dim3(MOE_THREADS), 0, s, (const bf16*)act, lda, (const bf16*)w_down,
                  (const bf16*)nullptr, offsets, order, tiles, top, down, ldd, width, ff, 0.0f, 0.0f);
    else if (act_dtype == HB_F32 && w_dtype == HB_F32)
        hb_launch(moe_product_kernel<float, float, float, 0>, dim3(grid), dim3(MOE_THREADS), 0, s, (const float*)act, lda, (const float*)w_down,
                  (const float*)nullptr, offsets, order, tiles, top, down, ldd, width, ff, 0.0f, 0.0f);
    else return hb_fail("moe_down: unsupported dtypes act %d w %d", act_dtype, w_dtype);
    return hb_check_launch("moe_down");
}

// ------------------------------------------------------------------------------------------------ combine
// `experts` with `n_real`: an entry whose expert number is n_real or more is an identity expert, whose result is the
// token's input row of `h` itself
template <typename TH>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ down, long long ldd, const float* __restrict__ weights, int top, float* __restrict__ out,
                   long long ldo, int width, int accumulate, const int* __restrict__ experts, int n_real, const TH* __restrict__ h,
                   long long ldh) {
    pdl_trigger();
    pdl_wait();
    down = pdl_fresh(down);
    weights = pdl_fresh(weights);
    experts = pdl_fresh(experts);
    h = pdl_fresh(h);
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += 256) {
        float v = accumulate ? out[(size_t)t * ldo + c] : 0.0f;
        for (int k = 0; k < top; k++) {
            const bool same = experts != nullptr && experts[(size_t)t * top + k] >= n_real;
            v = fmaf(weights[(size_t)t * top + k], same ? to_f32(h[(size_t)t * ldh + c]) : down[((size_t)t * top + k) * ldd + c], v);
        }
        out[(size_t)t * ldo + c] = v;
    }
}

extern "C" int hb_moe_combine(const float* down, long long ldd, const float* weights, int top, float* out, long long ldo, int n_tokens,
                              int width, int accumulate, const int* experts, int n_real, const void* h, int h_dtype, long long ldh,
                              void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && width > 0 && top >= 1, "moe_combine: bad sizes");
    HB_REQUIRE(experts == nullptr || (h != nullptr && ldh >= width && n_real >= 0), "moe_combine: identity experts need the input rows");
    cudaStream_t s = (cudaStream_t)stream;
    if (experts != nullptr && h_dtype == HB_BF16)
        hb_launch(moe_combine_kernel<bf16>, dim3(n_tokens), dim3(256), 0, s, down, ldd, weights, top, out, ldo, width, accumulate, experts, n_real,
                  (const bf16*)h, ldh);
    else if (experts == nullptr || h_dtype == HB_F32)
        hb_launch(moe_combine_kernel<float>, dim3(n_tokens), dim3(256), 0, s, down, ldd, weights, top, out, ldo, width, accumulate, experts, n_real,
                  (const float*)h, ldh);
    else return hb_fail("moe_combine: unsupported input dtype %d", h_dtype);
    return hb_check_launch("moe_combine");
}

// ------------------------------------------------------------------------------------------------ gelu_unit
// kind 0: out = gelu_tanh(in[:, :F]) * in[:, F:2F]  (a gated unit with the tanh form of gelu)
// kind 1: out = gelu_erf(in[:, :F]) * (row_gate >= 0 ? sigmoid(in[:, row_gate]) : 1)  (one matrix, the exact gelu, and a
//         per-row gate from one more column of the same product)
template <typename TO>
__global__ void __launch_bounds__(256)
gelu_unit_kernel(const float* __restrict__ in, long long ldi, TO* __restrict__ out, long long ldo, int F, int kind, int row_gate) {
    pdl_trigger();
    pdl_wait();
    in = pdl_fresh(in);
    const float* r = in + (size_t)blockIdx.y * ldi;
    float gate = 1.0f;
    if (kind == 1 && row_gate >= 0) gate = 1.0f / (1.0f + expf(-r[row_gate]));
    for (int i = blockIdx.x * 256 + threadIdx.x; i < F; i += gridDim.x * 256) {
        const float zv = r[i];
        float v;
        if (kind == 0) v = 0.5f * zv * (1.0f + tanhf(0.7978845608028654f * (zv + 0.044715f * zv * zv * zv))) * r[F + i];
        else v = moe_gelu_erf(zv) * gate;
        out[(size_t)blockIdx.y * ldo + i] = from_f32<TO>(v);
    }
}

extern "C" int hb_gelu_unit(const float* in, long long ldi, void* out, int out_dtype, long long ldo, int n_rows, int F, int kind,
                            int row_gate, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n_rows <= 65535 && F > 0 && ldo >= F && (kind == 0 || kind == 1), "gelu_unit: bad sizes");
    HB_REQUIRE(ldi >= (kind == 0 ? 2 * F : F) && row_gate < ldi, "gelu_unit: input rows are too short");
    dim3 grid(min((F + 255) / 256, 64), n_rows);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16) hb_launch(gelu_unit_kernel<bf16>, dim3(grid), dim3(256), 0, s, in, ldi, (bf16*)out, ldo, F, kind, row_gate);
    else if (out_dtype == HB_F32) hb_launch(gelu_unit_kernel<float>, dim3(grid), dim3(256), 0, s, in, ldi, (float*)out, ldo, F, kind, row_gate);
    else return hb_fail("gelu_unit: unsupported output dtype %d", out_dtype);
    return hb_check_launch("gelu_unit");
}

// ------------------------------------------------------------------------------------------------ glu_clamp
// in [rows][2 F] = [gate | up] in 32-bit, out [rows][F]
template <typename TO>
__global__ void __launch_bounds__(256)
glu_clamp_kernel(const float* __restrict__ in, long long ldi, TO* __restrict__ out, long long ldo, int F, float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    in = pdl_fresh(in);
    const float* r = in + (size_t)blockIdx.y * ldi;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < F; i += gridDim.x * 256)
        out[(size_t)blockIdx.y * ldo + i] = from_f32<TO>(moe_glu(r[i], r[F + i], limit, alpha));
}

extern "C" int hb_glu_clamp(const float* in, long long ldi, void* out, int out_dtype, long long ldo, int n_rows, int F, float limit,
                            float alpha, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n_rows <= 65535 && F > 0 && ldi >= 2 * F && ldo >= F, "glu_clamp: bad sizes");
    dim3 grid(min((F + 255) / 256, 64), n_rows);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16) hb_launch(glu_clamp_kernel<bf16>, dim3(grid), dim3(256), 0, s, in, ldi, (bf16*)out, ldo, F, limit, alpha);
    else if (out_dtype == HB_F32) hb_launch(glu_clamp_kernel<float>, dim3(grid), dim3(256), 0, s, in, ldi, (float*)out, ldo, F, limit, alpha);
    else return hb_fail("glu_clamp: unsupported output dtype %d", out_dtype);
    return hb_check_launch("glu_clamp");
}
