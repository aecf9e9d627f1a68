// Norm on a sublayer's OUTPUT on its way into the residual stream, and the weighted sum of two
// sublayers' outputs.
//
// rmsnorm_add: x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * (offset + w); with a second norm
// (w2, eps2, offset2) the row that was just made is normed again for the next sublayer,
// h[t] = x[t] / sqrt(mean(x[t]^2) + eps2) * (offset2 + w2), in the same pass: the new residual
// values stay in registers between the two.  Everything in 32-bit; h in the dtype the next
// matrix product reads.  One block per token.
#include "api.h"
#include "common.cuh"

#define PN_THREADS 256
#define PN_KEEP 8          // residual values a thread keeps in registers between the two norms (rows up to 2048 wide)

template <typename TO>
__global__ void __launch_bounds__(PN_THREADS)
rmsnorm_add_kernel(const float* __restrict__ y, long long ldy, const float* __restrict__ w, float eps, float offset,
                   float* __restrict__ x, long long ldx, const float* __restrict__ w2, float eps2, float offset2,
                   TO* __restrict__ h, long long ldh, int n) {
    pdl_trigger();
    pdl_wait();
    y = pdl_fresh(y);
    x = pdl_fresh(x);
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* yr = y + (size_t)t * ldy;
    float* xr = x + (size_t)t * ldx;
    float ss = 0.0f;
    for (int i = tid; i < n; i += PN_THREADS) {
        const float v = yr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)n + eps);
    float keep[PN_KEEP];
    float ss2 = 0.0f;
    int slot = 0;
    for (int i = tid; i < n; i += PN_THREADS, slot++) {
        const float v = xr[i] + yr[i] * r * (offset + w[i]);
        xr[i] = v;
        if (slot < PN_KEEP) keep[slot] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (h == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.0f / sqrtf(ss2 / (float)n + eps2);
    TO* hr = h + (size_t)t * ldh;
    slot = 0;
    for (int i = tid; i < n; i += PN_THREADS, slot++) {
        const float v = slot < PN_KEEP ? keep[slot] : xr[i];       // a thread reads back only what it wrote itself
        hr[i] = from_f32<TO>(v * r2 * (offset2 + w2[i]));
    }
}

extern "C" int hb_rmsnorm_add(const float* y, long long ldy, const float* w, float eps, float offset, float* x, long long ldx,
                              const float* w2, float eps2, float offset2, void* h, int h_dtype, long long ldh, int n_rows,
                              int n, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n > 0 && ldy >= n && ldx >= n, "rmsnorm_add: bad sizes");
    HB_REQUIRE(h == nullptr || (w2 != nullptr && ldh >= n), "rmsnorm_add: the second norm needs a weight and an output");
    cudaStream_t s = (cudaStream_t)stream;
    if (h == nullptr || h_dtype == HB_F32)
        hb_launch(rmsnorm_add_kernel<float>, dim3(n_rows), dim3(PN_THREADS), 0, s, y, ldy, w, eps, offset, x, ldx, w2, eps2, offset2,
                  (float*)h, ldh, n);
    else if (h_dtype == HB_BF16)
        hb_launch(rmsnorm_add_kernel<bf16>, dim3(n_rows), dim3(PN_THREADS), 0, s, y, ldy, w, eps, offset, x, ldx, w2, eps2, offset2,
                  (bf16*)h, ldh, n);
    else
        return hb_fail("rmsnorm_add: unsupported output dtype %d", h_dtype);
    return hb_check_launch("rmsnorm_add");
}

// scaled_add_norm: x[t] += m * y[t] (a sublayer's result times a fixed factor on its way into the residual stream); with a
// norm (w2, eps2, offset2) the new row is normed for the next sublayer in the same pass, as above.  One block per token.
template <typename TO>
__global__ void __launch_bounds__(PN_THREADS)
scaled_add_norm_kernel(const float* __restrict__ y, long long ldy, float m, float* __restrict__ x, long long ldx,
                       const float* __restrict__ w2, float eps2, float offset2, TO* __restrict__ h, long long ldh, int n) {
    pdl_trigger();
    pdl_wait();
    y = pdl_fresh(y);
    x = pdl_fresh(x);
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* yr = y + (size_t)t * ldy;
    float* xr = x + (size_t)t * ldx;
    float keep[PN_KEEP];
    float ss2 = 0.0f;
    int slot = 0;
    for (int i = tid; i < n; i += PN_THREADS, slot++) {
        const float v = fmaf(m, yr[i], xr[i]);
        xr[i] = v;
        if (slot < PN_KEEP) keep[slot] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (h == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.0f / sqrtf(ss2 / (float)n + eps2);
    TO* hr = h + (size_t)t * ldh;
    slot = 0;
    for (int i = tid; i < n; i += PN_THREADS, slot++) {
        const float v = slot < PN_KEEP ? keep[slot] : xr[i];
        hr[i] = from_f32<TO>(v * r2 * (offset2 + w2[i]));
    }
}

extern "C" int hb_scaled_add_norm(const float* y, long long ldy, float m, float* x, long long ldx, const float* w2, float eps2,
                                  float offset2, void* h, int h_dtype, long long ldh, int n_rows, int n, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n > 0 && ldy >= n && ldx >= n, "scaled_add_norm: bad sizes");
    HB_REQUIRE(h == nullptr || (w2 != nullptr && ldh >= n), "scaled_add_norm: the norm needs a weight and an output");
    cudaStream_t s = (cudaStream_t)stream;
    if (h == nullptr || h_dtype == HB_F32)
        hb_launch(scaled_add_norm_kernel<float>, dim3(n_rows), dim3(PN_THREADS), 0, s, y, ldy, m, x, ldx, w2, eps2, offset2, (float*)h, ldh, n);
    else if (h_dtype == HB_BF16)
        hb_launch(scaled_add_norm_kernel<bf16>, dim3(n_rows), dim3(PN_THREADS), 0, s, y, ldy, m, x, ldx, w2, eps2, offset2, (bf16*)h, ldh, n);
    else
        return hb_fail("scaled_add_norm: unsupported output dtype %d", h_dtype);
    return hb_check_launch("scaled_add_norm");
}

// normed_sum: out[t] (+)= a[t] / sqrt(mean(a[t]^2) + eps) * wa + b[t] / sqrt(mean(b[t]^2) + eps) * wb: two sublayers'
// results, each normed over the row with a weight of its own (any factor of the sum is part of the weights).
__global__ void __launch_bounds__(PN_THREADS)
normed_sum_kernel(const float* __restrict__ a, long long lda, const float* __restrict__ wa, const float* __restrict__ b, long long ldb,
                  const float* __restrict__ wb, float eps, float* __restrict__ out, long long ldo, int n, int accumulate) {
    pdl_trigger();
    pdl_wait();
    a = pdl_fresh(a);
    b = pdl_fresh(b);
    out = pdl_fresh(out);
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* ar = a + (size_t)t * lda;
    const float* br = b + (size_t)t * ldb;
    float sa = 0.0f, sb = 0.0f;
    for (int i = tid; i < n; i += PN_THREADS) {
        sa = fmaf(ar[i], ar[i], sa);
        sb = fmaf(br[i], br[i], sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ra = 1.0f / sqrtf(sa / (float)n + eps), rb = 1.0f / sqrtf(sb / (float)n + eps);
    float* o = out + (size_t)t * ldo;
    for (int i = tid; i < n; i += PN_THREADS) {
        const float v = ar[i] * ra * wa[i] + br[i] * rb * wb[i];
        o[i] = accumulate ? o[i] + v : v;
    }
}

extern "C" int hb_normed_sum(const float* a, long long lda, const float* wa, const float* b, long long ldb, const float* wb, float eps,
                             float* out, long long ldo, int n_rows, int n, int accumulate, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n > 0 && lda >= n && ldb >= n && ldo >= n, "normed_sum: bad sizes");
    hb_launch(normed_sum_kernel, dim3(n_rows), dim3(PN_THREADS), 0, (cudaStream_t)stream, a, lda, wa, b, ldb, wb, eps, out, ldo, n, accumulate);
    return hb_check_launch("normed_sum");
}

// out = sa * a + sb * b over contiguous 32-bit values (out may be a or b)
__global__ void __launch_bounds__(256)
scaled_sum_kernel(const float* a, float sa, const float* b, float sb, float* out, long long n) {
    pdl_trigger();
    pdl_wait();
    a = pdl_fresh(a);
    b = pdl_fresh(b);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = sa * a[i] + sb * b[i];
}

extern "C" int hb_scaled_sum(const float* a, float sa, const float* b, float sb, float* out, long long n, void* stream) {
    if (n == 0) return 0;
    HB_REQUIRE(n > 0, "scaled_sum: bad size");
    const long long blocks = (n + 255) / 256;
    hb_launch(scaled_sum_kernel, dim3((unsigned)(blocks < 2368 ? blocks : 2368)), dim3(256), 0, (cudaStream_t)stream, a, sa, b, sb, out, n);
    return hb_check_launch("scaled_sum");
}
