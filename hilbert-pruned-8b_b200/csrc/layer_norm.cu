// Layer norm with weight and bias, y = (x - mean) / sqrt(var + eps) * w + b (var = the mean squared
// deviation from the mean), as a norm of its own and as a norm that sits on a sublayer's OUTPUT.
//
// layernorm:      out[i] = norm(x[rows[i]])  (rows null: every row), in the dtype the next product reads.
// layernorm_add:  x[t] += norm(sa * y[t] + sb * y2[t])  (y2 null: norm(y[t])): the weighted sum of two
//                 sublayers' outputs never exists in memory; with `copy` the new row of x is also written
//                 there in copy's dtype: the sublayers of such a block read the residual stream itself, and
//                 a bfloat16 product reads this copy.
// convert:        out = x in out's dtype (the copy for the first block of a stack).
// Everything in 32-bit, two passes over the row for the variance (mean first, then deviations): one block
// per token, a thread keeps up to LN_KEEP of its values in registers between the passes.
#include "api.h"
#include "common.cuh"

#define LN_THREADS 256
#define LN_KEEP 8

template <typename TO>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w, const float* __restrict__ b, float eps,
                 TO* __restrict__ out, long long ldo, const int* __restrict__ rows, int n) {
    pdl_trigger();
    pdl_wait();
    x = pdl_fresh(x);
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* xr = x + (size_t)(rows ? rows[t] : t) * ldx;
    float keep[LN_KEEP];
    float sum = 0.0f;
    int slot = 0;
    for (int i = tid; i < n; i += LN_THREADS, slot++) {
        const float v = xr[i];
        if (slot < LN_KEEP) keep[slot] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)n;
    float ss = 0.0f;
    slot = 0;
    for (int i = tid; i < n; i += LN_THREADS, slot++) {
        const float d = (slot < LN_KEEP ? keep[slot] : xr[i]) - mean;
        ss = fmaf(d, d, ss);
    }
    const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
    TO* o = out + (size_t)t * ldo;
    slot = 0;
    for (int i = tid; i < n; i += LN_THREADS, slot++) {
        const float d = (slot < LN_KEEP ? keep[slot] : xr[i]) - mean;
        o[i] = from_f32<TO>(d * r * w[i] + b[i]);
    }
}

extern "C" int hb_layernorm(const float* x, long long ldx, const float* w, const float* b, float eps, void* out, int out_dtype,
                            long long ldo, const int* rows, int n_rows, int n, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n > 0 && ldx >= n && ldo >= n, "layernorm: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_F32) hb_launch(layernorm_kernel<float>, dim3(n_rows), dim3(LN_THREADS), 0, s, x, ldx, w, b, eps, (float*)out, ldo, rows, n);
    else if (out_dtype == HB_BF16) hb_launch(layernorm_kernel<bf16>, dim3(n_rows), dim3(LN_THREADS), 0, s, x, ldx, w, b, eps, (bf16*)out, ldo, rows, n);
    else return hb_fail("layernorm: unsupported output dtype %d", out_dtype);
    return hb_check_launch("layernorm");
}

template <typename TC>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_add_kernel(const float* __restrict__ y, long long ldy, const float* __restrict__ y2, long long ldy2, float sa, float sb,
                     const float* __restrict__ w, const float* __restrict__ b, float eps, float* __restrict__ x, long long ldx,
                     TC* __restrict__ copy, long long ldc, int n) {
    pdl_trigger();
    pdl_wait();
    y = pdl_fresh(y);
    y2 = pdl_fresh(y2);
    x = pdl_fresh(x);
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* yr = y + (size_t)t * ldy;
    const float* y2r = y2 ? y2 + (size_t)t * ldy2 : nullptr;
    float keep[LN_KEEP];
    float sum = 0.0f;
    int slot = 0;
    for (int i = tid; i < n; i += LN_THREADS, slot++) {
        const float v = y2r ? sa * yr[i] + sb * y2r[i] : yr[i];
        if (slot < LN_KEEP) keep[slot] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)n;
    float ss = 0.0f;
    slot = 0;
    for (int i = tid; i < n; i += LN_THREADS, slot++) {
        const float d = (slot < LN_KEEP ? keep[slot] : (y2r ? sa * yr[i] + sb * y2r[i] : yr[i])) - mean;
        ss = fmaf(d, d, ss);
    }
    const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
    float* xr = x + (size_t)t * ldx;
    slot = 0;
    for (int i = tid; i < n; i += LN_THREADS, slot++) {
        const float d = (slot < LN_KEEP ? keep[slot] : (y2r ? sa * yr[i] + sb * y2r[i] : yr[i])) - mean;
        const float v = xr[i] + (d * r * w[i] + b[i]);
        xr[i] = v;
        if (copy != nullptr) copy[(size_t)t * ldc + i] = from_f32<TC>(v);
    }
}

extern "C" int hb_layernorm_add(const float* y, long long ldy, const float* y2, long long ldy2, float sa, float sb, const float* w,
                                const float* b, float eps, float* x, long long ldx, void* copy, int copy_dtype, long long ldc,
                                int n_rows, int n, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && n > 0 && ldy >= n && ldx >= n && (y2 == nullptr || ldy2 >= n) && (copy == nullptr || ldc >= n),
               "layernorm_add: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    if (copy == nullptr || copy_dtype == HB_F32)
        hb_launch(layernorm_add_kernel<float>, dim3(n_rows), dim3(LN_THREADS), 0, s, y, ldy, y2, ldy2, sa, sb, w, b, eps, x, ldx, (float*)copy, ldc, n);
    else if (copy_dtype == HB_BF16)
        hb_launch(layernorm_add_kernel<bf16>, dim3(n_rows), dim3(LN_THREADS), 0, s, y, ldy, y2, ldy2, sa, sb, w, b, eps, x, ldx, (bf16*)copy, ldc, n);
    else return hb_fail("layernorm_add: unsupported copy dtype %d", copy_dtype);
    return hb_check_launch("layernorm_add");
}

template <typename TO>
__global__ void __launch_bounds__(256)
convert_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
    pdl_trigger();
    pdl_wait();
    x = pdl_fresh(x);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(x[i]);
}

extern "C" int hb_convert(const float* x, void* out, int out_dtype, long long n, void* stream) {
    if (n == 0) return 0;
    HB_REQUIRE(n > 0, "convert: bad size");
    const long long blocks = (n + 255) / 256;
    const dim3 grid((unsigned)(blocks < 4736 ? blocks : 4736));
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16) hb_launch(convert_kernel<bf16>, dim3(grid), dim3(256), 0, s, x, (bf16*)out, n);
    else if (out_dtype == HB_F32) hb_launch(convert_kernel<float>, dim3(grid), dim3(256), 0, s, x, (float*)out, n);
    else return hb_fail("convert: unsupported output dtype %d", out_dtype);
    return hb_check_launch("convert");
}
