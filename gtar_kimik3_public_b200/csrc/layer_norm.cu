// Layer norm with a weight and no bias on the 32-bit residual stream, fused with the add of a branch output that
// has not been added yet:
//
//   h += delta_scale * delta            (in place; skipped when there is no delta)
//   out = (h - mean(h)) / sqrt(mean((h - mean(h))^2) + eps) * w
//
// The variance is the mean of the squared deviations, formed in a second pass over the row (kept in shared
// memory), not from the mean of squares.  With `rows` only those rows are normed and the stream is not written.
// One block of a fixed size per row: the order of a row's sums depends on nothing but the row.  All arithmetic
// is 32-bit; the branch output may be bfloat16, the result bfloat16 or float32.

#include "common.cuh"

namespace {

constexpr int LN_THREADS = 256;

template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(LN_THREADS) add_layernorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                                                   float delta_scale, const TW* __restrict__ w,
                                                                   TO* __restrict__ out, const int* __restrict__ rows,
                                                                   int hidden, float eps) {
    extern __shared__ float row[];  // hidden floats
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* hrow = h + (size_t)src * hidden;
    const bool has_delta = delta != nullptr;
    const TD* drow = delta + (size_t)src * hidden;
    const bool write_back = rows == nullptr && has_delta;
    float sum = 0.f;
    for (int i = threadIdx.x; i < hidden; i += LN_THREADS) {
        float v = hrow[i];
        if (has_delta) v = fmaf(delta_scale, to_float(drow[i]), v);
        if (write_back) hrow[i] = v;
        row[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += LN_THREADS) {
        const float dev = row[i] - mean;
        ss = fmaf(dev, dev, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    TO* orow = out + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += LN_THREADS) orow[i] = from_float<TO>((row[i] - mean) * inv * to_float(w[i]));
}

// out = sa * a + sb * b, element by element, in 32-bit
template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, float sa, const T* __restrict__ b, float sb, float* __restrict__ out,
                                  long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) out[idx] = fmaf(sb, to_float(b[idx]), sa * to_float(a[idx]));
}

// x <- s * x in place (32-bit)
__global__ void scale_kernel(float* __restrict__ x, long long total, float s) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) x[idx] *= s;
}

// the square of relu, element by element
template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ in, T* __restrict__ out, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const float z = fmaxf(to_float(in[idx]), 0.f);
    out[idx] = from_float<T>(z * z);
}

__global__ void relu_squared_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long pieces) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pieces) return;
    uint4 raw = in[idx];
    __nv_bfloat162* pair = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 v = __bfloat1622float2(pair[i]);
        v.x = fmaxf(v.x, 0.f);
        v.y = fmaxf(v.y, 0.f);
        pair[i] = __floats2bfloat162_rn(v.x * v.x, v.y * v.y);
    }
    out[idx] = raw;
}

}  // namespace

GK_EXPORT int gk_add_layernorm(float* h, const void* delta, int delta_dtype, float delta_scale, const void* weight,
                               int weight_dtype, void* out, int out_dtype, const int* rows, int n_out_rows, int hidden,
                               float eps, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(delta_dtype) && GK_VALID_DTYPE(weight_dtype) && GK_VALID_DTYPE(out_dtype), "add_layernorm: bad dtype code");
    GK_REQUIRE(n_out_rows >= 0 && hidden > 0, "add_layernorm: bad sizes rows=%d hidden=%d", n_out_rows, hidden);
    GK_REQUIRE(eps > 0.f, "add_layernorm: eps must be positive");
    const size_t smem = (size_t)hidden * sizeof(float);
    GK_REQUIRE(smem <= 200 * 1024, "add_layernorm: rows of %d do not fit in shared memory", hidden);
    if (n_out_rows == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(delta_dtype, TD, {
        GK_DISPATCH_DTYPE(weight_dtype, TW, {
            GK_DISPATCH_DTYPE(out_dtype, TO, {
                if (smem > 48 * 1024)
                    cudaFuncSetAttribute(add_layernorm_kernel<TD, TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                gk_launch(add_layernorm_kernel<TD, TW, TO>, dim3(n_out_rows), dim3(LN_THREADS), smem, s, h, (const TD*)delta,
                          delta_scale, (const TW*)weight, (TO*)out, rows, hidden, eps);
            })
        })
    })
    GK_CHECK_LAUNCH("add_layernorm");
    return GK_OK;
}

GK_EXPORT int gk_scaled_sum(const void* a, float sa, const void* b, float sb, int dtype, float* out, long long total, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "scaled_sum: bad dtype %d", dtype);
    GK_REQUIRE(total >= 0, "scaled_sum: bad size");
    if (total == 0) return GK_OK;
    const long long blocks = (total + 255) / 256;
    GK_REQUIRE(blocks < 2147483647LL, "scaled_sum: too many elements");
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(scaled_sum_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)a, sa, (const T*)b, sb,
                  out, total);
    })
    GK_CHECK_LAUNCH("scaled_sum");
    return GK_OK;
}

GK_EXPORT int gk_scale(float* x, long long total, float s, void* stream) {
    GK_REQUIRE(total >= 0, "scale: bad size");
    if (total == 0) return GK_OK;
    const long long blocks = (total + 255) / 256;
    GK_REQUIRE(blocks < 2147483647LL, "scale: too many elements");
    gk_launch(scale_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, total, s);
    GK_CHECK_LAUNCH("scale");
    return GK_OK;
}

GK_EXPORT int gk_relu_squared(const void* in, void* out, int dtype, long long total, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "relu_squared: bad dtype %d", dtype);
    GK_REQUIRE(total >= 0, "relu_squared: bad size");
    if (total == 0) return GK_OK;
    const int threads = 256;
    if (dtype == GK_BF16 && total % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const long long pieces = total / 8, blocks8 = (pieces + threads - 1) / threads;
        GK_REQUIRE(blocks8 < 2147483647LL, "relu_squared: too many elements");
        gk_launch(relu_squared_bf16x8_kernel, dim3((unsigned)blocks8), dim3(threads), 0, (cudaStream_t)stream, (const uint4*)in,
                  (uint4*)out, pieces);
        GK_CHECK_LAUNCH("relu_squared");
        return GK_OK;
    }
    const long long blocks = (total + threads - 1) / threads;
    GK_REQUIRE(blocks < 2147483647LL, "relu_squared: too many elements");
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(relu_squared_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, (const T*)in, (T*)out, total);
    })
    GK_CHECK_LAUNCH("relu_squared");
    return GK_OK;
}
