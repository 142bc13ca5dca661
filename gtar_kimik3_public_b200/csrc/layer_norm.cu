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

// Steps in which every sequence brings ONE token: the add, the layer norm and the short convolution over time that
// reads its result, in one kernel (row t is the token of sequence tok_seq[t]).  With y the normed row,
//   out = y + sum_j cw[j] * y_(pos - (taps - 1 - j)),
// where the inputs of earlier positions come from the sequence's state [taps - 1, hidden] (zeros before the sequence's
// start) and, with `update`, the state is moved on by y.  The norm's and the convolution's sums have the order they have
// in the kernels that do one of the two, so the numbers are the same: the block has LNC_THREADS threads for the loads
// of the earlier inputs and for the convolution, a channel or two a thread, and its first LN_THREADS threads alone sum
// the row, as the norm's own kernel does (the others add zeros, which a sum over the warps does not see).
constexpr int LNC_THREADS = 1024;
__device__ __forceinline__ void lnc_copy4(float* smem, const float* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
template <typename TD, typename TO>
__global__ void __launch_bounds__(LNC_THREADS) add_layernorm_conv_single_kernel(
    float* __restrict__ h, const TD* __restrict__ delta, float delta_scale, const float* __restrict__ w, const float* __restrict__ cw,
    float* __restrict__ state, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
    TO* __restrict__ out, int hidden, int taps, float eps, int update) {
    extern __shared__ float row[];  // hidden floats; the sequence's taps - 1 earlier inputs; the taps' weights; the norm's
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int kept = taps - 1;
    float* past = row + hidden;                   // [kept, hidden]
    float* cws = past + (size_t)kept * hidden;    // [taps, hidden]
    float* ws = cws + (size_t)taps * hidden;      // [hidden]
    // Everything but the row itself comes in by asynchronous copies that no instruction waits for before the last loop:
    // the weights first (they wait for no earlier kernel), then the earlier inputs, whose place hangs on two index loads.
    for (int i = threadIdx.x; i < taps * hidden; i += LNC_THREADS) lnc_copy4(cws + i, cw + i);
    for (int i = threadIdx.x; i < hidden; i += LNC_THREADS) lnc_copy4(ws + i, w + i);
    pdl_wait();
    float* hrow = h + (size_t)t * hidden;
    const bool has_delta = delta != nullptr;
    const TD* drow = delta + (size_t)t * hidden;
    const int pos = tok_pos[t];
    float* mine = kept > 0 ? state + (size_t)slots[tok_seq[t]] * kept * hidden : nullptr;
    for (int j = 0; j < kept; ++j) {
        if (pos - (kept - j) < 0) {  // before the sequence's start
            for (int c = threadIdx.x; c < hidden; c += LNC_THREADS) past[(size_t)j * hidden + c] = 0.f;
        } else {
            for (int c = threadIdx.x; c < hidden; c += LNC_THREADS) lnc_copy4(past + (size_t)j * hidden + c, mine + (size_t)j * hidden + c);
        }
    }
    asm volatile("cp.async.commit_group;\n" ::);
    const bool sums = threadIdx.x < LN_THREADS;
    float sum = 0.f;
    if (sums)
        for (int i = threadIdx.x; i < hidden; i += LN_THREADS) {
            float v = hrow[i];
            if (has_delta) {
                v = fmaf(delta_scale, to_float(drow[i]), v);
                hrow[i] = v;
            }
            row[i] = v;
            sum += v;
        }
    const float mean = block_sum(sum, scratch) / (float)hidden;
    float ss = 0.f;
    if (sums)
        for (int i = threadIdx.x; i < hidden; i += LN_THREADS) {
            const float dev = row[i] - mean;
            ss = fmaf(dev, dev, ss);
        }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    TO* orow = out + (size_t)t * hidden;
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    for (int c = threadIdx.x; c < hidden; c += LNC_THREADS) {
        const float own = (row[c] - mean) * inv * ws[c];
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) acc = fmaf(cws[(size_t)j * hidden + c], j == kept ? own : past[(size_t)j * hidden + c], acc);
        orow[c] = from_float<TO>(own + acc);
        if (update && kept > 0) {
            // positions before the sequence's start stay zeros in the state, as they are where nothing was written yet
            for (int k = 0; k + 1 < kept; ++k) mine[(size_t)k * hidden + c] = past[(size_t)(k + 1) * hidden + c];
            mine[(size_t)(kept - 1) * hidden + c] = own;
        }
    }
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

// A quadratic above zero and an exponential below, joined smoothly at zero:
//   z > 0:  up * z^2 + z / 2          z <= 0:  down * (exp(z) - 1 - z) + z / 2
// `up` and `down` are the two finished constants (the caller forms them from the stored numbers once, at load).
__device__ __forceinline__ float xielu_f(float z, float up, float down) {
    return z > 0.f ? fmaf(up * z, z, 0.5f * z) : fmaf(down, expm1f(z) - z, 0.5f * z);
}

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ in, T* __restrict__ out, long long total, float up, float down) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    out[idx] = from_float<T>(xielu_f(to_float(in[idx]), up, down));
}

__global__ void xielu_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long pieces, float up, float down) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pieces) return;
    uint4 raw = in[idx];
    __nv_bfloat162* pair = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(pair[i]);
        pair[i] = __floats2bfloat162_rn(xielu_f(v.x, up, down), xielu_f(v.y, up, down));
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

// The row, its earlier inputs and the weights stay in shared memory: 2 taps + 1 rows of 32-bit numbers within this.
constexpr int GK_ADD_LAYERNORM_CONV_SINGLE_SMEM = 200 * 1024;

// weight [hidden] and conv_w [taps, hidden] 32-bit; state [n_slots, taps - 1, hidden] (may be null for one tap); one row a
// sequence.
GK_EXPORT int gk_add_layernorm_conv_single(float* h, const void* delta, int delta_dtype, float delta_scale, const float* weight,
                                           const float* conv_w, float* state, const int* tok_pos, const int* tok_seq, const int* slots,
                                           void* out, int out_dtype, int n_rows, int hidden, int taps, float eps, int update,
                                           void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(delta_dtype) && GK_VALID_DTYPE(out_dtype), "add_layernorm_conv_single: bad dtype code");
    GK_REQUIRE(n_rows >= 0 && hidden > 0 && taps >= 1, "add_layernorm_conv_single: bad sizes");
    GK_REQUIRE(taps == 1 || state != nullptr, "add_layernorm_conv_single: %d taps need the sequences' states", taps);
    GK_REQUIRE(eps > 0.f, "add_layernorm_conv_single: eps must be positive");
    const size_t smem = (size_t)hidden * (2 * taps + 1) * sizeof(float);
    GK_REQUIRE(smem <= (size_t)GK_ADD_LAYERNORM_CONV_SINGLE_SMEM, "add_layernorm_conv_single: rows of %d with %d taps do not fit in shared memory", hidden, taps);
    if (n_rows == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(delta_dtype, TD, {
        GK_DISPATCH_DTYPE(out_dtype, TO, {
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(add_layernorm_conv_single_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            gk_launch(add_layernorm_conv_single_kernel<TD, TO>, dim3(n_rows), dim3(LNC_THREADS), smem, s, h, (const TD*)delta, delta_scale,
                      weight, conv_w, state, tok_pos, tok_seq, slots, (TO*)out, hidden, taps, eps, update);
        })
    })
    GK_CHECK_LAUNCH("add_layernorm_conv_single");
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

GK_EXPORT int gk_xielu(const void* in, void* out, int dtype, long long total, float up, float down, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "xielu: bad dtype %d", dtype);
    GK_REQUIRE(total >= 0, "xielu: bad size");
    if (total == 0) return GK_OK;
    const int threads = 256;
    if (dtype == GK_BF16 && total % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const long long pieces = total / 8, blocks8 = (pieces + threads - 1) / threads;
        GK_REQUIRE(blocks8 < 2147483647LL, "xielu: too many elements");
        gk_launch(xielu_bf16x8_kernel, dim3((unsigned)blocks8), dim3(threads), 0, (cudaStream_t)stream, (const uint4*)in, (uint4*)out,
                  pieces, up, down);
        GK_CHECK_LAUNCH("xielu");
        return GK_OK;
    }
    const long long blocks = (total + threads - 1) / threads;
    GK_REQUIRE(blocks < 2147483647LL, "xielu: too many elements");
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(xielu_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, (const T*)in, (T*)out, total, up, down);
    })
    GK_CHECK_LAUNCH("xielu");
    return GK_OK;
}
