// Row-wise work on the 32-bit residual stream for layers that norm a branch before AND after it, scale it
// per channel, and mix the results of earlier layers into the stream; a short causal convolution over time with
// a per-sequence state; and the tanh form of GELU.  All arithmetic is 32-bit; only inputs that come out of a
// projection and outputs that go into one may be bfloat16.
//
//   merge:   v   = x + scale * (y / sqrt(mean(y^2) + eps_y)) * w_y          (w_y holds the effective weights)
//            kept[n] = v ;  v = sum_{j <= n} mix[j] * kept[j]               (if a history is given)
//            x_out = v ;  z = (v / sqrt(mean(v^2) + eps_z)) * w_z           (if a next norm is given)
//                         z = v in z's type                                 (if z is given without weights: the next
//                                                                            sublayer reads the stream itself)
//   conv:    g_t = a_t + sum_j w[j, :] * a_(t - taps + 1 + j)  (weights [taps, width]), a before the sequence's start = 0, a before the
//            step's start read from the sequence's state (its last taps - 1 inputs)
//   state:   after the step the state holds the sequence's last taps - 1 inputs
//
// One block per row with a fixed block size, so the order of a row's sums depends on nothing but the row.

#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

template <typename TY, typename TZ>
__global__ void __launch_bounds__(ROW_THREADS) branch_merge_kernel(
    const float* x, const TY* __restrict__ y, const float* __restrict__ w_y, const float* __restrict__ scale,
    float eps_y, float* __restrict__ kept, long long kept_stride, int n_kept, const float* __restrict__ mix,
    float* x_out, const float* __restrict__ w_z, float eps_z, TZ* __restrict__ z, int width) {
    extern __shared__ float row[];  // width floats
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t at = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += ROW_THREADS) {
        const float v = to_float(y[at + i]);
        row[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.f / sqrtf(ss / (float)width + eps_y);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < width; i += ROW_THREADS) {
        float branch = row[i] * r * w_y[i];
        if (scale != nullptr) branch *= scale[i];
        float v = x[at + i] + branch;
        if (kept != nullptr) {
            kept[(size_t)n_kept * kept_stride + at + i] = v;
            float acc = 0.f;
            for (int j = 0; j < n_kept; ++j) acc = fmaf(mix[j], kept[(size_t)j * kept_stride + at + i], acc);
            v = fmaf(mix[n_kept], v, acc);
        }
        x_out[at + i] = v;
        row[i] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (z == nullptr) return;
    if (w_z == nullptr) {  // each thread reads back what it wrote itself
        for (int i = threadIdx.x; i < width; i += ROW_THREADS) z[at + i] = from_float<TZ>(row[i]);
        return;
    }
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.f / sqrtf(ss2 / (float)width + eps_z);
    for (int i = threadIdx.x; i < width; i += ROW_THREADS) z[at + i] = from_float<TZ>(row[i] * r2 * w_z[i]);
}

// The same with four consecutive elements a thread and turn (width a multiple of 4, 16-byte aligned rows): 16-byte loads of
// the stream and the kept streams, 8- or 16-byte loads of the branch.  A row's sums are formed in an order of their own
// (which depends on the width alone), so the result of a row still depends on nothing but the row.
template <typename T>
__device__ __forceinline__ float4 load_x4(const T* p);
template <>
__device__ __forceinline__ float4 load_x4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load_x4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <typename T>
__device__ __forceinline__ void store_x4(T* p, float4 v);
template <>
__device__ __forceinline__ void store_x4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <>
__device__ __forceinline__ void store_x4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TY, typename TZ>
__global__ void __launch_bounds__(ROW_THREADS) branch_merge_x4_kernel(
    const float* x, const TY* __restrict__ y, const float* __restrict__ w_y, const float* __restrict__ scale,
    float eps_y, float* kept, long long kept_stride, int n_kept, const float* __restrict__ mix,
    float* x_out, const float* __restrict__ w_z, float eps_z, TZ* __restrict__ z, int width) {
    extern __shared__ __align__(16) float row[];  // width floats
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t at = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < width; i += ROW_THREADS * 4) {
        const float4 v = load_x4<TY>(y + at + i);
        *reinterpret_cast<float4*>(row + i) = v;
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.f / sqrtf(ss / (float)width + eps_y);
    float ss2 = 0.f;
    for (int i = threadIdx.x * 4; i < width; i += ROW_THREADS * 4) {
        const float4 b = *reinterpret_cast<const float4*>(row + i);
        const float4 wy = *reinterpret_cast<const float4*>(w_y + i);
        float br[4] = {b.x * r * wy.x, b.y * r * wy.y, b.z * r * wy.z, b.w * r * wy.w};
        if (scale != nullptr) {
            const float4 sc = *reinterpret_cast<const float4*>(scale + i);
            br[0] *= sc.x; br[1] *= sc.y; br[2] *= sc.z; br[3] *= sc.w;
        }
        const float4 xs = *reinterpret_cast<const float4*>(x + at + i);
        float v[4] = {xs.x + br[0], xs.y + br[1], xs.z + br[2], xs.w + br[3]};
        if (kept != nullptr) {
            *reinterpret_cast<float4*>(kept + (size_t)n_kept * kept_stride + at + i) = make_float4(v[0], v[1], v[2], v[3]);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < n_kept; ++j) {
                const float mj = mix[j];
                const float4 k = *reinterpret_cast<const float4*>(kept + (size_t)j * kept_stride + at + i);
                acc[0] = fmaf(mj, k.x, acc[0]); acc[1] = fmaf(mj, k.y, acc[1]);
                acc[2] = fmaf(mj, k.z, acc[2]); acc[3] = fmaf(mj, k.w, acc[3]);
            }
            const float mn = mix[n_kept];
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = fmaf(mn, v[e], acc[e]);
        }
        const float4 out4 = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(x_out + at + i) = out4;
        *reinterpret_cast<float4*>(row + i) = out4;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss2 = fmaf(v[e], v[e], ss2);
    }
    if (z == nullptr) return;
    if (w_z == nullptr) {  // each thread reads back what it wrote itself
        for (int i = threadIdx.x * 4; i < width; i += ROW_THREADS * 4) store_x4<TZ>(z + at + i, *reinterpret_cast<const float4*>(row + i));
        return;
    }
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.f / sqrtf(ss2 / (float)width + eps_z);
    for (int i = threadIdx.x * 4; i < width; i += ROW_THREADS * 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        const float4 wz = *reinterpret_cast<const float4*>(w_z + i);
        store_x4<TZ>(z + at + i, make_float4(v.x * r2 * wz.x, v.y * r2 * wz.y, v.z * r2 * wz.z, v.w * r2 * wz.w));
    }
}

// One thread per (token, channel).  `a` holds the step's inputs, `state` [n_slots, taps - 1, width] the inputs of
// before: entry k of a sequence's state is its input at position  past - (taps - 1) + k.
// `update` (only where every sequence of the step brings ONE token, so that this thread alone reads and writes its
// sequence's entries for the channel): the state is moved on by the token here and no second kernel is needed.
template <typename TO>
__global__ void causal_conv_kernel(const float* __restrict__ a, const float* __restrict__ w, float* state,
                                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                   const int* __restrict__ cu_q, const int* __restrict__ slots, TO* __restrict__ out,
                                   int n_tokens, int width, int taps, int update) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * width) return;
    const int t = (int)(idx / width), c = (int)(idx - (long long)t * width);
    const int seq = tok_seq[t], pos = tok_pos[t];
    const int first = cu_q[seq];      // the sequence's first row in this step
    const int past = pos - (t - first);
    const float own = a[idx];
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        float v;
        if (back == 0) v = own;
        else if (pos - back < 0) v = 0.f;
        else if (t - back >= first) v = a[idx - (long long)back * width];
        else v = state[((size_t)slots[seq] * (taps - 1) + (pos - back - past + taps - 1)) * width + c];
        acc = fmaf(w[(size_t)j * width + c], v, acc);
    }
    out[idx] = from_float<TO>(own + acc);
    if (update && taps > 1) {
        float* mine = state + (size_t)slots[seq] * (taps - 1) * width + c;
        for (int k = 0; k + 1 < taps - 1; ++k) mine[(size_t)k * width] = mine[(size_t)(k + 1) * width];
        mine[(size_t)(taps - 2) * width] = own;
    }
}

// The same for four consecutive channels a thread (width a multiple of 4): the token's numbers are looked up once for four
// outputs and the inputs come as 16-byte loads.
template <typename TO>
__global__ void causal_conv_x4_kernel(const float* __restrict__ a, const float* __restrict__ w, float* state,
                                      const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                      const int* __restrict__ cu_q, const int* __restrict__ slots, TO* __restrict__ out,
                                      int n_tokens, int width, int taps, int update) {
    pdl_launch_dependents();
    pdl_wait();
    const int quads = width >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * quads) return;
    const int t = (int)(idx / quads), c = (int)(idx - (long long)t * quads) * 4;
    const int seq = tok_seq[t], pos = tok_pos[t];
    const int first = cu_q[seq];
    const int past = pos - (t - first);
    const float* mine_a = a + (size_t)t * width + c;
    const float4 own = *reinterpret_cast<const float4*>(mine_a);
    float* st = taps > 1 ? state + (size_t)slots[seq] * (taps - 1) * width + c : nullptr;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        float4 v;
        if (back == 0) v = own;
        else if (pos - back < 0) v = make_float4(0.f, 0.f, 0.f, 0.f);
        else if (t - back >= first) v = *reinterpret_cast<const float4*>(mine_a - (size_t)back * width);
        else v = *reinterpret_cast<const float4*>(st + (size_t)(pos - back - past + taps - 1) * width);
        const float4 wj = *reinterpret_cast<const float4*>(w + (size_t)j * width + c);
        acc[0] = fmaf(wj.x, v.x, acc[0]);
        acc[1] = fmaf(wj.y, v.y, acc[1]);
        acc[2] = fmaf(wj.z, v.z, acc[2]);
        acc[3] = fmaf(wj.w, v.w, acc[3]);
    }
    TO* o = out + (size_t)t * width + c;
    o[0] = from_float<TO>(own.x + acc[0]);
    o[1] = from_float<TO>(own.y + acc[1]);
    o[2] = from_float<TO>(own.z + acc[2]);
    o[3] = from_float<TO>(own.w + acc[3]);
    if (update && taps > 1) {
        for (int k = 0; k + 1 < taps - 1; ++k)
            *reinterpret_cast<float4*>(st + (size_t)k * width) = *reinterpret_cast<const float4*>(st + (size_t)(k + 1) * width);
        *reinterpret_cast<float4*>(st + (size_t)(taps - 2) * width) = own;
    }
}

// One thread per (sequence, channel): entry k of the new state is the input at position  new_len - (taps - 1) + k,
// taken from the step's rows or, where the step brought fewer than taps - 1 tokens, from entry k + n of the old
// state (read before entry k is written, k going up).
__global__ void conv_state_kernel(const float* __restrict__ a, float* __restrict__ state, const int* __restrict__ cu_q,
                                  const int* __restrict__ slots, int n_seqs, int width, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_seqs * width) return;
    const int seq = (int)(idx / width), c = (int)(idx - (long long)seq * width);
    const int first = cu_q[seq], n = cu_q[seq + 1] - first;
    const int keep = taps - 1;
    float* mine = state + (size_t)slots[seq] * keep * width + c;
    for (int k = 0; k < keep; ++k) {
        const int row = n - keep + k;  // row of the step that holds this position, if not negative
        float v;
        if (row >= 0) v = a[(size_t)(first + row) * width + c];
        else v = mine[(size_t)(k + n) * width];
        mine[(size_t)k * width] = v;
    }
}

// The tanh form of GELU.  float: tanhf, one element a thread.  bfloat16: eight elements (16 bytes) a thread, and
// tanh(u) = 1 - 2 / (1 + e^(2u)) with the hardware's exponential, whose error is far below the result's rounding.
template <typename T>
__global__ void gelu_tanh_kernel(const T* __restrict__ in, T* __restrict__ out, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const float z = to_float(in[idx]);
    const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    out[idx] = from_float<T>(0.5f * z * (1.f + tanhf(inner)));
}

__device__ __forceinline__ float gelu_tanh_fast(float z) {
    const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    const float t = 1.f - __fdividef(2.f, 1.f + __expf(2.f * u));  // e^(2u) = inf gives 1, 0 gives -1
    return 0.5f * z * (1.f + t);
}

__global__ void gelu_tanh_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long pieces) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pieces) return;
    uint4 raw = in[idx];
    __nv_bfloat162* pair = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(pair[i]);
        pair[i] = __floats2bfloat162_rn(gelu_tanh_fast(v.x), gelu_tanh_fast(v.y));
    }
    out[idx] = raw;
}

// The 32-bit stream in another type, element by element (what a sublayer that reads the stream itself multiplies).
template <typename T>
__global__ void stream_cast_kernel(const float* __restrict__ x, T* __restrict__ out, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) out[idx] = from_float<T>(x[idx]);
}

}  // namespace

GK_EXPORT int gk_stream_cast(const float* x, void* out, int out_dtype, long long total, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(out_dtype) && total >= 0, "stream_cast: bad arguments");
    if (total == 0) return GK_OK;
    const long long blocks = (total + 255) / 256;
    GK_REQUIRE(blocks < 2147483647LL, "stream_cast: too many elements");
    GK_DISPATCH_DTYPE(out_dtype, T, {
        gk_launch(stream_cast_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, (T*)out, total);
    })
    GK_CHECK_LAUNCH("stream_cast");
    return GK_OK;
}

GK_EXPORT int gk_branch_merge(const float* x, const void* y, int y_dtype, const float* w_y, const float* scale, float eps_y,
                              float* kept, long long kept_stride, int n_kept, const float* mix, float* x_out,
                              const float* w_z, float eps_z, void* z, int z_dtype, int n_rows, int width, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(y_dtype) && GK_VALID_DTYPE(z_dtype), "branch_merge: bad dtype code");
    GK_REQUIRE(n_rows >= 0 && width > 0, "branch_merge: bad sizes rows=%d width=%d", n_rows, width);
    GK_REQUIRE(x && y && w_y && x_out, "branch_merge: the stream, the branch and its norm weights are needed");
    GK_REQUIRE(eps_y > 0.f && (w_z == nullptr || eps_z > 0.f), "branch_merge: eps must be positive");
    GK_REQUIRE((kept == nullptr) == (mix == nullptr) && n_kept >= 0, "branch_merge: a history needs mixing weights");
    GK_REQUIRE(w_z == nullptr || z != nullptr, "branch_merge: a next norm needs an output");
    const size_t smem = (size_t)width * sizeof(float);
    GK_REQUIRE(smem <= 200 * 1024, "branch_merge: rows of %d do not fit in shared memory", width);
    if (n_rows == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const uintptr_t all = (uintptr_t)x | (uintptr_t)y | (uintptr_t)w_y | (uintptr_t)scale | (uintptr_t)kept | (uintptr_t)x_out |
                          (uintptr_t)w_z | (uintptr_t)z;
    if (width % 4 == 0 && (all & 15) == 0 && kept_stride % 4 == 0) {
        GK_DISPATCH_DTYPE(y_dtype, TY, {
            GK_DISPATCH_DTYPE(z_dtype, TZ, {
                if (smem > 48 * 1024)
                    cudaFuncSetAttribute(branch_merge_x4_kernel<TY, TZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                gk_launch(branch_merge_x4_kernel<TY, TZ>, dim3(n_rows), dim3(ROW_THREADS), smem, s, x, (const TY*)y, w_y, scale, eps_y,
                          kept, kept_stride, n_kept, mix, x_out, w_z, eps_z, (TZ*)z, width);
            })
        })
        GK_CHECK_LAUNCH("branch_merge");
        return GK_OK;
    }
    GK_DISPATCH_DTYPE(y_dtype, TY, {
        GK_DISPATCH_DTYPE(z_dtype, TZ, {
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(branch_merge_kernel<TY, TZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            gk_launch(branch_merge_kernel<TY, TZ>, dim3(n_rows), dim3(ROW_THREADS), smem, s, x, (const TY*)y, w_y, scale, eps_y,
                      kept, kept_stride, n_kept, mix, x_out, w_z, eps_z, (TZ*)z, width);
        })
    })
    GK_CHECK_LAUNCH("branch_merge");
    return GK_OK;
}

GK_EXPORT int gk_causal_conv(const float* a, const float* w, float* state, const int* tok_pos, const int* tok_seq,
                             const int* cu_q, const int* slots, void* out, int out_dtype, int n_tokens, int width, int taps,
                             int update_single_token_state, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(out_dtype), "causal_conv: bad dtype code");
    GK_REQUIRE(n_tokens >= 0 && width > 0 && taps >= 1, "causal_conv: bad sizes");
    GK_REQUIRE(taps == 1 || state != nullptr, "causal_conv: more than one tap needs a state");
    const long long total = (long long)n_tokens * width;
    if (total == 0) return GK_OK;
    const int threads = 256;
    if (width % 4 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)state & 15) == 0 && ((uintptr_t)w & 15) == 0) {
        const long long blocks4 = (total / 4 + threads - 1) / threads;
        GK_REQUIRE(blocks4 < 2147483647LL, "causal_conv: too many elements");
        GK_DISPATCH_DTYPE(out_dtype, TO, {
            gk_launch(causal_conv_x4_kernel<TO>, dim3((unsigned)blocks4), dim3(threads), 0, (cudaStream_t)stream, a, w, state, tok_pos,
                      tok_seq, cu_q, slots, (TO*)out, n_tokens, width, taps, update_single_token_state);
        })
        GK_CHECK_LAUNCH("causal_conv");
        return GK_OK;
    }
    const long long blocks = (total + threads - 1) / threads;
    GK_REQUIRE(blocks < 2147483647LL, "causal_conv: too many elements");
    GK_DISPATCH_DTYPE(out_dtype, TO, {
        gk_launch(causal_conv_kernel<TO>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, a, w, state, tok_pos,
                  tok_seq, cu_q, slots, (TO*)out, n_tokens, width, taps, update_single_token_state);
    })
    GK_CHECK_LAUNCH("causal_conv");
    return GK_OK;
}

GK_EXPORT int gk_conv_state(const float* a, float* state, const int* cu_q, const int* slots, int n_seqs, int width, int taps,
                            void* stream) {
    GK_REQUIRE(n_seqs >= 0 && width > 0 && taps >= 1, "conv_state: bad sizes");
    const long long total = (long long)n_seqs * width;
    if (total == 0 || taps == 1) return GK_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    gk_launch(conv_state_kernel, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, a, state, cu_q, slots, n_seqs,
              width, taps);
    GK_CHECK_LAUNCH("conv_state");
    return GK_OK;
}

GK_EXPORT int gk_gelu_tanh(const void* in, void* out, int dtype, long long total, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "gelu_tanh: bad dtype %d", dtype);
    GK_REQUIRE(total >= 0, "gelu_tanh: bad size");
    if (total == 0) return GK_OK;
    const int threads = 256;
    if (dtype == GK_BF16 && total % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const long long pieces = total / 8, blocks8 = (pieces + threads - 1) / threads;
        GK_REQUIRE(blocks8 < 2147483647LL, "gelu_tanh: too many elements");
        gk_launch(gelu_tanh_bf16x8_kernel, dim3((unsigned)blocks8), dim3(threads), 0, (cudaStream_t)stream, (const uint4*)in, (uint4*)out,
                  pieces);
        GK_CHECK_LAUNCH("gelu_tanh");
        return GK_OK;
    }
    const long long blocks = (total + threads - 1) / threads;
    GK_REQUIRE(blocks < 2147483647LL, "gelu_tanh: too many elements");
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(gelu_tanh_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, (const T*)in, (T*)out,
                  total);
    })
    GK_CHECK_LAUNCH("gelu_tanh");
    return GK_OK;
}
