// A feed-forward of many small gated experts of which every token uses a few.
//
//   route        z = W_r h in 32-bit (a warp per token and eight experts), then, a warp per token: s = sigmoid(z),
//                choice = s + correction.  The experts form equal groups of neighbours; a group's score is the sum of its
//                two largest choice scores and only the experts of the best `keep` groups may be chosen.  The `top`
//                largest choice scores among them are chosen (ties: the lower index); a chosen expert's weight is its s
//                (without the correction) times a constant.
//                With `logits` = 1 the score is the logit itself plus a stored bias, s = z + b (no sigmoid, choice by s),
//                and the chosen experts' weights are the softmax over the chosen scores alone, times the constant.
//   experts_up   act[pair] = silu(W_gate[e] h_t) * (W_up[e] h_t) for every pair (token, chosen expert)
//   experts_down out_t = add_t + sum over the token's pairs, in the order they were chosen, of weight * W_down[e] act[pair]
//                (32-bit result: it is what goes into the residual stream)
//
// The two expert kernels take a pair at a time, one warp per output row: the path of single-token steps, of 32-bit
// runs and of sizes the tensor-core path does not take.  A token's result depends on the token alone.
//
//   sort, gather_rows, combine   many-token steps: the pairs put in the order of their experts, the tokens' rows copied
//                into that order (each expert's rows then go through one tensor-core product, made by the caller), and
//                the weighted sum of a token's expert outputs in the order the experts were chosen

#include "common.cuh"

namespace {

constexpr int ROUTE_WARPS = 4;


// z[t, e] = h_t . w_router[e] in 32-bit.  One warp per (SCORE_TOKENS tokens, SCORE_EXPERTS experts): four and eight where
// tokens are many (a router row is fetched once for four tokens; eight tokens a warp measured slower: 66 against 60 us
// for 2,048 tokens of 1,024 and 32 experts), four and two where they are few and the launch would otherwise be a handful
// of warps; a lane sums its elements of a row in index order and the lanes meet in the fixed order of warp_sum, so a
// score depends on the token's row alone.
template <typename T, int SCORE_EXPERTS, int SCORE_TOKENS>
__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_scores_kernel(const T* __restrict__ h, const float* __restrict__ w_router,
                                                                        float* __restrict__ z, int n_tokens, int width, int n_experts) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int parts = (n_experts + SCORE_EXPERTS - 1) / SCORE_EXPERTS;
    const int token_groups = (n_tokens + SCORE_TOKENS - 1) / SCORE_TOKENS;
    const long long unit = (long long)blockIdx.x * ROUTE_WARPS + warp;
    if (unit >= (long long)token_groups * parts) return;
    const int t0 = (int)(unit / parts) * SCORE_TOKENS, e0 = (int)(unit % parts) * SCORE_EXPERTS;
    float acc[SCORE_TOKENS][SCORE_EXPERTS];
#pragma unroll
    for (int a = 0; a < SCORE_TOKENS; ++a)
#pragma unroll
        for (int j = 0; j < SCORE_EXPERTS; ++j) acc[a][j] = 0.f;
#pragma unroll 4
    for (int i = lane; i < width; i += 32) {
        float xv[SCORE_TOKENS], wv[SCORE_EXPERTS];
#pragma unroll
        for (int a = 0; a < SCORE_TOKENS; ++a) xv[a] = t0 + a < n_tokens ? to_float(h[(size_t)(t0 + a) * width + i]) : 0.f;
#pragma unroll
        for (int j = 0; j < SCORE_EXPERTS; ++j) wv[j] = e0 + j < n_experts ? w_router[(size_t)(e0 + j) * width + i] : 0.f;
#pragma unroll
        for (int a = 0; a < SCORE_TOKENS; ++a)
#pragma unroll
            for (int j = 0; j < SCORE_EXPERTS; ++j) acc[a][j] = fmaf(xv[a], wv[j], acc[a][j]);
    }
#pragma unroll
    for (int a = 0; a < SCORE_TOKENS; ++a)
#pragma unroll
        for (int j = 0; j < SCORE_EXPERTS; ++j) {
            const float sum = warp_sum(acc[a][j]);
            if (lane == 0 && t0 + a < n_tokens && e0 + j < n_experts) z[(size_t)(t0 + a) * n_experts + e0 + j] = sum;
        }
}

// The choice from the scores: one warp per token.
__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_choose_kernel(
    const float* __restrict__ z, const float* __restrict__ correction, int* __restrict__ ids, float* __restrict__ weights,
    int n_tokens, int n_experts, int top, int n_groups, int keep, float scale, int logits) {
    extern __shared__ float route_smem[];  // per warp: s [E] | choice [E] | group score [n_groups]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= n_tokens) return;
    float* s = route_smem + (size_t)warp * (2 * n_experts + n_groups);
    float* choice = s + n_experts;
    float* group_score = choice + n_experts;
    for (int e = lane; e < n_experts; e += 32) {
        const float ze = z[(size_t)t * n_experts + e];
        const float sg = logits ? ze + correction[e] : 1.f / (1.f + expf(-ze));
        s[e] = sg;
        choice[e] = logits ? sg : sg + correction[e];
    }
    __syncwarp();
    const int per = n_experts / n_groups;
    if (n_groups > 1 && keep < n_groups) {
        for (int gidx = lane; gidx < n_groups; gidx += 32) {
            float first = -INFINITY, second = -INFINITY;
            for (int e = gidx * per; e < (gidx + 1) * per; ++e) {
                const float c = choice[e];
                if (c > first) { second = first; first = c; }
                else if (c > second) second = c;
            }
            group_score[gidx] = per > 1 ? first + second : first;
        }
        __syncwarp();
        // the groups that are not among the best `keep` lose their experts
        for (int gidx = lane; gidx < n_groups; gidx += 32) {
            int better = 0;
            for (int o = 0; o < n_groups; ++o)
                better += (group_score[o] > group_score[gidx]) || (group_score[o] == group_score[gidx] && o < gidx);
            if (better >= keep)
                for (int e = gidx * per; e < (gidx + 1) * per; ++e) choice[e] = -INFINITY;
        }
        __syncwarp();
    }
    for (int pick = 0; pick < top; ++pick) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;  // nothing left to choose from: cannot happen when top <= allowed experts
        if (lane == 0) {
            ids[(size_t)t * top + pick] = arg;
            weights[(size_t)t * top + pick] = logits ? s[arg] : s[arg] * scale;
            choice[arg] = -INFINITY;
        }
        __syncwarp();
    }
    if (logits && lane == 0) {
        // softmax over the chosen scores, in the order they were chosen (the first is the largest)
        float* w = weights + (size_t)t * top;
        const float largest = w[0];
        float sum = 0.f;
        for (int pick = 0; pick < top; ++pick) sum += expf(w[pick] - largest);
        for (int pick = 0; pick < top; ++pick) w[pick] = expf(w[pick] - largest) / sum * scale;
    }
}

template <typename TW>
__device__ __forceinline__ float dot_smem(const float* __restrict__ x, const TW* __restrict__ w, int n, int lane);

template <>
__device__ __forceinline__ float dot_smem<float>(const float* __restrict__ x, const float* __restrict__ w, int n, int lane) {
    float acc = 0.f;
    if ((n & 3) == 0) {
#pragma unroll 4
        for (int i = lane * 4; i < n; i += 128) {
            const float4 a = *reinterpret_cast<const float4*>(w + i);
            acc = fmaf(x[i], a.x, acc); acc = fmaf(x[i + 1], a.y, acc); acc = fmaf(x[i + 2], a.z, acc); acc = fmaf(x[i + 3], a.w, acc);
        }
    } else {
        for (int i = lane; i < n; i += 32) acc = fmaf(x[i], w[i], acc);
    }
    return warp_sum(acc);
}

template <>
__device__ __forceinline__ float dot_smem<__nv_bfloat16>(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w, int n, int lane) {
    float acc = 0.f;
    if ((n & 7) == 0) {
#pragma unroll 4
        for (int i = lane * 8; i < n; i += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float2 f = __bfloat1622float2(p[c]);
                acc = fmaf(x[i + 2 * c], f.x, acc);
                acc = fmaf(x[i + 2 * c + 1], f.y, acc);
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) acc = fmaf(x[i], __bfloat162float(w[i]), acc);
    }
    return warp_sum(acc);
}

// A lane's share of NR dot products of one vector in shared memory with NR rows in memory, summed in index order; the
// rows' loads are independent, so all of them are on their way together.  The caller finishes each with warp_sum.
template <typename TW, int NR>
__device__ __forceinline__ void dot_parts(const float* __restrict__ x, const TW* const (&rows)[NR], int n, int lane, float (&acc)[NR]) {
#pragma unroll
    for (int j = 0; j < NR; ++j) acc[j] = 0.f;
    constexpr int VEC = 16 / sizeof(TW);
    if (n % VEC == 0) {
#pragma unroll 2
        for (int i = lane * VEC; i < n; i += 32 * VEC) {
            uint4 raw[NR];
#pragma unroll
            for (int j = 0; j < NR; ++j) raw[j] = *reinterpret_cast<const uint4*>(rows[j] + i);
#pragma unroll
            for (int j = 0; j < NR; ++j) {
                if constexpr (sizeof(TW) == 2) {
                    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float2 f = __bfloat1622float2(p[c]);
                        acc[j] = fmaf(x[i + 2 * c], f.x, acc[j]);
                        acc[j] = fmaf(x[i + 2 * c + 1], f.y, acc[j]);
                    }
                } else {
                    const float* f = reinterpret_cast<const float*>(&raw[j]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[j] = fmaf(x[i + c], f[c], acc[j]);
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32)
#pragma unroll
            for (int j = 0; j < NR; ++j) acc[j] = fmaf(x[i], to_float(rows[j][i]), acc[j]);
    }
}

constexpr int UP_WARPS = 8;

// grid (pairs, chunks of ff): w_gate_up [E, 2, ff, width] (gate rows then up rows of an expert)
template <typename T, typename TW>
__global__ void __launch_bounds__(UP_WARPS * 32) experts_up_kernel(
    const T* __restrict__ h, const TW* __restrict__ w_gate_up, const int* __restrict__ ids, T* __restrict__ act, int width,
    int ff, int top, int rows_per_block) {
    extern __shared__ __align__(16) float xs[];  // width
    pdl_launch_dependents();
    pdl_wait();
    const int pair = blockIdx.x, t = pair / top;
    const int e = ids[pair];
    for (int i = threadIdx.x; i < width; i += UP_WARPS * 32) xs[i] = to_float(h[(size_t)t * width + i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TW* wg = w_gate_up + (size_t)e * 2 * ff * width;
    const TW* wu = wg + (size_t)ff * width;
    const int f0 = blockIdx.y * rows_per_block;
    const int f_end = min(ff, f0 + rows_per_block);
    int f = f0 + warp;
    for (; f + UP_WARPS < f_end; f += 2 * UP_WARPS) {  // two rows of gate and of up at once: four rows' loads in flight
        const TW* const rows[4] = {wg + (size_t)f * width, wu + (size_t)f * width, wg + (size_t)(f + UP_WARPS) * width,
                                   wu + (size_t)(f + UP_WARPS) * width};
        float part[4];
        dot_parts<TW, 4>(xs, rows, width, lane, part);
#pragma unroll
        for (int j = 0; j < 4; ++j) part[j] = warp_sum(part[j]);
        if (lane == 0) {
            act[(size_t)pair * ff + f] = from_float<T>(part[0] / (1.f + expf(-part[0])) * part[1]);
            act[(size_t)pair * ff + f + UP_WARPS] = from_float<T>(part[2] / (1.f + expf(-part[2])) * part[3]);
        }
    }
    for (; f < f_end; f += UP_WARPS) {
        const TW* const rows[2] = {wg + (size_t)f * width, wu + (size_t)f * width};
        float part[2];
        dot_parts<TW, 2>(xs, rows, width, lane, part);
        const float gate = warp_sum(part[0]), up = warp_sum(part[1]);
        if (lane == 0) act[(size_t)pair * ff + f] = from_float<T>(gate / (1.f + expf(-gate)) * up);
    }
}

// grid (tokens, chunks of width): w_down [E, width, ff]
template <typename T, typename TW>
__global__ void __launch_bounds__(UP_WARPS * 32) experts_down_kernel(
    const T* __restrict__ act, const TW* __restrict__ w_down, const int* __restrict__ ids, const float* __restrict__ weights,
    const T* __restrict__ add, float* __restrict__ out, int width, int ff, int top, int rows_per_block) {
    extern __shared__ __align__(16) float as[];  // top * ff
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < top * ff; i += UP_WARPS * 32) as[i] = to_float(act[(size_t)t * top * ff + i]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = blockIdx.y * rows_per_block;
    for (int c = c0 + warp; c < min(width, c0 + rows_per_block); c += UP_WARPS) {
        float acc = add != nullptr ? to_float(add[(size_t)t * width + c]) : 0.f;
        int kk = 0;
        for (; kk + 1 < top; kk += 2) {  // two experts' rows in flight; the sum still takes them in the order they were chosen
            const int e0 = ids[(size_t)t * top + kk], e1 = ids[(size_t)t * top + kk + 1];
            const float d0 = dot_smem<TW>(as + (size_t)kk * ff, w_down + ((size_t)e0 * width + c) * ff, ff, lane);
            const float d1 = dot_smem<TW>(as + (size_t)(kk + 1) * ff, w_down + ((size_t)e1 * width + c) * ff, ff, lane);
            acc = fmaf(weights[(size_t)t * top + kk], d0, acc);
            acc = fmaf(weights[(size_t)t * top + kk + 1], d1, acc);
        }
        if (kk < top) {
            const int e = ids[(size_t)t * top + kk];
            const float d = dot_smem<TW>(as + (size_t)kk * ff, w_down + ((size_t)e * width + c) * ff, ff, lane);
            acc = fmaf(weights[(size_t)t * top + kk], d, acc);
        }
        if (lane == 0) out[(size_t)t * width + c] = acc;
    }
}

// ---- pairs in the order of their experts, for products that take all rows of an expert at once
// One block.  ends[e] = one past the last place of expert e (cumulative counts); place_of[pair] = the pair's place in
// that order; pair_at[place] = the pair that stands there.  Which of an expert's pairs gets which of its places is
// settled by atomic counters and may differ from run to run; a row's product does not depend on its place.
constexpr int SORT_THREADS = 1024;

__global__ void __launch_bounds__(SORT_THREADS) experts_sort_kernel(const int* __restrict__ ids, int n_pairs, int n_experts,
                                                                    int* __restrict__ ends, int* __restrict__ place_of,
                                                                    int* __restrict__ pair_at) {
    extern __shared__ int sort_smem[];  // counts [E] | starts [E]
    pdl_launch_dependents();
    int* counts = sort_smem;
    int* starts = sort_smem + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += SORT_THREADS) counts[e] = 0;
    __syncthreads();
    pdl_wait();
    for (int i = threadIdx.x; i < n_pairs; i += SORT_THREADS) atomicAdd(&counts[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < n_experts; ++e) {
            starts[e] = at;
            at += counts[e];
            ends[e] = at;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += SORT_THREADS) {
        const int place = atomicAdd(&starts[ids[i]], 1);
        place_of[i] = place;
        pair_at[place] = i;
    }
}

// out[place] = x[pair_at[place] / top]: the rows of the tokens in the order of their experts
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ pair_at, T* __restrict__ out, int width, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t place = blockIdx.x;
    const T* src = x + (size_t)(pair_at[place] / top) * width;
    T* dst = out + place * width;
    if ((width * sizeof(T)) % 16 == 0) {
        const int n16 = width * (int)sizeof(T) / 16;
        for (int i = threadIdx.x; i < n16; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

// out_t = add_t + sum_k weights[t, k] * y[place_of[t, k]] in the order the experts were chosen (32-bit)
template <typename T>
__global__ void experts_combine_kernel(const T* __restrict__ y, const int* __restrict__ place_of, const float* __restrict__ weights,
                                       const T* __restrict__ add, float* __restrict__ out, int width, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = add != nullptr ? to_float(add[t * width + c]) : 0.f;
        for (int kk = 0; kk < top; ++kk)
            acc = fmaf(weights[t * top + kk], to_float(y[(size_t)place_of[t * top + kk] * width + c]), acc);
        out[t * width + c] = acc;
    }
}

}  // namespace

GK_EXPORT int gk_experts_sort(const int* ids, int n_pairs, int n_experts, int* ends, int* place_of, int* pair_at, void* stream) {
    GK_REQUIRE(n_pairs >= 0 && n_experts > 0 && n_experts <= 4096, "experts_sort: bad sizes");
    gk_launch(experts_sort_kernel, dim3(1), dim3(SORT_THREADS), (size_t)2 * n_experts * sizeof(int), (cudaStream_t)stream, ids, n_pairs,
              n_experts, ends, place_of, pair_at);
    GK_CHECK_LAUNCH("experts_sort");
    return GK_OK;
}

GK_EXPORT int gk_gather_rows(const void* x, int dtype, const int* pair_at, void* out, int n_places, int width, int top, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && width > 0 && top > 0, "gather_rows: bad arguments");
    if (n_places == 0) return GK_OK;
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(gather_rows_kernel<T>, dim3(n_places), dim3(128), 0, (cudaStream_t)stream, (const T*)x, pair_at, (T*)out, width, top);
    })
    GK_CHECK_LAUNCH("gather_rows");
    return GK_OK;
}

GK_EXPORT int gk_experts_combine(const void* y, int dtype, const int* place_of, const float* weights, const void* add, float* out,
                                 int n_tokens, int width, int top, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && width > 0 && top > 0, "experts_combine: bad arguments");
    if (n_tokens == 0) return GK_OK;
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(experts_combine_kernel<T>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, (const T*)y, place_of, weights,
                  (const T*)add, out, width, top);
    })
    GK_CHECK_LAUNCH("experts_combine");
    return GK_OK;
}

GK_EXPORT int gk_route_groups(const void* h, int dtype, const float* w_router, const float* correction, float* z, int* ids,
                              float* weights, int n_tokens, int width, int n_experts, int top, int n_groups, int keep, float scale, int logits,
                              void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "route_groups: bad dtype %d", dtype);
    GK_REQUIRE(n_experts > 0 && top > 0 && top <= n_experts, "route_groups: %d of %d experts", top, n_experts);
    GK_REQUIRE(n_groups >= 1 && n_experts % n_groups == 0 && keep >= 1 && keep <= n_groups, "route_groups: %d groups, %d kept, %d experts",
               n_groups, keep, n_experts);
    GK_REQUIRE(top <= keep * (n_experts / n_groups), "route_groups: %d experts cannot come from %d groups of %d", top, keep,
               n_experts / n_groups);
    if (n_tokens == 0) return GK_OK;
    const size_t smem = (size_t)ROUTE_WARPS * (2 * n_experts + n_groups) * sizeof(float);
    GK_REQUIRE(smem <= 48 * 1024, "route_groups: too many experts (%d)", n_experts);
    cudaStream_t s = (cudaStream_t)stream;
    const bool many = (long long)((n_tokens + 7) / 8) * ((n_experts + 7) / 8) >= 512;
    const int per_warp = many ? 8 : 2;
    const int token_groups = (n_tokens + 3) / 4;
    const long long units = (long long)token_groups * ((n_experts + per_warp - 1) / per_warp);
    GK_REQUIRE(units / ROUTE_WARPS < 2147483647LL, "route_groups: too many tokens");
    const dim3 score_grid((unsigned)((units + ROUTE_WARPS - 1) / ROUTE_WARPS));
    GK_DISPATCH_DTYPE(dtype, T, {
        if (per_warp == 8)
            gk_launch(route_scores_kernel<T, 8, 4>, score_grid, dim3(ROUTE_WARPS * 32), 0, s, (const T*)h, w_router, z, n_tokens, width, n_experts);
        else
            gk_launch(route_scores_kernel<T, 2, 4>, score_grid, dim3(ROUTE_WARPS * 32), 0, s, (const T*)h, w_router, z, n_tokens, width, n_experts);
    })
    GK_CHECK_LAUNCH("route_scores");
    gk_launch(route_choose_kernel, dim3((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, s, (const float*)z,
              correction, ids, weights, n_tokens, n_experts, top, n_groups, keep, scale, logits);
    GK_CHECK_LAUNCH("route_groups");
    return GK_OK;
}

GK_EXPORT int gk_experts_up(const void* h, int dtype, const void* w_gate_up, int w_dtype, const int* ids, void* act, int n_tokens,
                            int width, int ff, int top, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && GK_VALID_DTYPE(w_dtype), "experts_up: bad dtype");
    GK_REQUIRE(width > 0 && ff > 0 && top > 0, "experts_up: bad sizes");
    if (n_tokens == 0) return GK_OK;
    const size_t smem = (size_t)width * sizeof(float);
    GK_REQUIRE(smem <= 200 * 1024, "experts_up: rows of %d are longer than the kernel stages", width);
    // few pairs: cut the expert's rows over more blocks, so that a single token still finds every SM a share
    const long long pairs = (long long)n_tokens * top;
    int chunks = 1;
    while (pairs * chunks < 592 && ff / (chunks * 2) >= UP_WARPS) chunks *= 2;
    const int rows = (ff + chunks - 1) / chunks;
    GK_REQUIRE(pairs < 2147483647LL, "experts_up: too many pairs");
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(dtype, T, {
        GK_DISPATCH_DTYPE(w_dtype, TW, {
            if (smem > 48 * 1024) cudaFuncSetAttribute(experts_up_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            gk_launch(experts_up_kernel<T, TW>, dim3((unsigned)pairs, (ff + rows - 1) / rows), dim3(UP_WARPS * 32), smem, s, (const T*)h,
                      (const TW*)w_gate_up, ids, (T*)act, width, ff, top, rows);
        })
    })
    GK_CHECK_LAUNCH("experts_up");
    return GK_OK;
}

GK_EXPORT int gk_experts_down(const void* act, int dtype, const void* w_down, int w_dtype, const int* ids, const float* weights,
                              const void* add, float* out, int n_tokens, int width, int ff, int top, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && GK_VALID_DTYPE(w_dtype), "experts_down: bad dtype");
    GK_REQUIRE(width > 0 && ff > 0 && top > 0, "experts_down: bad sizes");
    if (n_tokens == 0) return GK_OK;
    const size_t smem = (size_t)top * ff * sizeof(float);
    GK_REQUIRE(smem <= 200 * 1024, "experts_down: %d experts of %d are more than the kernel stages", top, ff);
    int chunks = 1;
    while ((long long)n_tokens * chunks < 592 && width / (chunks * 2) >= UP_WARPS) chunks *= 2;
    const int rows = (width + chunks - 1) / chunks;
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(dtype, T, {
        GK_DISPATCH_DTYPE(w_dtype, TW, {
            if (smem > 48 * 1024) cudaFuncSetAttribute(experts_down_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            gk_launch(experts_down_kernel<T, TW>, dim3(n_tokens, (width + rows - 1) / rows), dim3(UP_WARPS * 32), smem, s, (const T*)act,
                      (const TW*)w_down, ids, weights, (const T*)add, out, width, ff, top, rows);
        })
    })
    GK_CHECK_LAUNCH("experts_down");
    return GK_OK;
}
