// Linear attention with a fixed decay per head, and what stands between the projections and it.
//
//   heads_prepare:  a warp per (token, head) of the packed projection q | k | v: optional SiLU (on q and k, on v),
//                   rotation by position of the first `rot` entries of a q or k head (entry i paired with i + rot/2;
//                   cosines and sines from tables of rot/2 angles a position), then optional division of a q or k
//                   head by its root mean square (eps inside the root, no weight), then a constant on k.  With flag 8
//                   every value head turns by its own position over ALL of its dv entries (entry m paired with
//                   m + dv/2, tables of dv/2 angles a position of their own), so that it is cached turned.  The results
//                   go either to 32-bit arrays q, k [T, heads, d] and v [T, heads, dv] (what a recurrence reads), or
//                   q to an array of the run's type and k, v into the pages of the cache (what attention reads).
//   decay_scan:     per (sequence, head):  S <- decay_h S + k_t v_t^T ;  o_t = S^T q_t,  S [d, dv] 32-bit, read from
//                   the sequence's slot at the start of the step and written back at its end.  Prompts, portions and
//                   single tokens take the same path; a token's sums have the same order in all of them.
//   group_norm_gate: rows cut into groups (a head, or all heads together) that are divided by their root mean
//                   square, multiplied by an optional weight and by sigmoid or SiLU of a gate.
//
// Everything is 32-bit except the projection that is read and the activations that are handed on.

#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

constexpr int PREP_WARPS = 8;
constexpr int PREP_MAX = 16;  // heads of up to 512 entries

// flags: 1 SiLU on q and k, 2 SiLU on v, 4 unit root mean square of q and k, 8 values turned by position
template <typename T, typename TQ>
__global__ void __launch_bounds__(PREP_WARPS * 32) heads_prepare_kernel(
    const T* __restrict__ proj, long long ld, int q_at, int k_at, int v_at, int n_q, int n_k, int d, int dv, int flags,
    int rot, const float* __restrict__ cos_t, const float* __restrict__ sin_t, const float* __restrict__ v_cos,
    const float* __restrict__ v_sin, float unit_eps, float k_scale, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
    TQ* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ v_out, T* __restrict__ k_pages,
    T* __restrict__ v_pages, const int* __restrict__ block_table, int max_pages, int page_size, int write_kv, long long n_items) {
    extern __shared__ float stage[];  // PREP_WARPS * max(d, dv)
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * PREP_WARPS + warp;
    if (item >= n_items) return;
    const int per_token = n_q + 2 * n_k;
    const int t = (int)(item / per_token);
    int head = (int)(item - (long long)t * per_token);
    const int kind = head < n_q ? 0 : head < n_q + n_k ? 1 : 2;  // q, k, v
    head -= kind == 0 ? 0 : kind == 1 ? n_q : n_q + n_k;
    const int width = kind == 2 ? dv : d;
    const T* src = proj + (size_t)t * ld + (kind == 0 ? q_at : kind == 1 ? k_at : v_at) + (size_t)head * width;
    const bool to_pages = k_pages != nullptr;
    if (to_pages && kind != 0 && !write_kv) return;
    float x[PREP_MAX];
    const bool act = kind == 2 ? (flags & 2) != 0 : (flags & 1) != 0;
#pragma unroll
    for (int c = 0; c < PREP_MAX; ++c) {
        const int i = lane + 32 * c;
        x[c] = 0.f;
        if (i < width) {
            x[c] = to_float(src[i]);
            if (act) x[c] = silu_f(x[c]);
        }
    }
    const int pos = tok_pos[t];
    if (kind != 2) {
        if (rot > 0) {
            float* mine = stage + (size_t)warp * (d > dv ? d : dv);
#pragma unroll
            for (int c = 0; c < PREP_MAX; ++c) {
                const int i = lane + 32 * c;
                if (i < width) mine[i] = x[c];
            }
            __syncwarp();
            const int half = rot >> 1;
            const float* cs = cos_t + (size_t)pos * half;
            const float* sn = sin_t + (size_t)pos * half;
#pragma unroll
            for (int c = 0; c < PREP_MAX; ++c) {
                const int i = lane + 32 * c;
                if (i < half) x[c] = mine[i] * cs[i] - mine[i + half] * sn[i];
                else if (i < rot) x[c] = mine[i] * cs[i - half] + mine[i - half] * sn[i - half];
            }
        }
        if (flags & 4) {
            float ss = 0.f;
#pragma unroll
            for (int c = 0; c < PREP_MAX; ++c) ss = fmaf(x[c], x[c], ss);
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)d + unit_eps);
#pragma unroll
            for (int c = 0; c < PREP_MAX; ++c) x[c] *= r;
        }
        if (kind == 1 && k_scale != 1.f) {
#pragma unroll
            for (int c = 0; c < PREP_MAX; ++c) x[c] *= k_scale;
        }
    }
    if (kind == 2 && (flags & 8)) {
        float* mine = stage + (size_t)warp * (d > dv ? d : dv);
#pragma unroll
        for (int c = 0; c < PREP_MAX; ++c) {
            const int i = lane + 32 * c;
            if (i < width) mine[i] = x[c];
        }
        __syncwarp();
        const int half = dv >> 1;
        const float* cs = v_cos + (size_t)pos * half;
        const float* sn = v_sin + (size_t)pos * half;
#pragma unroll
        for (int c = 0; c < PREP_MAX; ++c) {
            const int i = lane + 32 * c;
            if (i < half) x[c] = mine[i] * cs[i] - mine[i + half] * sn[i];
            else if (i < 2 * half) x[c] = mine[i] * cs[i - half] + mine[i - half] * sn[i - half];
        }
    }
    if (kind == 0) {
        TQ* dst = q_out + ((size_t)t * n_q + head) * d;
#pragma unroll
        for (int c = 0; c < PREP_MAX; ++c) {
            const int i = lane + 32 * c;
            if (i < width) dst[i] = from_float<TQ>(x[c]);
        }
        return;
    }
    if (!to_pages) {
        float* dst = (kind == 1 ? k_out : v_out) + ((size_t)t * n_k + head) * width;
#pragma unroll
        for (int c = 0; c < PREP_MAX; ++c) {
            const int i = lane + 32 * c;
            if (i < width) dst[i] = x[c];
        }
        return;
    }
    const int page = block_table[(size_t)slots[tok_seq[t]] * max_pages + pos / page_size];
    T* dst = (kind == 1 ? k_pages : v_pages) + (((size_t)page * n_k + head) * page_size + pos % page_size) * width;
#pragma unroll
    for (int c = 0; c < PREP_MAX; ++c) {
        const int i = lane + 32 * c;
        if (i < width) dst[i] = from_float<T>(x[c]);
    }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

constexpr int SCAN_LANES = 8;      // lanes that share a column of the state
constexpr int SCAN_MAX_COLS = 32;  // columns a block at most (256 threads)

// A column of S never meets another column, so the work is cut by (sequence, head, group of columns); a column's d
// entries are spread over eight adjacent lanes, R consecutive rows a lane.  The step's tokens come through a two-stage
// cp.async ring, TB at a time.  A token costs a lane 2 R multiply-adds and three shuffles.
template <int R, int TB>
__global__ void __launch_bounds__(SCAN_LANES * SCAN_MAX_COLS) decay_scan_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ decay,
    float* __restrict__ state /* [slots, H, d, dv] */, float* __restrict__ out /* [T, H, dv] */, const int* __restrict__ cu_q,
    const int* __restrict__ slots, int n_heads, int d, int dv) {
    constexpr int PIECE = R == 4 ? 4 : R + 4, VEC = SCAN_LANES * PIECE;  // a lane's piece starts a bank group apart from its neighbours'
    __shared__ __align__(16) float sq[2][TB][VEC], sk[2][TB][VEC];
    __shared__ __align__(16) float sv[2][TB][SCAN_MAX_COLS];
    pdl_launch_dependents();
    const int n_threads = blockDim.x, n_cols = n_threads / SCAN_LANES;
    const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * n_cols;
    const int sub = threadIdx.x % SCAN_LANES, col = col0 + threadIdx.x / SCAN_LANES;
    const bool live = col < dv;
    for (int i = threadIdx.x; i < 2 * TB * VEC; i += n_threads) {  // the pieces beyond d stay zero in every stage
        (&sq[0][0][0])[i] = 0.f;
        (&sk[0][0][0])[i] = 0.f;
    }
    __syncthreads();
    const float gamma = decay[head];
    pdl_wait();
    const int t0 = cu_q[seq], n = cu_q[seq + 1] - t0;
    float* my_state = state + (((size_t)slots[seq] * n_heads + head) * d) * dv + col;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = sub * R + r;
        S[r] = (live && row < d) ? my_state[(size_t)row * dv] : 0.f;
    }
    const int quads = d / 4;
    auto stage = [&](int buf, int first) {
        const int count = min(TB, n - first);
        if (d & 3) {  // rows that do not start on 16 bytes: one entry a copy
            for (int i = threadIdx.x; i < count * d; i += n_threads) {
                const int tt = i / d, c = i - tt * d;
                const int at = (c / R) * PIECE + c % R;
                const size_t tok = (size_t)(t0 + first + tt);
                cp_async4(&sq[buf][tt][at], q + (tok * n_heads + head) * d + c);
                cp_async4(&sk[buf][tt][at], k + (tok * n_heads + head) * d + c);
            }
        } else
        for (int i = threadIdx.x; i < count * quads; i += n_threads) {
            const int tt = i / quads, c4 = (i - tt * quads) * 4;
            const int at = (c4 / R) * PIECE + c4 % R;
            const size_t tok = (size_t)(t0 + first + tt);
            cp_async16(&sq[buf][tt][at], q + (tok * n_heads + head) * d + c4);
            cp_async16(&sk[buf][tt][at], k + (tok * n_heads + head) * d + c4);
        }
        for (int i = threadIdx.x; i < count * n_cols; i += n_threads) {
            const int tt = i / n_cols, cc = i - tt * n_cols;
            if (col0 + cc < dv) cp_async4(&sv[buf][tt][cc], v + ((size_t)(t0 + first + tt) * n_heads + head) * dv + col0 + cc);
        }
        cp_async_commit();
    };
    stage(0, 0);
    int buf = 0;
    for (int first = 0; first < n; first += TB, buf ^= 1) {
        if (first + TB < n) {
            stage(buf ^ 1, first + TB);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int count = min(TB, n - first);
        float* out_at = out + ((size_t)(t0 + first) * n_heads + head) * dv + col;
        const float* v_at = &sv[buf][0][threadIdx.x / SCAN_LANES];
        const float4* pq = reinterpret_cast<const float4*>(&sq[buf][0][sub * PIECE]);
        const float4* pk = reinterpret_cast<const float4*>(&sk[buf][0][sub * PIECE]);
        const size_t out_step = (size_t)n_heads * dv;
#pragma unroll 2
        for (int tt = 0; tt < count; ++tt, out_at += out_step, v_at += SCAN_MAX_COLS, pq += VEC / 4, pk += VEC / 4) {
            const float vv = live ? *v_at : 0.f;
            float b4[4] = {0.f, 0.f, 0.f, 0.f};  // four partial sums: chains of R / 4 dependent operations
#pragma unroll
            for (int r4 = 0; r4 < R / 4; ++r4) {
                const float4 k4 = pk[r4], q4 = pq[r4];
                const float ks[4] = {k4.x, k4.y, k4.z, k4.w}, qs[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = 4 * r4 + e;
                    S[r] = fmaf(ks[e], vv, gamma * S[r]);
                    b4[e] = fmaf(S[r], qs[e], b4[e]);
                }
            }
            float b = (b4[0] + b4[1]) + (b4[2] + b4[3]);
#pragma unroll
            for (int o = 1; o < SCAN_LANES; o <<= 1) b += __shfl_xor_sync(0xffffffffu, b, o);
            if (live && sub == 0) *out_at = b;
        }
        __syncthreads();  // the stage is free for the load after next
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = sub * R + r;
        if (live && row < d) my_state[(size_t)row * dv] = S[r];
    }
}

// gate_kind: 0 sigmoid, 1 SiLU
template <typename T, typename TG>
__global__ void __launch_bounds__(256) group_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                              const TG* __restrict__ gate, long long ld_gate, T* __restrict__ out,
                                                              long long n_rows, int n_groups, int size, float eps, int gate_kind) {
    pdl_launch_dependents();
    pdl_wait();
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const long long t = row / n_groups;
    const int g = (int)(row - t * n_groups);
    const float* xr = x + (size_t)row * size;
    float ss = 0.f;
    for (int i = lane; i < size; i += 32) ss = fmaf(xr[i], xr[i], ss);
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)size + eps);
    const TG* gt = gate + (size_t)t * ld_gate + (size_t)g * size;
    for (int i = lane; i < size; i += 32) {
        const float z = to_float(gt[i]);
        float y = xr[i] * r;
        if (weight != nullptr) y *= weight[i];
        out[(size_t)row * size + i] = from_float<T>(y * (gate_kind == 0 ? sigmoid_f(z) : silu_f(z)));
    }
}

// The same for wide groups, a block per row: a warp alone would walk a row of a thousand entries in 32 dependent rounds.
template <typename T, typename TG>
__global__ void __launch_bounds__(256) group_norm_gate_wide_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                                   const TG* __restrict__ gate, long long ld_gate, T* __restrict__ out,
                                                                   int n_groups, int size, float eps, int gate_kind) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const long long row = blockIdx.x;
    const long long t = row / n_groups;
    const int g = (int)(row - t * n_groups);
    const float* xr = x + (size_t)row * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += 256) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum(ss, scratch);
    const float r = 1.f / sqrtf(ss / (float)size + eps);
    const TG* gt = gate + (size_t)t * ld_gate + (size_t)g * size;
    for (int i = threadIdx.x; i < size; i += 256) {
        const float z = to_float(gt[i]);
        float y = xr[i] * r;
        if (weight != nullptr) y *= weight[i];
        out[(size_t)row * size + i] = from_float<T>(y * (gate_kind == 0 ? sigmoid_f(z) : silu_f(z)));
    }
}

}  // namespace

GK_EXPORT int gk_heads_prepare(const void* proj, int dtype, long long ld, int q_at, int k_at, int v_at, int n_q, int n_k, int d,
                               int dv, int flags, int rot, const float* cos_t, const float* sin_t, const float* v_cos,
                               const float* v_sin, float unit_eps, float k_scale, const int* tok_pos, const int* tok_seq, const int* slots, void* q_out, int q_dtype, float* k_out,
                               float* v_out, void* k_pages, void* v_pages, const int* block_table, int max_pages, int page_size,
                               int write_kv, int n_tokens, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && GK_VALID_DTYPE(q_dtype), "heads_prepare: bad dtype");
    GK_REQUIRE(n_q > 0 && n_k > 0 && d > 0 && dv > 0 && n_tokens >= 0, "heads_prepare: bad sizes");
    GK_REQUIRE(d <= 32 * PREP_MAX && dv <= 32 * PREP_MAX, "heads_prepare: heads of %d / %d are more than a warp holds (%d)", d, dv, 32 * PREP_MAX);
    GK_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= d, "heads_prepare: %d rotated entries in heads of %d", rot, d);
    GK_REQUIRE(rot == 0 || (cos_t != nullptr && sin_t != nullptr), "heads_prepare: a rotation needs its tables");
    GK_REQUIRE(!(flags & 4) || unit_eps > 0.f, "heads_prepare: eps must be positive");
    GK_REQUIRE(!(flags & 8) || (v_cos != nullptr && v_sin != nullptr && dv % 2 == 0),
               "heads_prepare: turned values need their tables and an even size");
    const bool to_pages = k_pages != nullptr;
    GK_REQUIRE(to_pages ? (v_pages != nullptr && block_table != nullptr && page_size > 0 && q_dtype == dtype)
                        : (k_out != nullptr && v_out != nullptr && q_dtype == GK_F32),
               "heads_prepare: keys and values go either to pages (queries in the run's type) or to 32-bit arrays");
    if (n_tokens == 0) return GK_OK;
    const long long items = (long long)n_tokens * (n_q + 2 * n_k);
    const long long blocks = (items + PREP_WARPS - 1) / PREP_WARPS;
    GK_REQUIRE(blocks < 2147483647LL, "heads_prepare: too many tokens");
    const size_t smem = (size_t)PREP_WARPS * (d > dv ? d : dv) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(dtype, T, {
        if (to_pages) {
            gk_launch(heads_prepare_kernel<T, T>, dim3((unsigned)blocks), dim3(PREP_WARPS * 32), smem, s, (const T*)proj, ld, q_at,
                      k_at, v_at, n_q, n_k, d, dv, flags, rot, cos_t, sin_t, v_cos, v_sin, unit_eps, k_scale, tok_pos, tok_seq, slots, (T*)q_out,
                      (float*)nullptr, (float*)nullptr, (T*)k_pages, (T*)v_pages, block_table, max_pages, page_size, write_kv, items);
        } else {
            gk_launch(heads_prepare_kernel<T, float>, dim3((unsigned)blocks), dim3(PREP_WARPS * 32), smem, s, (const T*)proj, ld,
                      q_at, k_at, v_at, n_q, n_k, d, dv, flags, rot, cos_t, sin_t, v_cos, v_sin, unit_eps, k_scale, tok_pos, tok_seq, slots,
                      (float*)q_out, k_out, v_out, (T*)nullptr, (T*)nullptr, block_table, max_pages, page_size, write_kv, items);
        }
    })
    GK_CHECK_LAUNCH("heads_prepare");
    return GK_OK;
}

GK_EXPORT int gk_decay_scan(const float* q, const float* k, const float* v, const float* decay, float* state, float* out,
                            const int* cu_q, const int* slots, int n_seqs, int n_heads, int d, int dv, void* stream) {
    GK_REQUIRE(n_heads > 0 && n_heads <= 65535 && n_seqs >= 0 && n_seqs <= 65535, "decay_scan: bad counts");
    GK_REQUIRE(d > 0 && d <= 256, "decay_scan: key size %d must be at most 256", d);
    GK_REQUIRE(dv > 0, "decay_scan: bad value size");
    if (n_seqs == 0) return GK_OK;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (sms <= 0) sms = 148;
    }
    // fewer columns a block while the (sequence, head, column group) pairs do not fill the device twice: a column's
    // sums do not depend on the block's shape
    int cols = SCAN_MAX_COLS;
    while (cols > 4 && (long long)n_seqs * n_heads * ((dv + cols - 1) / cols) < 2LL * sms) cols /= 2;
    const dim3 grid((dv + cols - 1) / cols, n_heads, n_seqs), block(cols * SCAN_LANES);
    cudaStream_t s = (cudaStream_t)stream;
#define GK_SCAN(R, TB) gk_launch(decay_scan_kernel<R, TB>, grid, block, 0, s, q, k, v, decay, state, out, cu_q, slots, n_heads, d, dv)
    if (d <= 32) GK_SCAN(4, 16);
    else if (d <= 64) GK_SCAN(8, 16);
    else if (d <= 128) GK_SCAN(16, 8);
    else GK_SCAN(32, 4);
#undef GK_SCAN
    GK_CHECK_LAUNCH("decay_scan");
    return GK_OK;
}

GK_EXPORT int gk_group_norm_gate(const float* x, const float* weight, const void* gate, int gate_dtype, long long ld_gate, void* out,
                                 int out_dtype, long long n_tokens, int n_groups, int size, float eps, int gate_kind, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(gate_dtype) && GK_VALID_DTYPE(out_dtype), "group_norm_gate: bad dtype");
    GK_REQUIRE(n_groups > 0 && size > 0 && eps > 0.f && (gate_kind == 0 || gate_kind == 1), "group_norm_gate: bad sizes");
    if (n_tokens == 0) return GK_OK;
    const long long rows = n_tokens * n_groups;
    const long long blocks = (rows + 7) / 8;
    GK_REQUIRE(blocks < 2147483647LL, "group_norm_gate: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    const bool wide = size >= 512 && rows < 2147483647LL;  // by the group's size alone: a row's sums never depend on the step
    GK_DISPATCH_DTYPE(out_dtype, T, {
        GK_DISPATCH_DTYPE(gate_dtype, TG, {
            if (wide)
                gk_launch(group_norm_gate_wide_kernel<T, TG>, dim3((unsigned)rows), dim3(256), 0, s, x, weight, (const TG*)gate, ld_gate,
                          (T*)out, n_groups, size, eps, gate_kind);
            else
                gk_launch(group_norm_gate_kernel<T, TG>, dim3((unsigned)blocks), dim3(256), 0, s, x, weight, (const TG*)gate, ld_gate,
                          (T*)out, rows, n_groups, size, eps, gate_kind);
        })
    })
    GK_CHECK_LAUNCH("group_norm_gate");
    return GK_OK;
}
