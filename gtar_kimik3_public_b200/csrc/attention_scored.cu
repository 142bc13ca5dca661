// Causal grouped-query attention over the paged cache with a rule for the scores and a rule for the weights, any
// head sizes (keys of d, values of dv entries), any dtype: the exact kernel of this family.
//
// For a token at position i of its sequence, query head h, key/value head h / (n_q / n_kv), and a key at j <= i:
//   visible:  i - j < window  or  j < keep_first          (window = 0: every j <= i)
//   s_j = (q . k_j) * scale - r1_h * ln(1 + r2_h * (i - j))             (the second term only where r1, r2 are given)
//   weights = softmax over the visible keys:   o = sum_j softmax(s)_j v_j
//   weights = sigmoid:                         o = sum_j sigmoid(s_j + bias_h) v_j      (no sum over keys divides)
// A key that the window has left and the first tokens keep stays at its true position.
// Further rules, each present only where its argument is given:
//   chunk > 0:   a key is visible only from its own chunk, floor(i / chunk) = floor(j / chunk), chunks counted from
//                the sequence's first position
//   temp:        a number per query head on the product:  (q . k_j) * scale * temp_h
//   dist_bias:   a table [n_dist, n_q] of terms ADDED to the score, read at row min(i - j, n_dist - 1)
//   sink:        a number per query head whose exponential joins the softmax's denominator (and nothing else):
//                weights_j = exp(s_j) / (exp(sink_h) + sum_visible exp(s))
//
// One warp per (token, query head).  Keys are taken in blocks of 32 from key 0 upward, one key per lane; blocks
// that hold no visible key are passed over.  All sums are 32-bit, and the sequence of operations for a (token,
// head) depends only on its own position and keys: results are bit-equal however the tokens are cut into steps
// or batched.

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_ACC = 16;  // dv <= 512

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int d) {
    float acc = 0.f;
    if (d & 3) {  // rows that do not start on 16 bytes: one entry at a time
        for (int i = 0; i < d; ++i) acc = fmaf(q[i], k[i], acc);
        return acc;
    }
    for (int i = 0; i < d; i += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + i);
        acc = fmaf(q[i], kv.x, acc);
        acc = fmaf(q[i + 1], kv.y, acc);
        acc = fmaf(q[i + 2], kv.z, acc);
        acc = fmaf(q[i + 3], kv.w, acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int d) {
    float acc = 0.f;
    if (d & 7) {  // rows that do not start on 16 bytes: one entry at a time
        for (int i = 0; i < d; ++i) acc = fmaf(q[i], __bfloat162float(k[i]), acc);
        return acc;
    }
    for (int i = 0; i < d; i += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float2 f = __bfloat1622float2(p[c]);
            acc = fmaf(q[i + 2 * c], f.x, acc);
            acc = fmaf(q[i + 2 * c + 1], f.y, acc);
        }
    }
    return acc;
}

template <typename T, bool SIGMOID>
__global__ void __launch_bounds__(WARPS * 32) attention_scored_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ out,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
    const int* __restrict__ block_table, int n_tokens, int n_q, int n_kv, int d, int dv, int max_pages, int page_size,
    float scale, int window, int keep_first, const float* __restrict__ r1, const float* __restrict__ r2,
    const float* __restrict__ head_bias, int chunk, const float* __restrict__ temp, const float* __restrict__ dist_bias,
    int n_dist, const float* __restrict__ sink) {
    extern __shared__ float q_smem[];  // WARPS * d
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * WARPS + warp;
    if (wid >= (long long)n_tokens * n_q) return;  // whole warp leaves together; no block-wide sync below
    const int t = (int)(wid / n_q);
    const int hq = (int)(wid - (long long)t * n_q);
    const int hk = hq / (n_q / n_kv);
    const int pos = tok_pos[t];
    const int* pages = block_table + (size_t)slots[tok_seq[t]] * max_pages;
    float* qs = q_smem + warp * d;
    const T* qrow = q + ((size_t)t * n_q + hq) * d;
    for (int i = lane; i < d; i += 32) qs[i] = to_float(qrow[i]);
    __syncwarp();
    const bool biased = r1 != nullptr;
    const float b1 = biased ? r1[hq] : 0.f, b2 = biased ? r2[hq] : 0.f;
    const float add = head_bias != nullptr ? head_bias[hq] : 0.f;

    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;  // first key of the window
    if (chunk > 0) {
        const int first = (pos / chunk) * chunk;  // first key of the token's chunk
        if (first > 0) keep_first = 0;            // the kept first keys lie in an earlier chunk
        lo = max(lo, first);
    }
    if (temp != nullptr) scale *= temp[hq];
    // the sink opens the running softmax: a term exp(sink) in the denominator that carries no value
    float m = (!SIGMOID && sink != nullptr) ? sink[hq] : -INFINITY, l = (!SIGMOID && sink != nullptr) ? 1.f : 0.f;
    float acc[MAX_ACC];
#pragma unroll
    for (int c = 0; c < MAX_ACC; ++c) acc[c] = 0.f;
    const int n_acc = (dv + 31) >> 5;

    for (int j0 = 0; j0 <= pos; j0 += 32) {
        if (j0 + 31 < lo && j0 >= keep_first) {  // neither in the window nor among the kept first keys
            j0 = ((lo >> 5) << 5) - 32;  // on to the window's first block
            continue;
        }
        const int page = pages[j0 / page_size];  // page_size is a multiple of 32: one page per block
        const int in_page = j0 % page_size;
        const size_t row0 = ((size_t)page * n_kv + hk) * page_size + in_page;
        const int j = j0 + lane;
        const bool valid = j <= pos && (j >= lo || j < keep_first);
        float s = -INFINITY;
        if (valid) {
            s = dot_row<T>(qs, k_pages + (row0 + lane) * d, d) * scale;
            if (biased) s -= b1 * log1pf(b2 * (float)(pos - j));
            if (dist_bias != nullptr) s += dist_bias[(size_t)min(pos - j, n_dist - 1) * n_q + hq];
        }
        float p;
        if (SIGMOID) {
            p = valid ? 1.f / (1.f + expf(-(s + add))) : 0.f;
        } else {
            const float m_new = fmaxf(m, warp_max(s));
            p = valid ? expf(s - m_new) : 0.f;
            const float corr = expf(m - m_new);
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int c = 0; c < MAX_ACC; ++c)
                if (c < n_acc) acc[c] *= corr;
            m = m_new;
        }
        const int n_here = min(32, pos - j0 + 1);
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vrow = v_pages + (row0 + jj) * dv;
#pragma unroll
            for (int c = 0; c < MAX_ACC; ++c) {
                const int dim = lane + 32 * c;
                if (c < n_acc && dim < dv) acc[c] = fmaf(pj, to_float(vrow[dim]), acc[c]);
            }
        }
    }
    T* orow = out + ((size_t)t * n_q + hq) * dv;
    const float inv = SIGMOID ? 1.f : 1.f / l;
#pragma unroll
    for (int c = 0; c < MAX_ACC; ++c) {
        const int dim = lane + 32 * c;
        if (c < n_acc && dim < dv) orow[dim] = from_float<T>(SIGMOID ? acc[c] : acc[c] * inv);
    }
}

}  // namespace

// weights: 0 softmax, 1 sigmoid.  r1, r2 (per query head, both or neither) and head_bias (per query head) may be null.
GK_EXPORT int gk_attention_scored_exact(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype,
                                        const int* tok_pos, const int* tok_seq, const int* slots, const int* block_table,
                                        int n_tokens, int n_q, int n_kv, int d, int dv, int max_pages, int page_size, float scale,
                                        int window, int keep_first, const float* r1, const float* r2, const float* head_bias,
                                        int weights, int chunk, const float* temp, const float* dist_bias, int n_dist,
                                        const float* sink, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "attention_scored: bad dtype %d", dtype);
    GK_REQUIRE(n_tokens >= 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_scored: bad head counts %d/%d", n_q, n_kv);
    GK_REQUIRE(d > 0 && dv > 0 && dv <= 32 * MAX_ACC, "attention_scored: keys of %d must be positive, values of %d at most %d", d, dv,
               32 * MAX_ACC);
    GK_REQUIRE(page_size > 0 && page_size % 32 == 0, "attention_scored: page_size %d must be a multiple of 32", page_size);
    GK_REQUIRE(window >= 0 && keep_first >= 0, "attention_scored: window and kept first keys must be >= 0 (0 = none)");
    GK_REQUIRE((r1 == nullptr) == (r2 == nullptr), "attention_scored: the distance term needs both of its numbers");
    GK_REQUIRE(weights == 0 || weights == 1, "attention_scored: weights are softmax (0) or sigmoid (1)");
    GK_REQUIRE(chunk >= 0 && (dist_bias == nullptr || n_dist > 0), "attention_scored: bad chunk or distance table");
    GK_REQUIRE(sink == nullptr || weights == 0, "attention_scored: a sink belongs to the softmax");
    if (n_tokens == 0) return GK_OK;
    const long long warps = (long long)n_tokens * n_q;
    const long long blocks = (warps + WARPS - 1) / WARPS;
    GK_REQUIRE(blocks < 2147483647LL, "attention_scored: too many tokens");
    const size_t smem = (size_t)WARPS * d * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(dtype, T, {
        if (weights == 1)
            gk_launch(attention_scored_kernel<T, true>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, s, (const T*)q, (const T*)k_pages,
                      (const T*)v_pages, (T*)out, tok_pos, tok_seq, slots, block_table, n_tokens, n_q, n_kv, d, dv, max_pages, page_size,
                      scale, window, keep_first, r1, r2, head_bias, chunk, temp, dist_bias, n_dist, sink);
        else
            gk_launch(attention_scored_kernel<T, false>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, s, (const T*)q, (const T*)k_pages,
                      (const T*)v_pages, (T*)out, tok_pos, tok_seq, slots, block_table, n_tokens, n_q, n_kv, d, dv, max_pages, page_size,
                      scale, window, keep_first, r1, r2, head_bias, chunk, temp, dist_bias, n_dist, sink);
    })
    GK_CHECK_LAUNCH("attention_scored");
    return GK_OK;
}
