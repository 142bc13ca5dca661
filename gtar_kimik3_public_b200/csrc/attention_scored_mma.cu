// Scored attention on the tensor cores (bfloat16, keys and values of 64 or 128 entries): the same rules as the exact
// kernel of this family, for the new tokens of every sequence of a step over the paged cache.
//
//   visible:  j <= i  and  (window = 0  or  i - j < window  or  j < keep_first)
//   s_j = (q . k_j) * scale - r1_h * ln(1 + r2_h * (i - j))          (the second term only where r1, r2 are given)
//   softmax: o = sum_j softmax(s)_j v_j          sigmoid: o = sum_j sigmoid(s_j + bias_h) v_j
// and, each only where its argument is given: keys of the token's own chunk only (chunks of `chunk` positions counted
// from the sequence's start), a number per query head on the product (temp), a table [n_dist, n_q] of terms added to
// the score by distance (row min(i - j, n_dist - 1)), a number per query head whose exponential joins the softmax's
// denominator and carries no value (sink).
//
// The rows of a block's tile are (token, query head of one kv group) pairs, token-major, so the query heads that
// share a kv head share every loaded page; a warp owns 16 rows and K and V pages stream through a three-stage
// cp.async ring, as in the plain prefill kernel.  What differs: the pages a block walks are the kept first pages
// followed by the pages of its rows' windows; every score gets its distance term (one logarithm a score, formed in
// the base-2 domain of the softmax); the weights are either the running softmax or a sigmoid that nothing divides.
// Scores, weights, maxima and sums are 32-bit; the weights are rounded to bfloat16 only as the operand of the second
// product, whose sums are 32-bit again.
//
// The walk over a block's pages can be cut into `n_split` parts that run as blocks of their own (a step of single
// tokens has too few rows to fill the GPU otherwise).  Each part then leaves its unnormalised sums, and for the
// softmax its maximum and denominator, in a 32-bit workspace, and a second kernel adds the parts.

#include "attention_mma.cuh"

namespace {

using namespace attn;

constexpr int SC_WARPS = 4;
constexpr int SC_ROWS = SC_WARPS * 16;
constexpr int SC_STAGES = 3;
constexpr float LOG2E = 1.4426950408889634f;

template <int D>
struct ScoredSmem {
    __nv_bfloat16 k[SC_STAGES][PAGE * D];
    __nv_bfloat16 v[SC_STAGES][PAGE * D];
};

__device__ __forceinline__ float lg2_fast(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// MORE: which of the further rules are compiled in: 0 none, 1 the sink alone, 2 the chunk, the head temperature, the
// distance table and the sink.  Without them the kernel is the windowed one alone and keeps its registers (a third block
// a multiprocessor at heads of 64); the sink alone costs none.
template <int D, bool SIGMOID, int MORE>
__global__ void __launch_bounds__(SC_WARPS * 32, (MORE == 2 && D == 64) ? 3 : 0) attention_scored_mma_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ cu_q,
    const int* __restrict__ kv_len, const int* __restrict__ slots, const int* __restrict__ block_table, int n_tokens, int n_q,
    int n_kv, int max_pages, float sl2, int window, int keep_first, const float* __restrict__ r1, const float* __restrict__ r2,
    const float* __restrict__ head_bias, int n_split, int chunk, const float* __restrict__ temp,
    const float* __restrict__ dist_bias, int n_dist, const float* __restrict__ sink) {
    constexpr bool RULES = MORE == 2;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    ScoredSmem<D>& sm = *reinterpret_cast<ScoredSmem<D>*>(smem_raw);
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.z, hk = blockIdx.y;
    const int group = n_q / n_kv;
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int n_rows = q_len * group;
    const int n_blocks = (n_rows + SC_ROWS - 1) / SC_ROWS;
    const int row_block = (int)blockIdx.x / n_split, split = (int)blockIdx.x % n_split;
    if (row_block >= n_blocks) return;
    const int row0 = (n_blocks - 1 - row_block) * SC_ROWS;  // heavy blocks (late tokens) first
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int len = kv_len[seq], past = len - q_len;
    const int* pages = block_table + (size_t)slots[seq] * max_pages;

    const int wrow0 = row0 + warp * 16;
    int tok[2], pos[2], head[2];
    bool row_ok[2];
    float b1[2], b2[2], add[2], sl2h[2];
    int first[2];  // first key of the row's chunk
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = wrow0 + (lane >> 2) + 8 * h;
        row_ok[h] = r < n_rows;
        tok[h] = row_ok[h] ? r / group : 0;
        pos[h] = past + tok[h];
        head[h] = hk * group + (row_ok[h] ? r % group : 0);
        first[h] = RULES && chunk > 0 ? (pos[h] / chunk) * chunk : 0;
        sl2h[h] = RULES && temp != nullptr ? sl2 * temp[head[h]] : sl2;
        b1[h] = r1 != nullptr ? r1[head[h]] : 0.f;  // the distance term in the base-2 domain: r1 log2(1 + r2 gap)
        b2[h] = r1 != nullptr ? r2[head[h]] : 0.f;
        add[h] = head_bias != nullptr ? head_bias[head[h]] * LOG2E : 0.f;
    }
    const bool biased = r1 != nullptr;
    uint32_t qf[D / 16][4];
    {
        const int c0 = (lane & 3) * 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __nv_bfloat16* qrow = q + ((size_t)(q_begin + tok[h]) * n_q + head[h]) * D;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                qf[ks][h] = row_ok[h] ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + c0) : 0u;
                qf[ks][h + 2] = row_ok[h] ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + c0 + 8) : 0u;
            }
        }
    }
    // The block's pages: the kept first pages that lie before its rows' windows, then from the first page that its
    // first row's window touches to the page of its last row.
    const int last_row = min(row0 + SC_ROWS, n_rows) - 1;
    const int max_pos = past + last_row / group;
    const int min_pos = past + row0 / group;
    int lo_block = (window > 0 && min_pos - window + 1 > 0) ? min_pos - window + 1 : 0;
    if (RULES && chunk > 0) {
        const int chunk_first = (min_pos / chunk) * chunk;  // no row of the block sees a key before its first row's chunk
        if (chunk_first > 0) keep_first = 0;                // the kept first keys lie in an earlier chunk
        lo_block = max(lo_block, chunk_first);
    }
    const int p_begin = lo_block / PAGE, p_end = max_pos / PAGE + 1;
    const int kept_pages = window > 0 ? min((keep_first + PAGE - 1) / PAGE, p_begin) : 0;
    const int n_iter = kept_pages + p_end - p_begin;
    const int it0 = (int)((long long)n_iter * split / n_split), it1 = (int)((long long)n_iter * (split + 1) / n_split);
    // of this warp
    const int w_last_row = min(wrow0 + 16, n_rows) - 1;
    const int w_max_pos = w_last_row >= wrow0 ? past + w_last_row / group : -1;
    const int w_min_pos = past + wrow0 / group;
    int w_lo = (window > 0 && w_min_pos - window + 1 > 0) ? w_min_pos - window + 1 : 0;
    if (RULES && chunk > 0) w_lo = max(w_lo, (w_min_pos / chunk) * chunk);

    auto page_index = [&](int it) { return it < kept_pages ? it : p_begin + it - kept_pages; };
    auto issue = [&](int it) {
        if (it < it1) {
            const int p = page_index(it);
            const int page = pages[p];
            const int valid = min(PAGE, len - p * PAGE);
            const size_t base = ((size_t)page * n_kv + hk) * PAGE * D;
            const int stage = (it - it0) % SC_STAGES;
            load_page_async<D, SC_WARPS * 32>(sm.k[stage], k_pages + base, valid, tid);
            load_page_async<D, SC_WARPS * 32>(sm.v[stage], v_pages + base, valid, tid);
        }
        cp_async_commit();
    };

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    if (MORE >= 1 && !SIGMOID && sink != nullptr && split == 0) {
        // the sink opens the running softmax of the first part: a term exp(sink) in the denominator that carries no value
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m[h] = sink[head[h]] * LOG2E;
            l[h] = 1.f;
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;

#pragma unroll
    for (int st = 0; st < SC_STAGES - 1; ++st) issue(it0 + st);
    for (int it = it0; it < it1; ++it) {
        cp_async_wait<SC_STAGES - 2>();
        __syncthreads();
        issue(it + SC_STAGES - 1);
        const int stage = (it - it0) % SC_STAGES;
        const int key_base = page_index(it) * PAGE;
        // warp-uniform: some key of the page is not in the future of all rows, and is inside some row's window or kept
        if (key_base <= w_max_pos && (key_base + PAGE > w_lo || key_base < keep_first)) {
            const int n16 = min(PAGE / 16, (w_max_pos - key_base) / 16 + 1);
            float s[8][4];
            uint32_t p[4][4];
            qk_page<D, false>(s, qf, sm.k[stage], n16, lane);
#pragma unroll
            for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int key = key_base + n * 8 + (lane & 3) * 2 + c;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int gap = pos[h] - key;
                        const bool hidden = gap < 0 || (window > 0 && gap >= window && key >= keep_first) || (RULES && key < first[h]);
                        float t = s[n][2 * h + c] * (RULES ? sl2h[h] : sl2);
                        if (biased) t -= b1[h] * lg2_fast(fmaf(b2[h], (float)max(gap, 0), 1.f));
                        if (RULES && dist_bias != nullptr)
                            t = fmaf(__ldg(dist_bias + (size_t)min(max(gap, 0), n_dist - 1) * n_q + head[h]), LOG2E, t);
                        if (SIGMOID)
                            s[n][2 * h + c] = hidden ? 0.f : __fdividef(1.f, 1.f + exp2_fast(-(t + add[h])));
                        else
                            s[n][2 * h + c] = hidden ? -INFINITY : t;
                    }
                }
            if (SIGMOID) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    p[g][0] = pack_bf16(s[2 * g][0], s[2 * g][1]);
                    p[g][1] = pack_bf16(s[2 * g][2], s[2 * g][3]);
                    p[g][2] = pack_bf16(s[2 * g + 1][0], s[2 * g + 1][1]);
                    p[g][3] = pack_bf16(s[2 * g + 1][2], s[2 * g + 1][3]);
                }
            } else {
                softmax_page<D>(s, m, l, o, p, 1.0f);
            }
            pv_page<D, false>(o, p, sm.v[stage], n16, lane);
        }
    }
    cp_async_wait<0>();

    const int c0 = (lane & 3) * 2;
    if (n_split == 1) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (!row_ok[h]) continue;
            const float inv = SIGMOID ? 1.f : 1.0f / l[h];
            __nv_bfloat16* orow = out + ((size_t)(q_begin + tok[h]) * n_q + head[h]) * D;
#pragma unroll
            for (int j = 0; j < D / 8; ++j)
                *reinterpret_cast<uint32_t*>(orow + j * 8 + c0) = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!row_ok[h]) continue;
        const size_t item = ((size_t)split * n_tokens + q_begin + tok[h]) * n_q + head[h];
        float* orow = part_o + item * D;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) *reinterpret_cast<float2*>(orow + j * 8 + c0) = make_float2(o[j][2 * h], o[j][2 * h + 1]);
        if (!SIGMOID && (lane & 3) == 0) *reinterpret_cast<float2*>(part_ml + item * 2) = make_float2(m[h], l[h]);
    }
}

// One warp per (token, query head): the parts' sums brought to one maximum and added.
template <int D, bool SIGMOID>
__global__ void __launch_bounds__(128) attention_scored_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                    __nv_bfloat16* __restrict__ out, long long n_items, int n_split) {
    pdl_launch_dependents();
    pdl_wait();
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= n_items) return;
    const int lane = threadIdx.x & 31;
    float top = -INFINITY;
    if (!SIGMOID)
        for (int s = 0; s < n_split; ++s) top = fmaxf(top, part_ml[((size_t)s * n_items + item) * 2]);
    float acc[D / 32], denom = 0.f;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) acc[c] = 0.f;
    for (int s = 0; s < n_split; ++s) {
        float w = 1.f;
        if (!SIGMOID) {
            const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((size_t)s * n_items + item) * 2);
            w = ml.x == -INFINITY ? 0.f : exp2_fast(ml.x - top);
            denom = fmaf(ml.y, w, denom);
        }
        const float* src = part_o + ((size_t)s * n_items + item) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) acc[c] = fmaf(src[lane + 32 * c], w, acc[c]);
    }
    const float inv = SIGMOID ? 1.f : 1.f / denom;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) out[(size_t)item * D + lane + 32 * c] = __float2bfloat16(acc[c] * inv);
}

template <int D, bool SIGMOID, int MORE>
int launch_scored(const void* q, const void* k_pages, const void* v_pages, void* out, float* part_o, float* part_ml, const int* cu_q,
                  const int* kv_len, const int* slots, const int* block_table, int n_seqs, int max_q_len, int n_tokens, int n_q,
                  int n_kv, int max_pages, float scale, int window, int keep_first, const float* r1, const float* r2,
                  const float* head_bias, int n_split, int chunk, const float* temp, const float* dist_bias, int n_dist,
                  const float* sink, cudaStream_t stream) {
    const size_t smem = sizeof(ScoredSmem<D>);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_scored_mma_kernel<D, SIGMOID, MORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "attention_scored_mma: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int group = n_q / n_kv;
    const long long blocks = (((long long)max_q_len * group + SC_ROWS - 1) / SC_ROWS) * n_split;
    GK_REQUIRE(blocks <= 2147483647LL, "attention_scored_mma: too many rows");
    gk_launch(attention_scored_mma_kernel<D, SIGMOID, MORE>, dim3((unsigned)blocks, n_kv, n_seqs), dim3(SC_WARPS * 32), smem, stream,
              (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out, part_o, part_ml,
              cu_q, kv_len, slots, block_table, n_tokens, n_q, n_kv, max_pages, scale * LOG2E, window, keep_first, r1, r2, head_bias,
              n_split, chunk, temp, dist_bias, n_dist, sink);
    GK_CHECK_LAUNCH("attention_scored_mma");
    if (n_split > 1) {
        const long long items = (long long)n_tokens * n_q;
        gk_launch(attention_scored_join_kernel<D, SIGMOID>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (const float*)part_o,
                  (const float*)part_ml, (__nv_bfloat16*)out, items, n_split);
        GK_CHECK_LAUNCH("attention_scored_join");
    }
    return GK_OK;
}

}  // namespace

// q, out: [n_tokens, n_q, head_dim] bfloat16 packed by sequence (cu_q[i] = first token of sequence i); kv_len[i] counts
// the sequence's cached tokens including this step's; max_q_len = the longest part of the step.  weights: 0 softmax,
// 1 sigmoid.  r1, r2 (both or neither) and head_bias, a number per query head, may be null.  With n_split > 1,
// part_o [n_split, n_tokens, n_q, head_dim] and (softmax) part_ml [n_split, n_tokens, n_q, 2] are 32-bit workspaces.
GK_EXPORT int gk_attention_scored_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, float* part_o,
                                       float* part_ml, const int* cu_q, const int* kv_len, const int* slots, const int* block_table,
                                       int n_seqs, int max_q_len, int n_tokens, int n_q, int n_kv, int head_dim, int max_pages,
                                       int page_size, float scale, int window, int keep_first, const float* r1, const float* r2,
                                       const float* head_bias, int weights, int n_split, int chunk, const float* temp,
                                       const float* dist_bias, int n_dist, const float* sink, void* stream) {
    GK_REQUIRE(n_seqs >= 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_scored_mma: bad head counts %d/%d", n_q, n_kv);
    GK_REQUIRE(page_size == attn::PAGE, "attention_scored_mma: page_size must be %d, got %d", attn::PAGE, page_size);
    GK_REQUIRE(head_dim == 64 || head_dim == 128, "attention_scored_mma: head size %d is not 64 or 128 (use the exact kernel)", head_dim);
    GK_REQUIRE(n_kv <= 65535 && n_seqs <= 65535, "attention_scored_mma: grid too large");
    GK_REQUIRE(window >= 0 && keep_first >= 0 && max_q_len >= 0, "attention_scored_mma: bad window, kept keys or length");
    GK_REQUIRE((r1 == nullptr) == (r2 == nullptr), "attention_scored_mma: the distance term needs both of its numbers");
    GK_REQUIRE(weights == 0 || weights == 1, "attention_scored_mma: weights are softmax (0) or sigmoid (1)");
    GK_REQUIRE(n_split >= 1 && (n_split == 1 || (part_o != nullptr && (weights == 1 || part_ml != nullptr))),
               "attention_scored_mma: %d parts need their workspaces", n_split);
    GK_REQUIRE(chunk >= 0 && (dist_bias == nullptr || n_dist > 0), "attention_scored_mma: bad chunk or distance table");
    GK_REQUIRE(sink == nullptr || weights == 0, "attention_scored_mma: a sink belongs to the softmax");
    if (n_seqs == 0 || max_q_len == 0 || n_tokens == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int more = (chunk > 0 || temp != nullptr || dist_bias != nullptr) ? 2 : sink != nullptr ? 1 : 0;
#define GK_SCORED(D, SIG)                                                                                                             \
    do {                                                                                                                              \
        if (more == 2)                                                                                                                \
            return launch_scored<D, SIG, 2>(q, k_pages, v_pages, out, part_o, part_ml, cu_q, kv_len, slots, block_table, n_seqs,      \
                                            max_q_len, n_tokens, n_q, n_kv, max_pages, scale, window, keep_first, r1, r2,             \
                                            head_bias, n_split, chunk, temp, dist_bias, n_dist, sink, s);                             \
        if (more == 1)                                                                                                                \
            return launch_scored<D, SIG, 1>(q, k_pages, v_pages, out, part_o, part_ml, cu_q, kv_len, slots, block_table, n_seqs,      \
                                            max_q_len, n_tokens, n_q, n_kv, max_pages, scale, window, keep_first, r1, r2,             \
                                            head_bias, n_split, chunk, temp, dist_bias, n_dist, sink, s);                             \
        return launch_scored<D, SIG, 0>(q, k_pages, v_pages, out, part_o, part_ml, cu_q, kv_len, slots, block_table, n_seqs,      \
                                            max_q_len, n_tokens, n_q, n_kv, max_pages, scale, window, keep_first, r1, r2, head_bias,  \
                                            n_split, chunk, temp, dist_bias, n_dist, sink, s);                                        \
    } while (0)
    if (head_dim == 64) {
        if (weights == 1) GK_SCORED(64, true);
        GK_SCORED(64, false);
    }
    if (weights == 1) GK_SCORED(128, true);
    GK_SCORED(128, false);
#undef GK_SCORED
}
