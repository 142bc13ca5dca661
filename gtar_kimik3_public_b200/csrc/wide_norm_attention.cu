// What an attention layer with one norm over the whole query projection and one over the whole key projection,
// values that ARE the keys as projected, and a gate on its result needs around the attention kernel:
//
//   wide_norm_rope_write   per token: q <- w_q * q / sqrt(mean(q^2) + eps) over all query heads at once, the same for
//                          k over all key heads; then, in each head, the first `rot` entries turn by the token's
//                          position (entry i paired with i + rot/2; cos and sin from tables [positions, rot/2]) and the
//                          rest pass; the finished key goes into the key pages and the key AS PROJECTED (before norm
//                          and rotation) into the value pages.  One block per token, 32-bit arithmetic.
//                          With v_at >= 0 the values are a projection of their own (n_kv heads of dv entries from
//                          column v_at of the row) and go into the value pages as projected; with has_k = 0 the row
//                          holds queries only (a layer that reads another layer's keys and values).  Without rotation and
//                          with rows of whole 16-byte pieces the row is held in registers (read once, 16-byte accesses).
//   sigmoid_gate           out = o * sigmoid(gate), the gate read from a column range of a wider row
//   softcap                x <- cap * tanh(x / cap), in place (32-bit logits)
//   turn_back_gate         every head's read-out o [dv] turned by MINUS the reading token's position over all of its
//                          entries (entry m paired with m + dv/2; what undoes, for the sum over keys, a turn of every
//                          value by its own position), then times sigmoid of ONE number per head, read from a column
//                          range of a wider row.  Either half may be left out.

#include "common.cuh"

namespace {

constexpr int WN_THREADS = 256;

template <typename T, typename TC>
__global__ void __launch_bounds__(WN_THREADS) wide_norm_rope_write_kernel(
    const T* __restrict__ proj, long long ld, const float* __restrict__ w_q, const float* __restrict__ w_k,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seq, const int* __restrict__ slots, const int* __restrict__ block_table,
    T* __restrict__ q_out, TC* __restrict__ k_pages, TC* __restrict__ v_pages, int n_q, int n_kv, int d, int rot,
    int max_pages, int page_size, float eps, int v_at, int dv, int has_k) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * ld;
    const int nq = n_q * d, nk = has_k ? n_kv * d : 0;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += WN_THREADS) { const float v = to_float(row[i]); sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < nk; i += WN_THREADS) { const float v = to_float(row[nq + i]); sk = fmaf(v, v, sk); }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    const float rq = 1.f / sqrtf(sq / (float)nq + eps), rk = nk ? 1.f / sqrtf(sk / (float)nk + eps) : 0.f;
    const int pos = tok_pos[t];
    const int half = rot >> 1;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    for (int i = threadIdx.x; i < nq + nk; i += WN_THREADS) {
        const bool is_q = i < nq;
        const int at = is_q ? i : i - nq;
        const int j = at % d;
        const float r = is_q ? rq : rk;
        const float* w = is_q ? w_q : w_k;
        const float mine = to_float(row[i]) * r * w[at];
        float res = mine;
        if (j < half) {
            const float other = to_float(row[i + half]) * r * w[at + half];
            res = mine * cs[j] - other * sn[j];
        } else if (j < rot) {
            const float other = to_float(row[i - half]) * r * w[at - half];
            res = mine * cs[j - half] + other * sn[j - half];
        }
        if (is_q) {
            q_out[(size_t)t * nq + at] = from_float<T>(res);
        } else if (k_pages != nullptr) {
            const int hk = at / d;
            const int page = block_table[(size_t)slots[tok_seq[t]] * max_pages + pos / page_size];
            const size_t dst = (((size_t)page * n_kv + hk) * page_size + pos % page_size) * d + j;
            k_pages[dst] = from_float<TC>(res);
            if (v_at < 0) v_pages[dst] = from_float<TC>(to_float(row[i]));
        }
    }
    if (v_at >= 0 && nk && k_pages != nullptr) {
        const int page = block_table[(size_t)slots[tok_seq[t]] * max_pages + pos / page_size];
        for (int i = threadIdx.x; i < n_kv * dv; i += WN_THREADS) {
            const int hk = i / dv, j = i - hk * dv;
            v_pages[(((size_t)page * n_kv + hk) * page_size + pos % page_size) * dv + j] = from_float<TC>(to_float(row[v_at + i]));
        }
    }
}

// The same without rotation for rows that are whole 16-byte pieces (heads, the values' column and the row stride all
// multiples of eight bfloat16 or four float32 entries; cache pages of the rows' type): a thread holds up to four pieces of
// the row in registers, so that the row is read once, with 16-byte loads, and written with 16-byte stores.  A block's
// sums are formed in a fixed order of their own (a thread its pieces in index order, a warp by shuffles, the eight
// warps one after another), which depends on the sizes alone.
constexpr int WN_HELD = 4;

template <typename T>
__global__ void __launch_bounds__(WN_THREADS) wide_norm_write_vec_kernel(
    const T* __restrict__ proj, long long ld, const float* __restrict__ w_q, const float* __restrict__ w_k,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
    const int* __restrict__ block_table, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_q, int n_kv,
    int d, int max_pages, int page_size, float eps, int v_at, int dv, int has_k) {
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float red[2][WN_THREADS / 32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * ld;
    const int nq = n_q * d, nk = has_k ? n_kv * d : 0;
    const int q_pieces = nq / VEC, pieces = (nq + nk) / VEC;
    uint4 held[WN_HELD];
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int h = 0; h < WN_HELD; ++h) {
        const int c = threadIdx.x + h * WN_THREADS;
        if (c >= pieces) break;
        held[h] = *reinterpret_cast<const uint4*>(row + (size_t)c * VEC);
        const T* e = reinterpret_cast<const T*>(&held[h]);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) { const float v = to_float(e[i]); ss = fmaf(v, v, ss); }
        if (c < q_pieces) sq += ss;
        else sk += ss;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if ((threadIdx.x & 31) == 0) {
        red[0][threadIdx.x >> 5] = sq;
        red[1][threadIdx.x >> 5] = sk;
    }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int w = 0; w < WN_THREADS / 32; ++w) { tq += red[0][w]; tk += red[1][w]; }
    const float rq = 1.f / sqrtf(tq / (float)nq + eps), rk = nk ? 1.f / sqrtf(tk / (float)nk + eps) : 0.f;
    const int pos = tok_pos[t];
    const bool write = k_pages != nullptr;
    const int page = write ? block_table[(size_t)slots[tok_seq[t]] * max_pages + pos / page_size] : 0;
    const int in_page = pos % page_size;
#pragma unroll
    for (int h = 0; h < WN_HELD; ++h) {
        const int c = threadIdx.x + h * WN_THREADS;
        if (c >= pieces) break;
        const bool is_q = c < q_pieces;
        if (!is_q && !write) continue;
        const int at = (is_q ? c : c - q_pieces) * VEC;
        const float r = is_q ? rq : rk;
        const float* w = (is_q ? w_q : w_k) + at;
        const T* e = reinterpret_cast<const T*>(&held[h]);
        uint4 res;
        T* o = reinterpret_cast<T*>(&res);
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = from_float<T>(to_float(e[i]) * r * w[i]);
        if (is_q) {
            *reinterpret_cast<uint4*>(q_out + (size_t)t * nq + at) = res;
        } else {
            const int hk = at / d, j = at - hk * d;
            const size_t dst = (((size_t)page * n_kv + hk) * page_size + in_page) * d + j;
            *reinterpret_cast<uint4*>(k_pages + dst) = res;
            if (v_at < 0) *reinterpret_cast<uint4*>(v_pages + dst) = held[h];
        }
    }
    if (v_at >= 0 && nk && write) {
        const int v_pieces = n_kv * dv / VEC;
        for (int c = threadIdx.x; c < v_pieces; c += WN_THREADS) {
            const int at = c * VEC, hk = at / dv, j = at - hk * dv;
            *reinterpret_cast<uint4*>(v_pages + (((size_t)page * n_kv + hk) * page_size + in_page) * dv + j) =
                *reinterpret_cast<const uint4*>(row + v_at + at);
        }
    }
}

template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ o, const T* __restrict__ gate, long long ld_gate, T* __restrict__ out,
                                    long long n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / width;
    const int c = (int)(i - t * width);
    const float g = to_float(gate[t * ld_gate + c]);
    out[i] = from_float<T>(to_float(o[i]) / (1.f + expf(-g)));
}

__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// One thread per (token, head, pair of entries).
template <typename T>
__global__ void turn_back_gate_kernel(const T* __restrict__ o, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      const int* __restrict__ tok_pos, const T* __restrict__ gate, long long ld_gate,
                                      T* __restrict__ out, long long n, int n_heads, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int half = dv >> 1;
    const long long th = i / half;
    const int m = (int)(i - th * half);
    const long long t = th / n_heads;
    const int h = (int)(th - t * n_heads);
    const size_t at = (size_t)th * dv;
    float a = to_float(o[at + m]), b = to_float(o[at + m + half]);
    if (cos_t != nullptr) {
        const size_t row = (size_t)tok_pos[t] * half + m;
        const float c = cos_t[row], s = sin_t[row];
        const float ra = a * c + b * s, rb = b * c - a * s;  // the turn by minus the angle
        a = ra;
        b = rb;
    }
    if (gate != nullptr) {
        const float g = 1.f / (1.f + expf(-to_float(gate[t * ld_gate + h])));
        a *= g;
        b *= g;
    }
    out[at + m] = from_float<T>(a);
    out[at + m + half] = from_float<T>(b);
}

// The same for bfloat16 read-outs whose halves are whole 16-byte pieces (dv a multiple of 16): a thread takes eight
// pairs, with 16-byte loads of both halves and 32-byte loads of the cosines and sines.
__global__ void turn_back_gate_x8_kernel(const __nv_bfloat16* __restrict__ o, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         const int* __restrict__ tok_pos, const __nv_bfloat16* __restrict__ gate, long long ld_gate,
                                         __nv_bfloat16* __restrict__ out, long long n8, int n_heads, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const int half = dv >> 1, pieces = half >> 3;
    const long long th = i / pieces;
    const int m = (int)(i - th * pieces) * 8;
    const long long t = th / n_heads;
    const int h = (int)(th - t * n_heads);
    const size_t at = (size_t)th * dv + m;
    uint4 lo = *reinterpret_cast<const uint4*>(o + at), hi = *reinterpret_cast<const uint4*>(o + at + half);
    __nv_bfloat162* pl = reinterpret_cast<__nv_bfloat162*>(&lo);
    __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&hi);
    float a[8], b[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 fa = __bfloat1622float2(pl[e]), fb = __bfloat1622float2(ph[e]);
        a[2 * e] = fa.x; a[2 * e + 1] = fa.y;
        b[2 * e] = fb.x; b[2 * e + 1] = fb.y;
    }
    if (cos_t != nullptr) {
        float c[8], s[8];
        const size_t row = (size_t)tok_pos[t] * half + m;
        load32(cos_t + row, c);
        load32(sin_t + row, s);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float ra = a[e] * c[e] + b[e] * s[e], rb = b[e] * c[e] - a[e] * s[e];  // the turn by minus the angle
            a[e] = ra;
            b[e] = rb;
        }
    }
    if (gate != nullptr) {
        const float g = 1.f / (1.f + expf(-__bfloat162float(gate[t * ld_gate + h])));
#pragma unroll
        for (int e = 0; e < 8; ++e) { a[e] *= g; b[e] *= g; }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        pl[e] = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
        ph[e] = __floats2bfloat162_rn(b[2 * e], b[2 * e + 1]);
    }
    *reinterpret_cast<uint4*>(out + at) = lo;
    *reinterpret_cast<uint4*>(out + at + half) = hi;
}

}  // namespace

GK_EXPORT int gk_turn_back_gate(const void* o, const float* cos_t, const float* sin_t, int table_positions, int max_position,
                                const int* tok_pos, const void* gate, long long ld_gate, void* out, int dtype, long long n_tokens,
                                int n_heads, int dv, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && n_heads > 0 && dv > 0 && dv % 2 == 0, "turn_back_gate: bad arguments");
    GK_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "turn_back_gate: a turn needs both tables");
    GK_REQUIRE(cos_t == nullptr || (tok_pos != nullptr && max_position < table_positions),
               "turn_back_gate: position %d is beyond the tables (%d)", max_position, table_positions);
    if (n_tokens == 0) return GK_OK;
    const uintptr_t all = (uintptr_t)o | (uintptr_t)out | (uintptr_t)cos_t | (uintptr_t)sin_t;
    if (dtype == GK_BF16 && dv % 16 == 0 && (all & 31) == 0) {
        const long long n8 = n_tokens * n_heads * (dv / 16);
        const long long blocks8 = (n8 + 255) / 256;
        GK_REQUIRE(blocks8 < 2147483647LL, "turn_back_gate: too many elements");
        gk_launch(turn_back_gate_x8_kernel, dim3((unsigned)blocks8), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)o, cos_t, sin_t,
                  tok_pos, (const __nv_bfloat16*)gate, ld_gate, (__nv_bfloat16*)out, n8, n_heads, dv);
        GK_CHECK_LAUNCH("turn_back_gate");
        return GK_OK;
    }
    const long long n = n_tokens * n_heads * (dv / 2);
    const long long blocks = (n + 255) / 256;
    GK_REQUIRE(blocks < 2147483647LL, "turn_back_gate: too many elements");
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(turn_back_gate_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)o, cos_t, sin_t, tok_pos,
                  (const T*)gate, ld_gate, (T*)out, n, n_heads, dv);
    })
    GK_CHECK_LAUNCH("turn_back_gate");
    return GK_OK;
}

GK_EXPORT int gk_wide_norm_rope_write(const void* proj, int dtype, long long ld, const float* w_q, const float* w_k,
                                      const float* cos_t, const float* sin_t, int table_positions, const int* tok_pos,
                                      const int* tok_seq, const int* slots, const int* block_table, void* q_out, void* k_pages,
                                      void* v_pages, int cache_dtype, int n_tokens, int n_q, int n_kv, int d, int rot,
                                      int max_pages, int page_size, float eps, int max_position, int v_at, int dv, int has_k,
                                      void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && GK_VALID_DTYPE(cache_dtype), "wide_norm_rope_write: bad dtype");
    GK_REQUIRE(n_q > 0 && n_kv > 0 && d > 0, "wide_norm_rope_write: bad sizes");
    GK_REQUIRE(v_at < 0 || dv > 0, "wide_norm_rope_write: values of their own need a size");
    GK_REQUIRE(has_k || k_pages == nullptr, "wide_norm_rope_write: a row without keys writes no pages");
    GK_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= d, "wide_norm_rope_write: %d rotated entries in heads of %d", rot, d);
    GK_REQUIRE(rot == 0 || (cos_t != nullptr && sin_t != nullptr && max_position < table_positions),
               "wide_norm_rope_write: position %d is beyond the rotation tables (%d)", max_position, table_positions);
    if (n_tokens == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    {
        const int vec = dtype == GK_BF16 ? 8 : 4;
        const uintptr_t all = (uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)w_q | (uintptr_t)w_k;
        const long long row_pieces = ((long long)n_q * d + (has_k ? (long long)n_kv * d : 0)) / vec;
        if (rot == 0 && dtype == cache_dtype && d % vec == 0 && ld % vec == 0 && (all & 15) == 0 && row_pieces <= WN_THREADS * WN_HELD &&
            (v_at < 0 || (dv % vec == 0 && v_at % vec == 0))) {
            GK_DISPATCH_DTYPE(dtype, T, {
                gk_launch(wide_norm_write_vec_kernel<T>, dim3(n_tokens), dim3(WN_THREADS), 0, s, (const T*)proj, ld, w_q, w_k, tok_pos, tok_seq,
                          slots, block_table, (T*)q_out, (T*)k_pages, (T*)v_pages, n_q, n_kv, d, max_pages, page_size, eps, v_at, dv, has_k);
            })
            GK_CHECK_LAUNCH("wide_norm_rope_write");
            return GK_OK;
        }
    }
    GK_DISPATCH_DTYPE(dtype, T, {
        GK_DISPATCH_DTYPE(cache_dtype, TC, {
            gk_launch(wide_norm_rope_write_kernel<T, TC>, dim3(n_tokens), dim3(WN_THREADS), 0, s, (const T*)proj, ld, w_q, w_k, cos_t,
                      sin_t, tok_pos, tok_seq, slots, block_table, (T*)q_out, (TC*)k_pages, (TC*)v_pages, n_q, n_kv, d, rot, max_pages,
                      page_size, eps, v_at, dv, has_k);
        })
    })
    GK_CHECK_LAUNCH("wide_norm_rope_write");
    return GK_OK;
}

GK_EXPORT int gk_sigmoid_gate(const void* o, const void* gate, long long ld_gate, void* out, int dtype, long long n_tokens, int width,
                              void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && width > 0, "sigmoid_gate: bad arguments");
    if (n_tokens == 0) return GK_OK;
    const long long n = n_tokens * width;
    const long long blocks = (n + 255) / 256;
    GK_REQUIRE(blocks < 2147483647LL, "sigmoid_gate: too many elements");
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(sigmoid_gate_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)o, (const T*)gate, ld_gate,
                  (T*)out, n, width);
    })
    GK_CHECK_LAUNCH("sigmoid_gate");
    return GK_OK;
}

GK_EXPORT int gk_softcap(float* x, long long n, float cap, void* stream) {
    GK_REQUIRE(cap > 0.f, "softcap: the cap must be positive");
    if (n == 0) return GK_OK;
    const long long blocks = (n + 255) / 256;
    GK_REQUIRE(blocks < 2147483647LL, "softcap: too many elements");
    gk_launch(softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, n, cap);
    GK_CHECK_LAUNCH("softcap");
    return GK_OK;
}
