// Linear attention with a fixed decay per head over many tokens at once: the recurrence
//     S <- g S + k_t v_t^T ;   o_t = S^T q_t                       (g = decay_h, S [d, dv] 32-bit)
// cut into chunks of 64 tokens, so that the work inside a chunk is matrix products that all chunks do side by side and
// only one small step per chunk stays in sequence.  For a chunk of n tokens (i, j count from 0 inside it) that starts
// from the state S0:
//     L    = sum_j g^(n-1-j) k_j v_j^T                               (local:  what the chunk adds to the state)
//     S1   = g^n S0 + L                                               (carry:  the state behind the chunk)
//     o_i  = g^(i+1) S0^T q_i + sum_{j<=i} g^(i-j) (q_i . k_j) v_j    (read:   from the state before, and inside)
// Every power of g has a non-negative exponent, so nothing grows: decays of 0 and of 1 are as good as any.  Three
// kernels a wave of chunks: `local` (a block per chunk, head and 64 value columns), `carry` (an element of the state
// per thread, the wave's chunks in sequence; it leaves S0 of every chunk where L was), `read` (a block per chunk, head
// and 64 value columns; S0's columns come into shared memory where the keys were, once the weights are formed).  All arithmetic is 32-bit on the FP32 pipe: products of 4 x 4 register tiles whose operands
// come from shared memory as 16-byte vectors.  A token's sums have another order than in the token-by-token kernel:
// the two agree within rounding, not bit by bit.

#include "common.cuh"

namespace {

constexpr int CHUNK = 64;
constexpr int LDT = CHUNK + 4;  // row stride of the transposed tiles: 16-byte aligned, and rows start 4 banks apart
constexpr int THREADS = 256;    // 16 x 16 threads, a 4 x 4 tile each: 64 x 64 results a pass

__device__ __forceinline__ void powers(float* pw, float g) {
    for (int n = threadIdx.x; n <= CHUNK; n += THREADS) pw[n] = n == 0 ? 1.f : powf(g, (float)n);
}

// L of one chunk, 64 value columns a block.  ws [n_seqs, wave, H, d, dv].
__global__ void __launch_bounds__(THREADS) decay_chunk_local_kernel(
    const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ decay, float* __restrict__ ws,
    const int* __restrict__ cu_q, int n_heads, int d, int dv, int chunk0, int wave, int col_tiles) {
    extern __shared__ __align__(16) float smem[];
    float* ks = smem;                 // [CHUNK][d], row j times g^(n-1-j)
    float* vs = ks + CHUNK * d;       // [CHUNK][64]
    float* pw = vs + CHUNK * CHUNK;   // [CHUNK + 1]
    pdl_launch_dependents();
    const int in_wave = blockIdx.x / col_tiles, c0 = (blockIdx.x - in_wave * col_tiles) * CHUNK;
    const int head = blockIdx.y, seq = blockIdx.z;
    powers(pw, decay[head]);
    pdl_wait();
    const int t0 = cu_q[seq], len = cu_q[seq + 1] - t0;
    const int first = (chunk0 + in_wave) * CHUNK;
    if (first >= len) return;
    const int n = min(CHUNK, len - first);
    __syncthreads();
    const int dq = d >> 2;
    for (int i = threadIdx.x; i < CHUNK * dq; i += THREADS) {
        const int j = i / dq, c4 = (i - j * dq) << 2;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < n) {
            x = *reinterpret_cast<const float4*>(k + ((size_t)(t0 + first + j) * n_heads + head) * d + c4);
            const float w = pw[n - 1 - j];
            x.x *= w, x.y *= w, x.z *= w, x.w *= w;
        }
        *reinterpret_cast<float4*>(ks + j * d + c4) = x;
    }
    for (int i = threadIdx.x; i < CHUNK * (CHUNK / 4); i += THREADS) {
        const int j = i >> 4, c4 = (i & 15) << 2;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < n && c0 + c4 < dv) x = *reinterpret_cast<const float4*>(v + ((size_t)(t0 + first + j) * n_heads + head) * dv + c0 + c4);
        *reinterpret_cast<float4*>(vs + j * CHUNK + c4) = x;
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int col = c0 + tx * 4;
    float* dst = ws + (((size_t)seq * wave + in_wave) * n_heads + head) * (size_t)d * dv;
    for (int r0 = 0; r0 < d; r0 += CHUNK) {
        const int row = r0 + ty * 4;
        if (row >= d) continue;  // no barrier below
        float acc[4][4] = {};
#pragma unroll 4
        for (int j = 0; j < n; ++j) {
            const float4 a = *reinterpret_cast<const float4*>(ks + j * d + row);
            const float4 b = *reinterpret_cast<const float4*>(vs + j * CHUNK + tx * 4);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int p = 0; p < 4; ++p)
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[p][r] = fmaf(av[p], bv[r], acc[p][r]);
        }
        if (col < dv) {
#pragma unroll
            for (int p = 0; p < 4; ++p)
                *reinterpret_cast<float4*>(dst + (size_t)(row + p) * dv + col) = make_float4(acc[p][0], acc[p][1], acc[p][2], acc[p][3]);
        }
    }
}

// The wave's chunks in sequence, four entries of the state a thread: ws goes from L to S0 chunk by chunk, and the
// state in the sequence's slot from before the wave to behind it.
__global__ void __launch_bounds__(THREADS) decay_chunk_carry_kernel(
    float* __restrict__ ws, float* __restrict__ state, const float* __restrict__ decay, const int* __restrict__ cu_q,
    const int* __restrict__ slots, int n_heads, int size4 /* d * dv / 4 */, int chunk0, int wave) {
    pdl_launch_dependents();
    const int e = blockIdx.x * THREADS + threadIdx.x;
    const int head = blockIdx.y, seq = blockIdx.z;
    const float g = decay[head];
    pdl_wait();
    if (e >= size4) return;
    const int len = cu_q[seq + 1] - cu_q[seq];
    const int here = min(wave, (len + CHUNK - 1) / CHUNK - chunk0);
    if (here <= 0) return;
    float4* st = reinterpret_cast<float4*>(state + ((size_t)slots[seq] * n_heads + head) * (size_t)size4 * 4) + e;
    float4* w = reinterpret_cast<float4*>(ws + ((size_t)seq * wave * n_heads + head) * (size_t)size4 * 4) + e;
    const size_t step = (size_t)n_heads * size4;
    float4 s = *st;
    const float g_full = powf(g, (float)CHUNK);
    constexpr int AHEAD = 8;  // loads in flight: the chain itself is one multiply-add a chunk
    for (int c0 = 0; c0 < here; c0 += AHEAD) {
        float4 add[AHEAD];
#pragma unroll
        for (int a = 0; a < AHEAD; ++a)
            if (c0 + a < here) add[a] = __ldcg(w + (size_t)a * step);
#pragma unroll
        for (int a = 0; a < AHEAD; ++a) {
            if (c0 + a >= here) break;
            const int n = min(CHUNK, len - (chunk0 + c0 + a) * CHUNK);
            const float gn = n == CHUNK ? g_full : powf(g, (float)n);
            __stcg(w + (size_t)a * step, s);
            s.x = fmaf(gn, s.x, add[a].x), s.y = fmaf(gn, s.y, add[a].y), s.z = fmaf(gn, s.z, add[a].z), s.w = fmaf(gn, s.w, add[a].w);
        }
        w += (size_t)AHEAD * step;
    }
    *st = s;
}

// o of one chunk, 64 value columns a block, from S0 (in ws) and the chunk's own keys and values.
__global__ void __launch_bounds__(THREADS) decay_chunk_read_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ decay,
    const float* __restrict__ ws, float* __restrict__ out, const int* __restrict__ cu_q, int n_heads, int d, int dv, int chunk0,
    int wave, int col_tiles) {
    extern __shared__ __align__(16) float smem[];
    float* qt = smem;                  // [d][LDT]: entry kk of token i at qt[kk * LDT + i]
    float* kt = qt + d * LDT;          // [d][LDT]
    float* vs = kt + d * LDT;          // [CHUNK][64]
    float* pt = vs + CHUNK * CHUNK;    // [CHUNK][LDT]: weight of key j for token i at pt[j * LDT + i]
    float* pw = pt + CHUNK * LDT;      // [CHUNK + 1]
    pdl_launch_dependents();
    const int in_wave = blockIdx.x / col_tiles, c0 = (blockIdx.x - in_wave * col_tiles) * CHUNK;
    const int head = blockIdx.y, seq = blockIdx.z;
    powers(pw, decay[head]);
    pdl_wait();
    const int t0 = cu_q[seq], len = cu_q[seq + 1] - t0;
    const int first = (chunk0 + in_wave) * CHUNK;
    if (first >= len) return;
    const int n = min(CHUNK, len - first);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = warp; i < CHUNK; i += THREADS / 32) {
        const size_t at = ((size_t)(t0 + first + i) * n_heads + head) * d;
        for (int kk = lane; kk < d; kk += 32) {
            qt[kk * LDT + i] = i < n ? q[at + kk] : 0.f;
            kt[kk * LDT + i] = i < n ? k[at + kk] : 0.f;
        }
    }
    for (int i = threadIdx.x; i < CHUNK * (CHUNK / 4); i += THREADS) {
        const int j = i >> 4, c4 = (i & 15) << 2;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < n && c0 + c4 < dv) x = *reinterpret_cast<const float4*>(v + ((size_t)(t0 + first + j) * n_heads + head) * dv + c0 + c4);
        *reinterpret_cast<float4*>(vs + j * CHUNK + c4) = x;
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int i0 = ty * 4;
    {   // weights of the chunk's own keys: g^(i-j) (q_i . k_j) for j <= i
        const int j0 = tx * 4;
        float acc[4][4] = {};
        if (j0 <= i0 + 3) {
#pragma unroll 4
            for (int kk = 0; kk < d; ++kk) {
                const float4 a = *reinterpret_cast<const float4*>(qt + kk * LDT + i0);
                const float4 b = *reinterpret_cast<const float4*>(kt + kk * LDT + j0);
                const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int p = 0; p < 4; ++p)
#pragma unroll
                    for (int r = 0; r < 4; ++r) acc[p][r] = fmaf(av[p], bv[r], acc[p][r]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float w[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const int i = i0 + p, j = j0 + r;
                w[p] = j <= i ? acc[p][r] * pw[i - j] : 0.f;
            }
            *reinterpret_cast<float4*>(pt + (j0 + r) * LDT + i0) = make_float4(w[0], w[1], w[2], w[3]);
        }
    }
    __syncthreads();
    // the keys' tile has done its work: the 64 columns of S0 take its place
    float* s0 = kt;  // [d][64]
    {
        const float* src = ws + (((size_t)seq * wave + in_wave) * n_heads + head) * (size_t)d * dv + c0;
        for (int i = threadIdx.x; i < d * (CHUNK / 4); i += THREADS) {
            const int kk = i >> 4, c4 = (i & 15) << 2;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c0 + c4 < dv) x = __ldcg(reinterpret_cast<const float4*>(src + (size_t)kk * dv + c4));
            *reinterpret_cast<float4*>(s0 + kk * CHUNK + c4) = x;
        }
    }
    __syncthreads();
    const int col = c0 + tx * 4;
    if (col >= dv || i0 >= n) return;  // no barrier below
    float acc[4][4] = {};
#pragma unroll 4
    for (int kk = 0; kk < d; ++kk) {
        const float4 a = *reinterpret_cast<const float4*>(qt + kk * LDT + i0);
        const float4 b = *reinterpret_cast<const float4*>(s0 + kk * CHUNK + tx * 4);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int p = 0; p < 4; ++p)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[p][r] = fmaf(av[p], bv[r], acc[p][r]);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float w = pw[i0 + p + 1];
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[p][r] *= w;
    }
    const int last = min(n, i0 + 4);  // keys behind the tile's last token weigh nothing
#pragma unroll 4
    for (int j = 0; j < last; ++j) {
        const float4 a = *reinterpret_cast<const float4*>(pt + j * LDT + i0);
        const float4 b = *reinterpret_cast<const float4*>(vs + j * CHUNK + tx * 4);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int p = 0; p < 4; ++p)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[p][r] = fmaf(av[p], bv[r], acc[p][r]);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p)
        if (i0 + p < n)
            *reinterpret_cast<float4*>(out + ((size_t)(t0 + first + i0 + p) * n_heads + head) * dv + col) =
                make_float4(acc[p][0], acc[p][1], acc[p][2], acc[p][3]);
}

size_t local_smem(int d) { return (size_t)(CHUNK * d + CHUNK * CHUNK + CHUNK + 4) * sizeof(float); }
size_t read_smem(int d) { return (size_t)(2 * d * LDT + CHUNK * CHUNK + CHUNK * LDT + CHUNK + 4) * sizeof(float); }

}  // namespace

// Heads that the chunked kernels take: rows of 16-byte vectors, tiles within shared memory.
static bool chunked_fits(int d, int dv) {
    return d > 0 && dv > 0 && d % 4 == 0 && dv % 4 == 0 && read_smem(d) <= 200 * 1024 && local_smem(d) <= 200 * 1024;
}

// The recurrence over the step's tokens of every sequence, from and to state [slots, H, d, dv]; q, k [T, H, d],
// v [T, H, dv], out [T, H, dv], all 32-bit.  `max_len` bounds the sequences' token counts in this step; `ws` holds
// n_seqs * wave * H * d * dv floats, `wave` chunks of every sequence are in flight at a time.
GK_EXPORT int gk_decay_scan_chunked(const float* q, const float* k, const float* v, const float* decay, float* state, float* out,
                                    float* ws, const int* cu_q, const int* slots, int n_seqs, int n_heads, int d, int dv, int max_len,
                                    int wave, void* stream) {
    GK_REQUIRE(n_heads > 0 && n_heads <= 65535 && n_seqs >= 0 && n_seqs <= 65535, "decay_scan_chunked: bad counts");
    GK_REQUIRE(chunked_fits(d, dv), "decay_scan_chunked: heads of %d / %d do not fit (multiples of 4, keys up to about 300)", d, dv);
    GK_REQUIRE(max_len >= 0 && wave > 0 && ws != nullptr, "decay_scan_chunked: bad sizes");
    if (n_seqs == 0 || max_len == 0) return GK_OK;
    static bool prepared = false;
    if (!prepared) {
        cudaFuncSetAttribute(decay_chunk_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(decay_chunk_read_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        prepared = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int chunks = (max_len + CHUNK - 1) / CHUNK, col_tiles = (dv + CHUNK - 1) / CHUNK, size4 = d * dv / 4;
    for (int chunk0 = 0; chunk0 < chunks; chunk0 += wave) {
        const int here = chunks - chunk0 < wave ? chunks - chunk0 : wave;
        const dim3 tiles(here * col_tiles, n_heads, n_seqs);
        gk_launch(decay_chunk_local_kernel, tiles, dim3(THREADS), local_smem(d), s, k, v, decay, ws, cu_q, n_heads, d, dv, chunk0, wave,
                  col_tiles);
        gk_launch(decay_chunk_carry_kernel, dim3((size4 + THREADS - 1) / THREADS, n_heads, n_seqs), dim3(THREADS), 0, s, ws, state, decay,
                  cu_q, slots, n_heads, size4, chunk0, wave);
        gk_launch(decay_chunk_read_kernel, tiles, dim3(THREADS), read_smem(d), s, q, k, v, decay, (const float*)ws, out, cu_q, n_heads, d,
                  dv, chunk0, wave, col_tiles);
    }
    GK_CHECK_LAUNCH("decay_scan_chunked");
    return GK_OK;
}
