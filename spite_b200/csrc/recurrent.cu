// Recurrent mixers whose state is a matrix per head, carried from token to token in float32.
//
// mlstm_scan: the matrix memory with exponential gates and a running maximum (one request's state per slot):
//     i_t = cap tanh((a_t + b_i) / cap)                      a_t, c_t: the gates' columns of the projection
//     f_t = logsigmoid(cap tanh((c_t + b_f) / cap))
//     m_t = max(f_t + m_(t-1), i_t)
//     S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        (n_t alike, with k_t alone)
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),   q_t scaled by q_scale
// A state that is all zeros (m included) is the start of a sequence.  Everything is float32: the inputs are the
// float32 sums of the projection, and no intermediate is rounded below that.
//
// One kernel serves prompt portions and decoded tokens: a block owns 32 value columns of one (segment, head) and
// walks the segment's tokens in order; a warp owns 8 of the columns, a lane the key rows lane, lane + 32, ... of
// them (RPL rows a lane), so the sums over the key rows are warp shuffles and no block-wide barrier stands in the
// token loop.  The next token's inputs are loaded while the current one is worked on.  A decoded token costs one
// read and one write of the state (a lane moves 8 consecutive floats of a key row: whole 32-byte sectors).
#include "common.cuh"

struct MlstmParams {
    const float* proj;          // [tokens, stride]: the projection's float32 output
    long long stride;
    int q_col, k_col, v_col, i_col, f_col;   // first column of q [heads * dim], k [heads * dim], v [heads * vdim], i [heads], f [heads]
    const float* i_bias;        // [heads]
    const float* f_bias;        // [heads]
    float* out;                 // [tokens, heads * vdim]
    // [slots, heads, head_stride]: S row-major [dim, vdim], then for every block of 32 value columns its own copy of
    // n [dim] and m, each copy rounded up to a multiple of four floats (a block reads and writes its own copy only, so
    // no block reads what another block of the same step has already renewed)
    float* state;
    long long head_stride;      // floats of one head's state (>= dim * vdim + ceil(vdim / 32) * round_up(dim + 1, 4))
    const int* cu_seqlens;      // [segments + 1]: a segment's tokens are the rows cu[s] .. cu[s + 1] - 1
    const int* slots;           // [segments]: the state slot of a segment's request
    int n_segments, heads, dim, vdim;
    float gate_cap, q_scale;
    int chunked;                // not 0: segments are walked 32 tokens at a time (prompts and their portions)
};

namespace {

constexpr int COLS_PER_WARP = 8;
constexpr int COLS_PER_BLOCK = 32;

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <int RPL>
__global__ void __launch_bounds__(128) mlstm_scan_kernel(const MlstmParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int seg = blockIdx.z, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c0 = blockIdx.x * COLS_PER_BLOCK + warp * COLS_PER_WARP;       // this warp's first value column
    const int t0 = p.cu_seqlens[seg], t1 = p.cu_seqlens[seg + 1];
    const int dim = p.dim, vdim = p.vdim;
    if (t0 >= t1) return;
    const int slot = p.slots[seg];
    // A captured step pads its rows with copies of its first row: a copy would update the first row's state a second
    // time.  It leaves zeros instead (its results are never read).
    if (seg > 0 && slot == p.slots[0]) {
        for (int t = t0; t < t1; ++t)
            for (int c = lane; c < COLS_PER_WARP; c += 32)
                if (c0 + c < vdim) p.out[(size_t)t * p.heads * vdim + (size_t)head * vdim + c0 + c] = 0.f;
        return;
    }
    float* st = p.state + ((size_t)slot * p.heads + head) * (size_t)p.head_stride;
    float* st_n = st + (size_t)dim * vdim + (size_t)blockIdx.x * ((dim + 1 + 3) & ~3);
    // a key row's 8 columns move as two groups of four floats where every such group is aligned
    const bool full_cols = c0 + COLS_PER_WARP <= vdim && (vdim % 4) == 0 && (p.head_stride % 4) == 0 &&
                           (((uintptr_t)p.state) & 15) == 0;

    float S[RPL][COLS_PER_WARP], n[RPL];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int d = lane + 32 * r;
        n[r] = 0.f;
#pragma unroll
        for (int c = 0; c < COLS_PER_WARP; ++c) S[r][c] = 0.f;
        if (d < dim) {
            n[r] = st_n[d];
            if (c0 >= vdim) continue;
            const float* row = st + (size_t)d * vdim + c0;
            if (full_cols) {
                const float4 a = *(const float4*)row, b = *(const float4*)(row + 4);
                S[r][0] = a.x; S[r][1] = a.y; S[r][2] = a.z; S[r][3] = a.w;
                S[r][4] = b.x; S[r][5] = b.y; S[r][6] = b.z; S[r][7] = b.w;
            } else {
#pragma unroll
                for (int c = 0; c < COLS_PER_WARP; ++c)
                    if (c0 + c < vdim) S[r][c] = row[c];
            }
        }
    }
    float m = st_n[dim];
    __syncthreads();             // every warp of the block has read n and m before the first warp to finish renews them
    if (c0 >= vdim) return;

    // the inputs of one token: q and k by key row, v by column (lane c < 8 holds column c0 + c), the two gates
    float q[RPL], k[RPL], v = 0.f, gi = 0.f, gf = 0.f;
    auto load = [&](int t, float (&qq)[RPL], float (&kk)[RPL], float& vv, float& ii, float& ff) {
        const float* row = p.proj + (size_t)t * p.stride;
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int d = lane + 32 * r;
            qq[r] = d < dim ? row[p.q_col + head * dim + d] * p.q_scale : 0.f;
            kk[r] = d < dim ? row[p.k_col + head * dim + d] : 0.f;
        }
        vv = (lane < COLS_PER_WARP && c0 + lane < vdim) ? row[p.v_col + head * vdim + c0 + lane] : 0.f;
        ii = row[p.i_col + head];
        ff = row[p.f_col + head];
    };
    load(t0, q, k, v, gi, gf);
    const float bi = p.i_bias ? p.i_bias[head] : 0.f, bf = p.f_bias ? p.f_bias[head] : 0.f;
    const float cap = p.gate_cap, inv_cap = 1.0f / p.gate_cap;

    for (int t = t0; t < t1; ++t) {
        float qn[RPL], kn[RPL], vn = 0.f, gin = 0.f, gfn = 0.f;
        if (t + 1 < t1) load(t + 1, qn, kn, vn, gin, gfn);
        else {
#pragma unroll
            for (int r = 0; r < RPL; ++r) qn[r] = kn[r] = 0.f;
        }
        const float ig = cap * tanhf((gi + bi) * inv_cap);
        const float fg = log_sigmoid(cap * tanhf((gf + bf) * inv_cap));
        const float m_new = fmaxf(fg + m, ig);
        const float keep = expf(fg + m - m_new), take = expf(ig - m_new);
        m = m_new;
        float vc[COLS_PER_WARP];
#pragma unroll
        for (int c = 0; c < COLS_PER_WARP; ++c) vc[c] = __shfl_sync(0xffffffffu, v, c);
        float num[COLS_PER_WARP], nq = 0.f;
#pragma unroll
        for (int c = 0; c < COLS_PER_WARP; ++c) num[c] = 0.f;
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const float tk = take * k[r];
            n[r] = keep * n[r] + tk;
            nq = fmaf(n[r], q[r], nq);
#pragma unroll
            for (int c = 0; c < COLS_PER_WARP; ++c) {
                S[r][c] = fmaf(tk, vc[c], keep * S[r][c]);
                num[c] = fmaf(S[r][c], q[r], num[c]);
            }
        }
        nq = warp_sum(nq);
#pragma unroll
        for (int c = 0; c < COLS_PER_WARP; ++c) num[c] = warp_sum(num[c]);
        const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
        float mine = 0.f;
#pragma unroll
        for (int c = 0; c < COLS_PER_WARP; ++c)
            if (lane == c) mine = num[c];
        if (lane < COLS_PER_WARP && c0 + lane < vdim)
            p.out[(size_t)t * p.heads * vdim + (size_t)head * vdim + c0 + lane] = mine / den;
#pragma unroll
        for (int r = 0; r < RPL; ++r) { q[r] = qn[r]; k[r] = kn[r]; }
        v = vn; gi = gin; gf = gfn;
    }

#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int d = lane + 32 * r;
        if (d >= dim) continue;
        float* row = st + (size_t)d * vdim + c0;
        if (full_cols) {
            *(float4*)row = make_float4(S[r][0], S[r][1], S[r][2], S[r][3]);
            *(float4*)(row + 4) = make_float4(S[r][4], S[r][5], S[r][6], S[r][7]);
        } else {
#pragma unroll
            for (int c = 0; c < COLS_PER_WARP; ++c)
                if (c0 + c < vdim) row[c] = S[r][c];
        }
        if (warp == 0) st_n[d] = n[r];                           // (the same in every warp of the block)
    }
    if (warp == 0 && lane == 0) st_n[dim] = m;
}

// ---- the same recurrence, 32 tokens at a time (prompts and their portions).
// With F_t the sum of the log forget gates from the chunk's first token to t, a_s = i_s - F_s, m0 the maximum the chunk
// starts from and M_t = max(m0, max_{s<=t} a_s), the recurrence unrolls to m_t = F_t + M_t and
//     S_t = exp(m0 - M_t) S_0 + sum_{s<=t} exp(a_s - M_t) k_s v_s^T                 (n_t alike)
// so a chunk is small matrix products in float32 on the CUDA cores, none of which waits for a token before it:
//     q k^T and the gates' a_s, F_t   (they do not depend on the state: a kernel of its own computes them for every
//                                      chunk and head of the step at once, into working memory),
//     [q S_0 | q n_0]                 (tokens x (32 value columns, 1), over the key rows),
//     numerators = exp(m0 - M_t) q S_0 + sum_{s<=t} exp(a_s - M_t) (q_t . k_s) v_s   (the denominator's n . q alike),
//     S <- exp(m0 - M_last) S + sum_s exp(a_s - M_last) k_s v_s^T.
// Every exponent is <= 0.  In the second kernel a block owns 32 value columns of one (segment, head), as in the kernel
// above, with the state tile, the chunk's q, k and v in shared memory; 256 threads.
constexpr int CL = 32;            // tokens of a chunk
constexpr int SROW = 36;          // floats of a row of the state tile: 32 value columns, n, three zeros

template <int RPL2> struct ChunkSmem {
    static constexpr int DP = 64 * RPL2;          // key rows, padded with zeros
    static constexpr int FLOATS = DP * SROW + 2 * CL * DP + 3 * CL * CL + 7 * CL + 4;      // (two of the small arrays hold doubles)
    // 115,600 bytes at 256 key rows: two blocks fit a multiprocessor
};

__device__ __forceinline__ double warp_prefix_sum(double v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
    }
    return v;
}
__device__ __forceinline__ double warp_prefix_max(double v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v = fmax(v, u);
    }
    return v;
}

constexpr int CHUNK_RECORD = CL * CL + 4 * CL;   // floats a chunk and head: q k^T [CL][CL], then a_s and F_t as doubles, each [CL]

// the number of chunks of the segments before `seg` (chunks are numbered segment by segment)
__device__ __forceinline__ int chunks_before(const int* cu_seqlens, int seg) {
    int n = 0;
    for (int s = 0; s < seg; ++s) n += (cu_seqlens[s + 1] - cu_seqlens[s] + CL - 1) / CL;
    return n;
}

// What a chunk needs that does not depend on the state: the scores q_t . k_s (s <= t, q not yet scaled) and, from the
// gates, F_t and a_s = i_s - F_s as doubles (-1e300 behind the segment's end).  One block a (chunk, head).
template <int RPL2>
__global__ void __launch_bounds__(256) mlstm_scores_kernel(const MlstmParams p, float* __restrict__ scratch) {
    constexpr int DP = 64 * RPL2, ROW = DP + 4;
    extern __shared__ __align__(16) float sm[];
    float* q_s = sm;                              // [CL][ROW]
    float* k_s = q_s + CL * ROW;                  // [CL][ROW]
    pdl_wait();
    pdl_launch_dependents();
    const int head = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int seg = 0, rest = blockIdx.x;
    for (; seg < p.n_segments; ++seg) {
        const int n = (p.cu_seqlens[seg + 1] - p.cu_seqlens[seg] + CL - 1) / CL;
        if (rest < n) break;
        rest -= n;
    }
    if (seg >= p.n_segments) return;
    const int c0 = p.cu_seqlens[seg] + rest * CL, len = min(CL, p.cu_seqlens[seg + 1] - c0), dim = p.dim;
    float* rec = scratch + ((size_t)blockIdx.x * p.heads + head) * CHUNK_RECORD;
    const float* rows = p.proj + (size_t)c0 * p.stride;
    const bool vec4 = (dim % 4) == 0 && (p.stride % 4) == 0 && (p.q_col % 4) == 0 && (p.k_col % 4) == 0 && (((uintptr_t)p.proj) & 15) == 0;
    if (vec4) {
#pragma unroll 4
        for (int e = tid; e < CL * (DP / 4); e += 256) {
            const int t = e / (DP / 4), d = (e - t * (DP / 4)) * 4;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
            if (t < len && d < dim) {
                a = *(const float4*)&rows[(size_t)t * p.stride + p.q_col + head * dim + d];
                b = *(const float4*)&rows[(size_t)t * p.stride + p.k_col + head * dim + d];
            }
            *(float4*)&q_s[t * ROW + d] = a;
            *(float4*)&k_s[t * ROW + d] = b;
        }
    } else {
        for (int e = tid; e < CL * DP; e += 256) {
            const int t = e / DP, d = e - t * DP;
            const bool on = t < len && d < dim;
            q_s[t * ROW + d] = on ? rows[(size_t)t * p.stride + p.q_col + head * dim + d] : 0.f;
            k_s[t * ROW + d] = on ? rows[(size_t)t * p.stride + p.k_col + head * dim + d] : 0.f;
        }
    }
    if (warp == 0) {
        const bool on = lane < len;
        const float bi = p.i_bias ? p.i_bias[head] : 0.f, bf = p.f_bias ? p.f_bias[head] : 0.f;
        const float cap = p.gate_cap, inv_cap = 1.0f / p.gate_cap;
        float ig = 0.f, fg = 0.f;
        if (on) {
            ig = cap * tanhf((rows[(size_t)lane * p.stride + p.i_col + head] + bi) * inv_cap);
            fg = log_sigmoid(cap * tanhf((rows[(size_t)lane * p.stride + p.f_col + head] + bf) * inv_cap));
        }
        const double F = warp_prefix_sum((double)fg, lane);
        double* gd = reinterpret_cast<double*>(rec + CL * CL);
        gd[lane] = on ? (double)ig - F : -1.0e300;
        gd[CL + lane] = F;
    }
    __syncthreads();
    {   // a thread has one token and the keys sg, sg + 8, ... (rows 8 apart: eight lanes read eight banks' worth)
        const int t = tid >> 3, sg = tid & 7;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (t < len) {
            for (int d = 0; d < DP; d += 4) {
                const float4 qv = *(const float4*)&q_s[t * ROW + d];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (sg + 8 * j > t) continue;
                    const float4 kv = *(const float4*)&k_s[(sg + 8 * j) * ROW + d];
                    acc[j] = fmaf(qv.x, kv.x, acc[j]); acc[j] = fmaf(qv.y, kv.y, acc[j]);
                    acc[j] = fmaf(qv.z, kv.z, acc[j]); acc[j] = fmaf(qv.w, kv.w, acc[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) rec[t * CL + sg + 8 * j] = acc[j];
    }
}

__device__ __forceinline__ void copy16_async(void* smem, const void* gmem, int src_bytes) {     // the rest of the 16 bytes: zeros
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

template <int RPL2>
__global__ void __launch_bounds__(256, RPL2 <= 4 ? 2 : 1) mlstm_chunk_kernel(const MlstmParams p, const float* __restrict__ scratch) {
    constexpr int DP = ChunkSmem<RPL2>::DP;
    extern __shared__ __align__(16) float sm[];
    float* S_s = sm;                              // [DP][SROW]: the state's 32 columns, then n
    // [CL][DP]; element d of token t lies at d ^ 4 (t & 7), so that the rows of eight tokens in a row, read four
    // floats at a time at the same d, fall on different banks
    float* q_s = S_s + DP * SROW;                 // (not yet scaled: q_scale multiplies the sums)
    float* k_s = q_s + CL * DP;                   // [CL][DP]
    float* v_s = k_s + CL * DP;                 // [CL][32]: the block's value columns
    float* X0 = v_s + CL * CL;                    // [CL][32]: q S_0 scaled by exp(m0 - M_t)
    float* X1 = X0 + CL * CL;                     // [CL][CL]: q k^T, then weighted and masked
    // a_s and M_t as doubles: they are differences of sums over the chunk's gates, and exp(a_s - M_t) is to be as exact
    // as exp of a single gate in the walk token by token, also where the gates are large
    double* g_a = reinterpret_cast<double*>(X1 + CL * CL);
    double* g_M = g_a + CL;
    float* g_m = reinterpret_cast<float*>(g_M + CL);       // [CL] each: m_t, exp(m0 - M_t), exp(a_s - M_last)
    float* g_g = g_m + CL;
    float* g_w = g_g + CL;
    float* g_last_s = g_w + CL;                   // [1]: exp(m0 - M_last)

    pdl_wait();
    pdl_launch_dependents();
    const int seg = blockIdx.z, head = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cb0 = blockIdx.x * 32;
    const int t0 = p.cu_seqlens[seg], t1 = p.cu_seqlens[seg + 1];
    const int dim = p.dim, vdim = p.vdim;
    if (t0 >= t1) return;
    const int slot = p.slots[seg];
    const size_t out_stride = (size_t)p.heads * vdim;
    if (seg > 0 && slot == p.slots[0]) {          // a padding row of a captured step (see the kernel above)
        for (int e = tid; e < (t1 - t0) * 32; e += 256)
            if (cb0 + (e & 31) < vdim) p.out[(size_t)(t0 + (e >> 5)) * out_stride + (size_t)head * vdim + cb0 + (e & 31)] = 0.f;
        return;
    }
    float* st = p.state + ((size_t)slot * p.heads + head) * (size_t)p.head_stride;
    float* st_n = st + (size_t)dim * vdim + (size_t)blockIdx.x * ((dim + 1 + 3) & ~3);
    for (int e = tid; e < DP * SROW; e += 256) {
        const int d = e / SROW, c = e - d * SROW;
        float x = 0.f;
        if (d < dim) {
            if (c < 32) { if (cb0 + c < vdim) x = st[(size_t)d * vdim + cb0 + c]; }
            else if (c == 32) x = st_n[d];
        }
        S_s[e] = x;
    }
    float m_run = st_n[dim];
    // q and k rows move as groups of four floats where every such group is aligned
    const bool vec4 = (dim % 4) == 0 && (p.stride % 4) == 0 && (p.q_col % 4) == 0 && (p.k_col % 4) == 0 && (((uintptr_t)p.proj) & 15) == 0;

    // The next chunk's inputs are asked for while the current one is worked on: q and k by asynchronous copies of 16
    // bytes straight into shared memory (q once the products that read it are done, k once the state is renewed), the
    // 32 x 32 values and the gates into registers.  Rows that are not 16-byte aligned are loaded at the chunk's start.
    auto fetch_rows = [&](int c, int col, float* dst, bool swizzle) {
        if (!vec4 || c >= t1) return;
        const float* rows = p.proj + (size_t)c * p.stride + col + head * dim;
        const int len = min(CL, t1 - c);
#pragma unroll 4
        for (int e = tid; e < CL * (DP / 4); e += 256) {
            const int t = e / (DP / 4), d = (e - t * (DP / 4)) * 4;
            const bool on = t < len && d < dim;
            copy16_async(&dst[t * DP + (swizzle ? (d ^ ((t & 7) << 2)) : d)], on ? (const void*)&rows[(size_t)t * p.stride + d] : (const void*)p.proj, on ? 16 : 0);
        }
        copy_async_commit();
    };
    float v_next[4];
    float4 qk_next = make_float4(0.f, 0.f, 0.f, 0.f);        // four of the chunk's scores: token tid / 8, keys 4 (tid % 8) ...
    double a_next = 0.0, F_next = 0.0;                        // warp 0: a lane a token
    int chunk_id = chunks_before(p.cu_seqlens, seg);
    auto fetch_small = [&](int c, int chunk) {
        if (c >= t1) return;
        const float* rows = p.proj + (size_t)c * p.stride;
        const int len = min(CL, t1 - c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + 256 * i, t = e >> 5, cc = e & 31;
            v_next[i] = (t < len && cb0 + cc < vdim) ? rows[(size_t)t * p.stride + p.v_col + head * vdim + cb0 + cc] : 0.f;
        }
        const float* rec = scratch + ((size_t)chunk * p.heads + head) * CHUNK_RECORD;
        qk_next = *(const float4*)&rec[tid * 4];
        if (warp == 0) {
            const double* gd = reinterpret_cast<const double*>(rec + CL * CL);
            a_next = gd[lane];
            F_next = gd[CL + lane];
        }
    };
    fetch_rows(t0, p.q_col, q_s, true);
    fetch_rows(t0, p.k_col, k_s, false);
    fetch_small(t0, chunk_id);

    for (int c0 = t0; c0 < t1; c0 += CL, ++chunk_id) {
        const int len = min(CL, t1 - c0);
        // ---- the chunk's q, k and v are in place; the gates and what follows from them (warp 0, a lane a token)
        if (vec4) copy_async_wait_all();
        else {
            const float* rows = p.proj + (size_t)c0 * p.stride;
            for (int e = tid; e < CL * DP; e += 256) {
                const int t = e / DP, d = e - t * DP;
                const bool on = t < len && d < dim;
                q_s[t * DP + (d ^ ((t & 7) << 2))] = on ? rows[(size_t)t * p.stride + p.q_col + head * dim + d] : 0.f;
                k_s[t * DP + d] = on ? rows[(size_t)t * p.stride + p.k_col + head * dim + d] : 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) v_s[tid + 256 * i] = v_next[i];
        *(float4*)&X1[tid * 4] = qk_next;
        if (warp == 0) {
            const bool on = lane < len;
            const double a = a_next, F = F_next;
            const double M = fmax((double)m_run, warp_prefix_max(a, lane));
            const double M_last = __shfl_sync(0xffffffffu, M, len - 1), F_last = __shfl_sync(0xffffffffu, F, len - 1);
            g_a[lane] = a;
            g_M[lane] = M;
            g_m[lane] = (float)(F + M);
            g_g[lane] = expf((float)((double)m_run - M));
            // The maximum goes on as a float.  The state is scaled to that rounded value, not to the sum it was rounded
            // from, so that state and maximum agree exactly, as they do in the walk token by token.
            const float m_next = (float)(F_last + M_last);
            const double M_state = (double)m_next - F_last;
            g_w[lane] = on ? expf((float)(a - M_state)) : 0.f;
            if (lane == 0) g_last_s[0] = expf((float)((double)m_run - M_state));
            m_run = m_next;
        }
        __syncthreads();

        // ---- q S_0: a thread has 4 tokens (tg, tg + 8, ...) by 4 columns over a quarter of the key rows (every fourth
        // group of four); the quarters meet by shuffles, and the lane of quarter kq writes token tg + 8 kq
        {
            const int kq = lane >> 3, tg = lane & 7, cg = warp;
            float acc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
            for (int d = 4 * kq; d < DP; d += 16) {
                float4 qv[4], sv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) qv[i] = *(const float4*)&q_s[(tg + 8 * i) * DP + (d ^ (tg << 2))];
#pragma unroll
                for (int e = 0; e < 4; ++e) sv[e] = *(const float4*)&S_s[(d + e) * SROW + 4 * cg];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float qe[4] = {qv[i].x, qv[i].y, qv[i].z, qv[i].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        acc[i][0] = fmaf(qe[e], sv[e].x, acc[i][0]);
                        acc[i][1] = fmaf(qe[e], sv[e].y, acc[i][1]);
                        acc[i][2] = fmaf(qe[e], sv[e].z, acc[i][2]);
                        acc[i][3] = fmaf(qe[e], sv[e].w, acc[i][3]);
                    }
                }
            }
            float mine[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float x = acc[i][j];
                    x += __shfl_xor_sync(0xffffffffu, x, 8);
                    x += __shfl_xor_sync(0xffffffffu, x, 16);
                    if (i == kq) mine[j] = x;
                }
            const int t = tg + 8 * kq;
            const float g = g_g[t] * p.q_scale;
            *(float4*)&X0[t * CL + 4 * cg] = make_float4(mine[0] * g, mine[1] * g, mine[2] * g, mine[3] * g);
        }
        // q . n_0 for token tid / 8: each of its 8 threads sums an eighth of the key rows (the same threads write the token's outputs)
        float nq0 = 0.f;
        for (int d = tid & 7; d < DP; d += 8) nq0 = fmaf(q_s[(tid >> 3) * DP + (d ^ (((tid >> 3) & 7) << 2))], S_s[d * SROW + 32], nq0);
        nq0 += __shfl_xor_sync(0xffffffffu, nq0, 1);
        nq0 += __shfl_xor_sync(0xffffffffu, nq0, 2);
        nq0 += __shfl_xor_sync(0xffffffffu, nq0, 4);
        {   // the scores of the thread's token and four keys: weighted, masked
            const int t = tid >> 3, s0 = (tid & 7) * 4;
            const double M = g_M[t];
            const float4 x = *(const float4*)&X1[tid * 4];
            float r[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) r[j] = (s0 + j <= t && s0 + j < len) ? expf((float)(g_a[s0 + j] - M)) * (r[j] * p.q_scale) : 0.f;
            *(float4*)&X1[tid * 4] = make_float4(r[0], r[1], r[2], r[3]);
        }
        __syncthreads();
        fetch_rows(c0 + CL, p.q_col, q_s, true);      // (nothing reads this chunk's q any more)
        fetch_small(c0 + CL, chunk_id + 1);

        // ---- the state after the chunk: a warp has 8 columns (warps 0..3 and 4..7: the two halves of the key rows),
        // a lane the rows lane, lane + 32, ...; the warps of the first columns also renew n
        {
            const int cu0 = 8 * (warp & 3), d0 = (warp >> 2) * (DP / 2) + lane;
            const bool with_n = (warp & 3) == 0;
            const float g_last = g_last_s[0];
            float a[RPL2][8], an[RPL2];
#pragma unroll
            for (int r = 0; r < RPL2; ++r) {
                const float* row = &S_s[(d0 + 32 * r) * SROW];
                const float4 x = *(const float4*)&row[cu0], y = *(const float4*)&row[cu0 + 4];
                a[r][0] = g_last * x.x; a[r][1] = g_last * x.y; a[r][2] = g_last * x.z; a[r][3] = g_last * x.w;
                a[r][4] = g_last * y.x; a[r][5] = g_last * y.y; a[r][6] = g_last * y.z; a[r][7] = g_last * y.w;
                an[r] = g_last * row[32];
            }
            for (int s = 0; s < len; ++s) {
                const float ws = g_w[s];
                const float4 x = *(const float4*)&v_s[s * CL + cu0], y = *(const float4*)&v_s[s * CL + cu0 + 4];
                const float vw[8] = {ws * x.x, ws * x.y, ws * x.z, ws * x.w, ws * y.x, ws * y.y, ws * y.z, ws * y.w};
#pragma unroll
                for (int r = 0; r < RPL2; ++r) {
                    const float kv = k_s[s * DP + d0 + 32 * r];
#pragma unroll
                    for (int j = 0; j < 8; ++j) a[r][j] = fmaf(kv, vw[j], a[r][j]);
                    an[r] = fmaf(kv, ws, an[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < RPL2; ++r) {
                float* row = &S_s[(d0 + 32 * r) * SROW];
                *(float4*)&row[cu0] = make_float4(a[r][0], a[r][1], a[r][2], a[r][3]);
                *(float4*)&row[cu0 + 4] = make_float4(a[r][4], a[r][5], a[r][6], a[r][7]);
                if (with_n) row[32] = an[r];
            }
        }
        __syncthreads();
        fetch_rows(c0 + CL, p.k_col, k_s, false);      // (the state is renewed: nothing reads this chunk's k any more)

        // ---- the outputs: a thread has one token and 4 value columns
        {
            const int t = tid >> 3, cc = (tid & 7) * 4;
            if (t < len) {
                float nq = nq0 * (g_g[t] * p.q_scale);
                float4 o = *(const float4*)&X0[t * CL + cc];
                for (int s = 0; s <= t; ++s) {
                    const float pw = X1[t * CL + s];
                    const float4 vv = *(const float4*)&v_s[s * CL + cc];
                    o.x = fmaf(pw, vv.x, o.x); o.y = fmaf(pw, vv.y, o.y); o.z = fmaf(pw, vv.z, o.z); o.w = fmaf(pw, vv.w, o.w);
                    nq += pw;
                }
                const float den = fmaxf(fabsf(nq), expf(-g_m[t])) + 1e-6f;
                float* dst = p.out + (size_t)(c0 + t) * out_stride + (size_t)head * vdim + cb0 + cc;
                const float r[4] = {o.x / den, o.y / den, o.z / den, o.w / den};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (cb0 + cc + j < vdim) dst[j] = r[j];
            }
        }

        __syncthreads();
    }

    for (int e = tid; e < DP * SROW; e += 256) {
        const int d = e / SROW, c = e - d * SROW;
        if (d >= dim) continue;
        if (c < 32) { if (cb0 + c < vdim) st[(size_t)d * vdim + cb0 + c] = S_s[e]; }
        else if (c == 32) st_n[d] = S_s[e];
    }
    if (tid == 0) st_n[dim] = m_run;
}

template <int RPL2>
int launch_mlstm_chunk(const MlstmParams& p, float* scratch, int scratch_chunks, dim3 grid, cudaStream_t st) {
    const size_t smem_scores = (size_t)2 * CL * (64 * RPL2 + 4) * sizeof(float);
    const size_t smem = (size_t)ChunkSmem<RPL2>::FLOATS * sizeof(float);
    auto scores = mlstm_scores_kernel<RPL2>;
    auto k = mlstm_chunk_kernel<RPL2>;
    if (cudaFuncSetAttribute(scores, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_scores) != cudaSuccess ||
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        return SPITE_LAUNCH_FAILED;
    SPITE_LAUNCH(scores, dim3(scratch_chunks, p.heads), 256, smem_scores, st, p, scratch);
    // (an ordinary launch: as a programmatic dependent of the scores' kernel, whose blocks let dependents start at
    // once, the pair took 925 us for a prompt of 2,048 tokens where it takes 599 us)
    k<<<grid, 256, smem, st>>>(p, (const float*)scratch);
    return spite_launch_status();
}

}  // namespace

static int mlstm_scan_launch(const MlstmParams* p, float* scratch, int scratch_chunks, void* stream) {
    if (!p || !p->proj || !p->out || !p->state || !p->cu_seqlens || !p->slots) return SPITE_BAD_ARG;
    if (p->n_segments < 0 || p->heads < 1 || p->dim < 1 || p->vdim < 1 || !(p->gate_cap > 0.f) || !(p->q_scale == p->q_scale))
        return SPITE_BAD_ARG;
    if (p->q_col < 0 || p->k_col < 0 || p->v_col < 0 || p->i_col < 0 || p->f_col < 0) return SPITE_BAD_ARG;
    const long long need = (long long)p->heads * (2LL * p->dim + p->vdim + 2);
    if (p->stride < need) return SPITE_BAD_ARG;
    if (p->dim > 512) return SPITE_UNSUPPORTED;
    if (p->heads > 65535 || p->n_segments > 65535) return SPITE_UNSUPPORTED;
    if (p->n_segments == 0) return SPITE_OK;
    const long long col_blocks = (p->vdim + COLS_PER_BLOCK - 1) / COLS_PER_BLOCK;
    if (p->head_stride < (long long)p->dim * p->vdim + col_blocks * ((p->dim + 1 + 3) & ~3)) return SPITE_BAD_ARG;
    dim3 grid((p->vdim + COLS_PER_BLOCK - 1) / COLS_PER_BLOCK, p->heads, p->n_segments);
    cudaStream_t st = (cudaStream_t)stream;
    if (p->chunked) {
        if (!scratch || scratch_chunks < 1 || (((uintptr_t)scratch) & 15)) return SPITE_BAD_ARG;
        if (p->dim <= 64) return launch_mlstm_chunk<1>(*p, scratch, scratch_chunks, grid, st);
        if (p->dim <= 128) return launch_mlstm_chunk<2>(*p, scratch, scratch_chunks, grid, st);
        if (p->dim <= 256) return launch_mlstm_chunk<4>(*p, scratch, scratch_chunks, grid, st);
        return launch_mlstm_chunk<8>(*p, scratch, scratch_chunks, grid, st);
    }
    if (p->dim <= 32) SPITE_LAUNCH(mlstm_scan_kernel<1>, grid, 128, 0, st, *p);
    else if (p->dim <= 64) SPITE_LAUNCH(mlstm_scan_kernel<2>, grid, 128, 0, st, *p);
    else if (p->dim <= 128) SPITE_LAUNCH(mlstm_scan_kernel<4>, grid, 128, 0, st, *p);
    else if (p->dim <= 256) SPITE_LAUNCH(mlstm_scan_kernel<8>, grid, 128, 0, st, *p);
    else SPITE_LAUNCH(mlstm_scan_kernel<16>, grid, 128, 0, st, *p);
    return spite_launch_status();
}

SPITE_API int spite_mlstm_scan(const MlstmParams* p, void* stream) {
    if (p && p->chunked) return SPITE_BAD_ARG;            // (32 tokens at a time needs working memory: the entry below)
    return mlstm_scan_launch(p, nullptr, 0, stream);
}

// `scratch`: [scratch_chunks, heads, 1152] floats of working memory, 16-byte aligned; scratch_chunks >= the step's
// chunks, the sum over the segments of ceil(tokens / 32).  Takes p->chunked as it is given.
SPITE_API int spite_mlstm_scan_chunked(const MlstmParams* p, float* scratch, int scratch_chunks, void* stream) {
    return mlstm_scan_launch(p, scratch, scratch_chunks, stream);
}
