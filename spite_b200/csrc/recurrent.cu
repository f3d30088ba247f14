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

}  // namespace

SPITE_API int spite_mlstm_scan(const MlstmParams* p, void* stream) {
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
    if (p->dim <= 32) SPITE_LAUNCH(mlstm_scan_kernel<1>, grid, 128, 0, st, *p);
    else if (p->dim <= 64) SPITE_LAUNCH(mlstm_scan_kernel<2>, grid, 128, 0, st, *p);
    else if (p->dim <= 128) SPITE_LAUNCH(mlstm_scan_kernel<4>, grid, 128, 0, st, *p);
    else if (p->dim <= 256) SPITE_LAUNCH(mlstm_scan_kernel<8>, grid, 128, 0, st, *p);
    else SPITE_LAUNCH(mlstm_scan_kernel<16>, grid, 128, 0, st, *p);
    return spite_launch_status();
}
