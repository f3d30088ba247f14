// The gated delta rule: a mixer whose state is a matrix per head, S [dim, vdim], carried from token to token in
// float32 in the request's state slot:
//     g_t    = exp(-exp(A_h) * softplus(a_t + dt_h))         a_t, b_t: two columns of the projection per head
//     beta_t = sigmoid(b_t)
//     k_t <- k_t / sqrt(|k_t|^2 + unit_eps),   q_t <- q_t / sqrt(|q_t|^2 + unit_eps) * q_scale
//     S <- g_t S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t
// A state of zeros is the start of a sequence.  `heads` value heads share `kv_heads` query/key heads (head h reads
// q/k head h / (heads / kv_heads)).  Everything is float32: the inputs are float32 (the projection's sums after the
// short convolution), and nothing in the recurrence is rounded below that.
//
// Token by token.  A block owns 32 value columns of one (segment, head); a warp 8 of them; a lane one column and
// every fourth key row (lane / 8, + 4, ...), RP rows in registers.  The sums over the key rows are a thread's own
// RP terms and two shuffles.  One pass over the state per token gives S^T k, S^T q and k . q together
// (o_t = g S_old^T q + u (k . q) is the read-out after the write, regrouped), a second one renews the state.  The
// tokens' inputs come through a ring of shared-memory stages filled by asynchronous copies several tokens ahead, so
// the walk waits for arithmetic, not for memory.
#include "common.cuh"

struct DeltaParams {
    const float* x;             // [tokens, stride]
    long long stride;
    int q_col, k_col, v_col, b_col, a_col;   // first columns of q, k [kv_heads * dim], v [heads * vdim], b, a [heads]
    const float* a_log;         // [heads]
    const float* dt_bias;       // [heads]
    float* out;                 // [tokens, heads * vdim]
    float* state;               // state + slot * slot_stride + head * dim * vdim: S row-major [dim, vdim]
    long long slot_stride;
    const int* cu_seqlens;      // [segments + 1]
    const int* slots;           // [segments]
    int n_segments, heads, kv_heads, dim, vdim;
    float q_scale, unit_eps;
};

namespace {

constexpr int COLS_PER_BLOCK = 32;
constexpr int NBUF = 8;                                        // tokens in flight

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ float sum4(float v) {               // over the four lanes that share a column
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    return v;
}

// grid (ceil(vdim / 32), heads, segments), block 128, shared memory NBUF * stage floats
template <int RP>
__global__ void __launch_bounds__(128) delta_scan_kernel(const DeltaParams p) {
    extern __shared__ float ring[];
    pdl_wait();
    pdl_launch_dependents();
    const int seg = blockIdx.z, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 3, cc = lane & 7;
    const int dim = p.dim, vdim = p.vdim;
    const int c0 = blockIdx.x * COLS_PER_BLOCK;
    const int j = c0 + warp * 8 + cc;                          // this thread's value column
    const bool col_ok = j < vdim;
    const int t0 = p.cu_seqlens[seg], t1 = p.cu_seqlens[seg + 1];
    if (t0 >= t1) return;
    const int slot = p.slots[seg];
    // A captured step pads its rows with copies of its first row: a copy would renew the first row's state a second
    // time.  It leaves zeros instead (its results are never read).
    if (seg > 0 && slot == p.slots[0]) {
        if (r == 0 && col_ok)
            for (int t = t0; t < t1; ++t) p.out[(size_t)t * p.heads * vdim + (size_t)head * vdim + j] = 0.f;
        return;
    }
    const int kvh = head / (p.heads / p.kv_heads);
    float* st = p.state + (size_t)slot * p.slot_stride + (size_t)head * dim * vdim;
    float S[RP];
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int row = r + 4 * i;
        S[i] = (row < dim && col_ok) ? st[(size_t)row * vdim + j] : 0.f;
    }
    const float decay_rate = expf(p.a_log[head]), dt = p.dt_bias[head];

    // a stage: k [dim], q [dim], v [32], b, a
    const int stage = 2 * dim + COLS_PER_BLOCK + 2;
    auto issue = [&](int t) {
        if (t < t1) {
            float* dst = ring + (size_t)((t - t0) % NBUF) * stage;
            const float* row = p.x + (size_t)t * p.stride;
            for (int e = threadIdx.x; e < stage; e += blockDim.x) {
                const float* src;
                if (e < dim) src = row + p.k_col + kvh * dim + e;
                else if (e < 2 * dim) src = row + p.q_col + kvh * dim + (e - dim);
                else if (e < 2 * dim + COLS_PER_BLOCK) {
                    const int c = c0 + e - 2 * dim;
                    src = row + p.v_col + head * vdim + (c < vdim ? c : vdim - 1);
                } else src = row + (e == 2 * dim + COLS_PER_BLOCK ? p.b_col : p.a_col) + head;
                cp_async4(dst + e, src);
            }
        }
        cp_commit();
    };
#pragma unroll 1
    for (int s = 0; s < NBUF - 1; ++s) issue(t0 + s);

#pragma unroll 1
    for (int t = t0; t < t1; ++t) {
        cp_wait<NBUF - 2>();
        __syncthreads();                                       // token t has landed, and every thread is done with token t - 1
        issue(t + NBUF - 1);                                   // (into the stage that token t - 1 had)
        const float* in = ring + (size_t)((t - t0) % NBUF) * stage;
        const float* kk = in, *qq = in + dim;
        float a = 0.f, b = 0.f, kq = 0.f, k2 = 0.f, q2 = 0.f;
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            const int row = r + 4 * i;
            const float kv = row < dim ? kk[row] : 0.f, qv = row < dim ? qq[row] : 0.f;
            a = fmaf(S[i], kv, a);
            b = fmaf(S[i], qv, b);
            kq = fmaf(kv, qv, kq);
            k2 = fmaf(kv, kv, k2);
            q2 = fmaf(qv, qv, q2);
        }
        a = sum4(a); b = sum4(b); kq = sum4(kq); k2 = sum4(k2); q2 = sum4(q2);
        const float rk = 1.0f / sqrtf(k2 + p.unit_eps), rq = p.q_scale / sqrtf(q2 + p.unit_eps);
        const float vj = in[2 * dim + warp * 8 + cc];
        const float zb = in[2 * dim + COLS_PER_BLOCK], za = in[2 * dim + COLS_PER_BLOCK + 1] + dt;
        const float beta = 1.0f / (1.0f + expf(-zb));
        const float softplus = fmaxf(za, 0.f) + log1pf(expf(-fabsf(za)));
        const float g = expf(-decay_rate * softplus);
        const float u = beta * (vj - g * (a * rk));
        const float o = g * (b * rq) + u * (kq * rk * rq);
        const float ku = u * rk;
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            const int row = r + 4 * i;
            const float kv = row < dim ? kk[row] : 0.f;
            S[i] = fmaf(kv, ku, g * S[i]);
        }
        if (r == 0 && col_ok) p.out[(size_t)t * p.heads * vdim + (size_t)head * vdim + j] = o;
    }
    cp_wait<0>();
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int row = r + 4 * i;
        if (row < dim && col_ok) st[(size_t)row * vdim + j] = S[i];
    }
}

}  // namespace

SPITE_API int spite_delta_scan(const DeltaParams* p, void* stream) {
    if (!p || !p->x || !p->a_log || !p->dt_bias || !p->out || !p->state || !p->cu_seqlens || !p->slots) return SPITE_BAD_ARG;
    if (p->n_segments < 0 || p->heads < 1 || p->kv_heads < 1 || p->heads % p->kv_heads || p->dim < 1 || p->vdim < 1) return SPITE_BAD_ARG;
    if (p->slot_stride < (long long)p->heads * p->dim * p->vdim || !(p->unit_eps >= 0.f)) return SPITE_BAD_ARG;
    const long long need = (long long)p->kv_heads * p->dim;
    if (p->q_col < 0 || p->k_col < 0 || p->v_col < 0 || p->b_col < 0 || p->a_col < 0) return SPITE_BAD_ARG;
    if (p->stride < p->q_col + need || p->stride < p->k_col + need || p->stride < p->v_col + (long long)p->heads * p->vdim ||
        p->stride < p->b_col + p->heads || p->stride < p->a_col + p->heads) return SPITE_BAD_ARG;
    if (p->dim > 512 || p->heads > 65535 || p->n_segments > 65535) return SPITE_UNSUPPORTED;
    if (p->n_segments == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((p->vdim + COLS_PER_BLOCK - 1) / COLS_PER_BLOCK, p->heads, p->n_segments);
    const size_t smem = (size_t)NBUF * (2 * p->dim + COLS_PER_BLOCK + 2) * sizeof(float);
    const int rp = (p->dim + 3) / 4;
    if (rp <= 16) SPITE_LAUNCH(delta_scan_kernel<16>, grid, 128, smem, st, *p);
    else if (rp <= 32) SPITE_LAUNCH(delta_scan_kernel<32>, grid, 128, smem, st, *p);
    else if (rp <= 64) SPITE_LAUNCH(delta_scan_kernel<64>, grid, 128, smem, st, *p);
    else SPITE_LAUNCH(delta_scan_kernel<128>, grid, 128, smem, st, *p);
    return spite_launch_status();
}
