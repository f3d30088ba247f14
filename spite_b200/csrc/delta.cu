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
// Token by token.  A block owns 32, 16 or 8 value columns of one (segment, head); a warp a quarter of them; a lane one
// column and a contiguous share of the key rows, RP rows in registers.  The sums over the key rows are a thread's own
// RP terms and two to four shuffles.  One pass over the state per token gives S^T k, S^T q and k . q together
// (o_t = g S_old^T q + u (k . q) is the read-out after the write, regrouped), a second one renews the state.  What
// does not depend on the state (the unit vectors' factors, beta, the decay) comes from a kernel that runs before.  The
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
    float* gates;               // scratch [tokens, 2 * kv_heads + 2 * heads]: per q/k head the factors that make k and q unit
                                // vectors (q's with q_scale), per head beta and the decay; written before the walk
    int n_tokens;
};

namespace {

constexpr int NBUF = 8;                                        // tokens in flight

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// grid (ceil(vdim / (4 CW)), heads, segments), block 128, shared memory NBUF * stage floats.
// What a token brings besides q, k, v does not depend on the state: one small kernel computes it for all tokens of the
// step, so that the walk's chain per token is multiply-adds and shuffles alone.  grid tokens, block 128: warp w takes
// the q/k heads w, w + 4, ... (sums over dim) and the heads w, w + 4, ... (beta, decay).
__global__ void __launch_bounds__(128) delta_gates_kernel(const DeltaParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = p.x + (size_t)t * p.stride;
    float* out = p.gates + (size_t)t * (2 * p.kv_heads + 2 * p.heads);
    for (int g = warp; g < p.kv_heads; g += 4) {
        float k2 = 0.f, q2 = 0.f;
        for (int i = lane; i < p.dim; i += 32) {
            const float kv = row[p.k_col + g * p.dim + i], qv = row[p.q_col + g * p.dim + i];
            k2 = fmaf(kv, kv, k2); q2 = fmaf(qv, qv, q2);
        }
        k2 = warp_sum(k2); q2 = warp_sum(q2);
        if (lane == 0) {
            out[g] = 1.0f / sqrtf(k2 + p.unit_eps);
            out[p.kv_heads + g] = p.q_scale / sqrtf(q2 + p.unit_eps);
        }
    }
    for (int h = threadIdx.x; h < p.heads; h += blockDim.x) {
        const float zb = row[p.b_col + h], za = row[p.a_col + h] + p.dt_bias[h];
        const float softplus = fmaxf(za, 0.f) + log1pf(expf(-fabsf(za)));
        out[2 * p.kv_heads + h] = 1.0f / (1.0f + expf(-zb));
        out[2 * p.kv_heads + p.heads + h] = expf(-expf(p.a_log[h]) * softplus);
    }
}

// CW: value columns a warp owns (8, 4 or 2); its 32 / CW lanes per column split the key rows, RP contiguous rows a lane
// (zeros beyond dim).  Fewer columns a warp means more and smaller blocks and fewer instructions a token and warp, which
// is what a long segment wants (the walk is bound by what one warp can issue); whole sectors of the state per row
// (CW = 8) is what a decode step wants.
template <int RP, int CW>
__global__ void __launch_bounds__(128) delta_scan_kernel(const DeltaParams p) {
    extern __shared__ __align__(16) float ring[];
    pdl_wait();
    constexpr int RS = 32 / CW, COLS = 4 * CW, DPAD = RS * RP;
    constexpr int STAGE = 2 * DPAD + ((COLS + 4 + 3) & ~3);    // k [DPAD], q [DPAD], v [COLS], rk, rq, beta, decay
    const int seg = blockIdx.z, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane / CW, cc = lane % CW;
    const int dim = p.dim, vdim = p.vdim;
    const int c0 = blockIdx.x * COLS;
    const int j = c0 + warp * CW + cc;                         // this thread's value column
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
        const int row = r * RP + i;
        S[i] = (row < dim && col_ok) ? st[(size_t)row * vdim + j] : 0.f;
    }
    const int n_gates = 2 * p.kv_heads + 2 * p.heads;
    // the rows of k and q beyond dim stay zero in every stage
    for (int e = threadIdx.x; e < NBUF * 2 * (DPAD - dim); e += blockDim.x) {
        const int s = e / (2 * (DPAD - dim)), i = e % (2 * (DPAD - dim));
        ring[(size_t)s * STAGE + (i < DPAD - dim ? dim + i : DPAD + dim + i - (DPAD - dim))] = 0.f;
    }

    auto issue = [&](int t) {
        if (t < t1) {
            float* dst = ring + (size_t)((t - t0) % NBUF) * STAGE;
            const float* row = p.x + (size_t)t * p.stride;
            for (int e = threadIdx.x; e < dim; e += blockDim.x) {
                cp_async4(dst + e, row + p.k_col + kvh * dim + e);
                cp_async4(dst + DPAD + e, row + p.q_col + kvh * dim + e);
            }
            if (threadIdx.x < COLS) {
                const int c = c0 + threadIdx.x;
                cp_async4(dst + 2 * DPAD + threadIdx.x, row + p.v_col + head * vdim + (c < vdim ? c : vdim - 1));
            } else if (threadIdx.x < COLS + 4) {
                const int w = threadIdx.x - COLS;              // rk, rq of the q/k head; beta, decay of the head
                const float* gt = p.gates + (size_t)t * n_gates;
                cp_async4(dst + 2 * DPAD + threadIdx.x, gt + (w == 0 ? kvh : w == 1 ? p.kv_heads + kvh : w == 2 ? 2 * p.kv_heads + head
                                                                                                            : 2 * p.kv_heads + p.heads + head));
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
        const float* in = ring + (size_t)((t - t0) % NBUF) * STAGE;
        const float4* kk = (const float4*)(in + r * RP);
        const float4* qq = (const float4*)(in + DPAD + r * RP);
        // (four partial sums each: a sum's multiply-adds would otherwise wait for one another)
        float a4[4] = {0.f, 0.f, 0.f, 0.f}, b4[4] = {0.f, 0.f, 0.f, 0.f}, kq4[4] = {0.f, 0.f, 0.f, 0.f};
        float kr[RP];
#pragma unroll
        for (int i = 0; i < RP / 4; ++i) {
            const float4 kv = kk[i], qv = qq[i];
            kr[4 * i] = kv.x; kr[4 * i + 1] = kv.y; kr[4 * i + 2] = kv.z; kr[4 * i + 3] = kv.w;
            a4[0] = fmaf(S[4 * i], kv.x, a4[0]); a4[1] = fmaf(S[4 * i + 1], kv.y, a4[1]);
            a4[2] = fmaf(S[4 * i + 2], kv.z, a4[2]); a4[3] = fmaf(S[4 * i + 3], kv.w, a4[3]);
            b4[0] = fmaf(S[4 * i], qv.x, b4[0]); b4[1] = fmaf(S[4 * i + 1], qv.y, b4[1]);
            b4[2] = fmaf(S[4 * i + 2], qv.z, b4[2]); b4[3] = fmaf(S[4 * i + 3], qv.w, b4[3]);
            kq4[0] = fmaf(kv.x, qv.x, kq4[0]); kq4[1] = fmaf(kv.y, qv.y, kq4[1]);
            kq4[2] = fmaf(kv.z, qv.z, kq4[2]); kq4[3] = fmaf(kv.w, qv.w, kq4[3]);
        }
        float a = (a4[0] + a4[1]) + (a4[2] + a4[3]), b = (b4[0] + b4[1]) + (b4[2] + b4[3]), kq = (kq4[0] + kq4[1]) + (kq4[2] + kq4[3]);
#pragma unroll
        for (int o = CW; o < 32; o <<= 1) {                    // over the lanes that share a column
            a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o);
            kq += __shfl_xor_sync(0xffffffffu, kq, o);
        }
        const float vj = in[2 * DPAD + warp * CW + cc];
        const float rk = in[2 * DPAD + COLS], rq = in[2 * DPAD + COLS + 1], beta = in[2 * DPAD + COLS + 2], g = in[2 * DPAD + COLS + 3];
        const float u = beta * (vj - g * (a * rk));
        const float o = g * (b * rq) + u * (kq * rk * rq);
        const float ku = u * rk;
#pragma unroll
        for (int i = 0; i < RP; ++i) S[i] = fmaf(kr[i], ku, g * S[i]);
        if (r == 0 && col_ok) p.out[(size_t)t * p.heads * vdim + (size_t)head * vdim + j] = o;
    }
    cp_wait<0>();
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int row = r * RP + i;
        if (row < dim && col_ok) st[(size_t)row * vdim + j] = S[i];
    }
    pdl_launch_dependents();                                   // (late: the next kernel's blocks would only sit and wait)
}

template <int RP, int CW>
static int launch_scan(const DeltaParams& p, cudaStream_t st) {
    constexpr int RS = 32 / CW, COLS = 4 * CW, DPAD = RS * RP;
    constexpr int STAGE = 2 * DPAD + ((COLS + 4 + 3) & ~3);
    dim3 grid((p.vdim + COLS - 1) / COLS, p.heads, p.n_segments);
    // Launched in the ordinary way, not as a programmatic dependent: started early, the walk's few blocks take whatever
    // multiprocessors the kernel before frees first, several to one, and stay there for the whole walk (2,048 tokens
    // of 16 heads of 128 x 128: 1.40 to 1.78 ms against 1.14 ms).
    delta_scan_kernel<RP, CW><<<grid, 128, (size_t)NBUF * STAGE * sizeof(float), st>>>(p);
    return spite_launch_status();
}

}  // namespace

// `split_rows`: more lanes a value column and fewer columns a block (for steps with long segments); without it a warp
// owns 8 columns, whole sectors of every row of the state (for decode steps).  The two differ in the order of sums.
SPITE_API int spite_delta_scan(const DeltaParams* p, int split_rows, void* stream) {
    if (!p || !p->x || !p->a_log || !p->dt_bias || !p->out || !p->state || !p->cu_seqlens || !p->slots || !p->gates) return SPITE_BAD_ARG;
    if (p->n_tokens < 0) return SPITE_BAD_ARG;
    if (p->n_segments < 0 || p->heads < 1 || p->kv_heads < 1 || p->heads % p->kv_heads || p->dim < 1 || p->vdim < 1) return SPITE_BAD_ARG;
    if (p->slot_stride < (long long)p->heads * p->dim * p->vdim || !(p->unit_eps >= 0.f)) return SPITE_BAD_ARG;
    const long long need = (long long)p->kv_heads * p->dim;
    if (p->q_col < 0 || p->k_col < 0 || p->v_col < 0 || p->b_col < 0 || p->a_col < 0) return SPITE_BAD_ARG;
    if (p->stride < p->q_col + need || p->stride < p->k_col + need || p->stride < p->v_col + (long long)p->heads * p->vdim ||
        p->stride < p->b_col + p->heads || p->stride < p->a_col + p->heads) return SPITE_BAD_ARG;
    if (p->dim > 512 || p->heads > 65535 || p->n_segments > 65535) return SPITE_UNSUPPORTED;
    if (p->n_segments == 0 || p->n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    SPITE_LAUNCH(delta_gates_kernel, p->n_tokens, 128, 0, st, *p);
    if (cudaGetLastError() != cudaSuccess) return SPITE_LAUNCH_FAILED;
    const int dim = p->dim;
    if (split_rows) {
        if (dim <= 32) return launch_scan<4, 4>(*p, st);
        if (dim <= 64) return launch_scan<8, 4>(*p, st);
        if (dim <= 128) return launch_scan<8, 2>(*p, st);
        if (dim <= 256) return launch_scan<16, 2>(*p, st);
        return launch_scan<32, 2>(*p, st);
    }
    if (dim <= 32) return launch_scan<8, 8>(*p, st);
    if (dim <= 64) return launch_scan<16, 8>(*p, st);
    if (dim <= 128) return launch_scan<32, 8>(*p, st);
    if (dim <= 256) return launch_scan<64, 8>(*p, st);
    return launch_scan<128, 8>(*p, st);
}
