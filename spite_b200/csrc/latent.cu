// Attention through latents: what happens between the products.
//
//  * latent_prepare: one row of the first product's float32 output holds a token's query latent, its
//    key/value latent, the key part that all heads share and the gate columns.  Both latents are RMS-normed
//    with a gain (float32 sums and scaling), the shared key part is rotated (neighbouring pairs or halves, angle
//    position * inv_freq[i], cos and sin times an amplitude), and the cache row of the token's position
//    becomes [normed key/value latent ; rotated shared part ; zeros].  The gates become sigmoid(column).
//  * latent_queries: the rotating tail of every query head is rotated the same way into the row that the
//    attention kernels read ([kv_rank elements left for the product with the heads' key matrices ; rotated
//    tail ; zeros]), the (token, head) rows are listed head by head for the products per head, and the unrotated
//    parts are laid out in that order, so that the product that follows reads its rows in place.
//
// One block a token; float32 arithmetic whatever the element type.
#include "attention.cuh"

struct LatentPrepareParams {
    const float* down;          // [tokens, down_stride]: query latent, key/value latent, shared key part, gate columns
    long long down_stride;
    void* cq_out;               // [tokens, q_rank] normed query latent (activation type)
    const float* q_gain;        // [q_rank]
    const float* kv_gain;       // [kv_rank]
    const float* inv_freq;      // [rot_dim / 2]
    float rot_amplitude;
    float eps;
    int q_rank, kv_rank, rot_dim;
    int num_gates;
    float* gates_out;           // [tokens, num_gates] or null
    int write_cache;
    int pairing;                // SPITE_PAIR_*: which two elements of the shared key part pair i is
};

struct LatentQueryParams {
    const void* q;              // [tokens, num_heads * (head_dim + rot_dim)]
    void* q_out;                // [tokens, num_heads * row]
    const float* inv_freq;      // [rot_dim / 2]
    float rot_amplitude;
    int num_heads, head_dim, rot_dim, kv_rank, row;
    const int* positions;       // [tokens]
    int n_tokens;
    int* rows_out;              // [num_heads * tokens]: rows_out[h * tokens + t] = t * num_heads + h
    int* offsets_out;           // [num_heads + 1]: offsets_out[h] = h * tokens
    void* q_sorted_out;         // [num_heads * tokens, head_dim] or null: the unrotated parts head by head (row h * tokens + t),
                                // the order in which the product with the heads' key matrices takes its rows
    int pairing;                // SPITE_PAIR_*: which two elements of a head's rotating tail pair i is
};

namespace {

// Two sums over a block of 256 threads at once; every thread receives both.  The order of the additions is a
// function of the block size only.
__device__ __forceinline__ void block_sum2(float& a, float& b, float (*scratch)[33]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    a = warp_sum(a); b = warp_sum(b);
    if (lane == 0) { scratch[0][warp] = a; scratch[1][warp] = b; }
    __syncthreads();
    if (warp == 0) {
        float x = lane < nwarps ? scratch[0][lane] : 0.f, y = lane < nwarps ? scratch[1][lane] : 0.f;
        x = warp_sum(x); y = warp_sum(y);
        if (lane == 0) { scratch[0][32] = x; scratch[1][32] = y; }
    }
    __syncthreads();
    a = scratch[0][32]; b = scratch[1][32];
}

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *(float4*)p = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2*)p = make_uint2(*(const unsigned*)&lo, *(const unsigned*)&hi);
}

// grid tokens, block 128 or 256.  VEC: both ranks and the row stride are multiples of four, q_rank <= 16 * threads and
// kv_rank <= 4 * threads: a thread keeps its elements of both latents in registers between the sums and the scaling
// (16-byte loads, one round of block-wide sums for both norms), and everything else the block reads (its page, its
// gate column, its pair of the shared key part) is asked for before the sums; otherwise the row is walked element by
// element, twice.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const LatentPrepareParams p, const StepTokens b,
                                                             const PagedCache c) {
    __shared__ float scratch[2][33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float* in = p.down + (size_t)t * p.down_stride;
    const float* kv = in + p.q_rank;
    const int pos = b.positions[t];
    constexpr int QV = 4;                                     // 16-byte groups of the query latent a thread holds
    float4 qv[QV], kvv = make_float4(0.f, 0.f, 0.f, 0.f);
    float sq = 0.f, sk = 0.f;
    // asked for before the sums, used after them (thread i: gate column i, pair i of the shared key part)
    int page = -1;
    if (p.write_cache) page = b.block_table[(size_t)b.seg_of_token[t] * b.table_width + pos / c.page_size];
    const float* kr = kv + p.kv_rank;
    const int first_gate = p.q_rank + p.kv_rank + p.rot_dim;
    float gate_in = 0.f, kr0 = 0.f, kr1 = 0.f;
    if (p.gates_out && (int)threadIdx.x < p.num_gates) gate_in = in[first_gate + threadIdx.x];
    const int half_rot = p.rot_dim / 2;
    const bool halves = p.pairing == SPITE_PAIR_HALVES;       // pair i: elements (i, i + rot_dim / 2) instead of (2i, 2i + 1)
    if ((int)threadIdx.x < half_rot) {
        kr0 = kr[halves ? threadIdx.x : 2 * threadIdx.x];
        kr1 = kr[halves ? threadIdx.x + half_rot : 2 * threadIdx.x + 1];
    }
    if (VEC) {
#pragma unroll
        for (int r = 0; r < QV; ++r) {
            const int i = 4 * (threadIdx.x + blockDim.x * r);
            qv[r] = i < p.q_rank ? *(const float4*)(in + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            sq += qv[r].x * qv[r].x + qv[r].y * qv[r].y + qv[r].z * qv[r].z + qv[r].w * qv[r].w;
        }
        if (4 * threadIdx.x < p.kv_rank) kvv = *(const float4*)(kv + 4 * threadIdx.x);
        sk = kvv.x * kvv.x + kvv.y * kvv.y + kvv.z * kvv.z + kvv.w * kvv.w;
    } else {
        for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) { const float v = in[i]; sq = fmaf(v, v, sq); }
        for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) { const float v = kv[i]; sk = fmaf(v, v, sk); }
    }
    block_sum2(sq, sk, scratch);

    // query latent
    const float mul_q = 1.0f / sqrtf(sq / (float)p.q_rank + p.eps);
    T* cq = (T*)p.cq_out + (size_t)t * p.q_rank;
    if (VEC) {
#pragma unroll
        for (int r = 0; r < QV; ++r) {
            const int i = 4 * (threadIdx.x + blockDim.x * r);
            if (i < p.q_rank) {
                const float4 g = *(const float4*)(p.q_gain + i);
                store4(cq + i, qv[r].x * mul_q * g.x, qv[r].y * mul_q * g.y, qv[r].z * mul_q * g.z, qv[r].w * mul_q * g.w);
            }
        }
    } else {
        for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) cq[i] = from_f32<T>(in[i] * mul_q * p.q_gain[i]);
    }

    // gates
    if (p.gates_out)
        for (int h = threadIdx.x; h < p.num_gates; h += blockDim.x)
            p.gates_out[(size_t)t * p.num_gates + h] = 1.0f / (1.0f + expf(-(h < (int)blockDim.x ? gate_in : in[first_gate + h])));

    // key/value latent and the shared key part: the cache row of this position
    if (!p.write_cache) return;
    if (page < 0 || page >= c.n_pages) return;               // the host never lets this happen
    const float mul_k = 1.0f / sqrtf(sk / (float)p.kv_rank + p.eps);
    T* row = (T*)c.kv + ((size_t)page * c.page_size + pos % c.page_size) * c.head_dim;
    if (VEC) {
        const int i = 4 * threadIdx.x;
        if (i < p.kv_rank) {
            row[i] = from_f32<T>(kvv.x * mul_k * p.kv_gain[i]); row[i + 1] = from_f32<T>(kvv.y * mul_k * p.kv_gain[i + 1]);
            row[i + 2] = from_f32<T>(kvv.z * mul_k * p.kv_gain[i + 2]); row[i + 3] = from_f32<T>(kvv.w * mul_k * p.kv_gain[i + 3]);
        }
    } else {
        for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) row[i] = from_f32<T>(kv[i] * mul_k * p.kv_gain[i]);
    }
    for (int i = threadIdx.x; 2 * i < p.rot_dim; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * p.inv_freq[i], &sn, &cs);
        sn *= p.rot_amplitude; cs *= p.rot_amplitude;
        const int e0 = halves ? i : 2 * i, e1 = halves ? i + half_rot : 2 * i + 1;
        const float a = i < (int)blockDim.x ? kr0 : kr[e0], bb = i < (int)blockDim.x ? kr1 : kr[e1];
        row[p.kv_rank + e0] = from_f32<T>(a * cs - bb * sn);
        row[p.kv_rank + e1] = from_f32<T>(bb * cs + a * sn);
    }
    for (int i = p.kv_rank + p.rot_dim + threadIdx.x; i < c.head_dim; i += blockDim.x) row[i] = from_f32<T>(0.f);
}

__device__ __forceinline__ void load_pair(const float* p, float& a, float& b) { const float2 v = *(const float2*)p; a = v.x; b = v.y; }
__device__ __forceinline__ void load_pair(const __nv_bfloat16* p, float& a, float& b) {
    const __nv_bfloat162 v = *(const __nv_bfloat162*)p;
    a = __low2float(v); b = __high2float(v);
}
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *(float2*)p = make_float2(a, b); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) { *(__nv_bfloat162*)p = __floats2bfloat162_rn(a, b); }
__device__ __forceinline__ void copy4(float* dst, const float* src) { *(float4*)dst = *(const float4*)src; }
__device__ __forceinline__ void copy4(__nv_bfloat16* dst, const __nv_bfloat16* src) { *(uint2*)dst = *(const uint2*)src; }

// grid tokens, block 128.  WIDE: head_dim and rot_dim are multiples of four and kv_rank and the row size are even, so a
// rotating pair moves as one word and the unrotated parts four elements at a time.
template <typename T, bool WIDE>
__global__ void __launch_bounds__(128) latent_queries_kernel(const LatentQueryParams p) {
    extern __shared__ float cs_sn[];                         // [rot_dim / 2] cos, then as many sin
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int half = p.rot_dim / 2;
    const int pos = p.positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * p.inv_freq[i], &sn, &cs);
        cs_sn[i] = cs * p.rot_amplitude;
        cs_sn[half + i] = sn * p.rot_amplitude;
    }
    __syncthreads();
    const int qh = p.head_dim + p.rot_dim;
    const T* q = (const T*)p.q + (size_t)t * p.num_heads * qh;
    T* out = (T*)p.q_out + (size_t)t * p.num_heads * p.row;
    for (int e = threadIdx.x; e < p.num_heads * half; e += blockDim.x) {
        const int h = e / half, i = e % half;
        const float cs = cs_sn[i], sn = cs_sn[half + i];
        if (p.pairing == SPITE_PAIR_HALVES) {                  // pair i: elements (i, i + rot_dim / 2)
            const T* src = q + h * qh + p.head_dim;
            T* dst = out + h * p.row + p.kv_rank;
            const float a = to_f32(src[i]), bb = to_f32(src[i + half]);
            dst[i] = from_f32<T>(a * cs - bb * sn);
            dst[i + half] = from_f32<T>(bb * cs + a * sn);
            continue;
        }
        const T* src = q + h * qh + p.head_dim + 2 * i;
        T* dst = out + h * p.row + p.kv_rank + 2 * i;
        float a, bb;
        if (WIDE) load_pair(src, a, bb);
        else { a = to_f32(src[0]); bb = to_f32(src[1]); }
        if (WIDE) store_pair(dst, a * cs - bb * sn, bb * cs + a * sn);
        else { dst[0] = from_f32<T>(a * cs - bb * sn); dst[1] = from_f32<T>(bb * cs + a * sn); }
    }
    if (p.q_sorted_out) {
        T* sorted = (T*)p.q_sorted_out;
        if (WIDE) {
            const int quarter = p.head_dim / 4;
            for (int e = threadIdx.x; e < p.num_heads * quarter; e += blockDim.x) {
                const int h = e / quarter, i = 4 * (e % quarter);
                copy4(sorted + ((size_t)h * p.n_tokens + t) * p.head_dim + i, q + h * qh + i);
            }
        } else {
            for (int e = threadIdx.x; e < p.num_heads * p.head_dim; e += blockDim.x) {
                const int h = e / p.head_dim, i = e % p.head_dim;
                sorted[((size_t)h * p.n_tokens + t) * p.head_dim + i] = q[h * qh + i];
            }
        }
    }
    const int pad = p.row - p.kv_rank - p.rot_dim;
    for (int e = threadIdx.x; e < p.num_heads * pad; e += blockDim.x)
        out[(e / pad) * p.row + p.kv_rank + p.rot_dim + e % pad] = from_f32<T>(0.f);
    for (int h = threadIdx.x; h < p.num_heads; h += blockDim.x) p.rows_out[(size_t)h * p.n_tokens + t] = t * p.num_heads + h;
    if (t == 0)
        for (int h = threadIdx.x; h <= p.num_heads; h += blockDim.x) p.offsets_out[h] = h * p.n_tokens;
}

}  // namespace

SPITE_API int spite_latent_prepare(int dtype, const LatentPrepareParams* p, const StepTokens* b, const PagedCache* c,
                                   void* stream) {
    if (!p || !b || !c || !p->down || !p->cq_out || !p->q_gain || !p->kv_gain || !p->inv_freq) return SPITE_BAD_ARG;
    if (!b->positions || !b->seg_of_token || !b->block_table || !c->kv) return SPITE_BAD_ARG;
    if (b->n_tokens < 0 || b->table_width < 1 || c->n_pages < 1 || c->page_size < 1 || c->num_kv_heads != 1) return SPITE_BAD_ARG;
    if (p->q_rank < 1 || p->kv_rank < 1 || p->rot_dim < 2 || p->rot_dim % 2 || p->num_gates < 0) return SPITE_BAD_ARG;
    if (p->pairing != SPITE_PAIR_NEIGHBOURS && p->pairing != SPITE_PAIR_HALVES) return SPITE_BAD_ARG;
    if (p->gates_out ? p->num_gates < 1 : false) return SPITE_BAD_ARG;
    if (p->down_stride < (long long)p->q_rank + p->kv_rank + p->rot_dim + (p->gates_out ? p->num_gates : 0)) return SPITE_BAD_ARG;
    if (c->head_dim < p->kv_rank + p->rot_dim) return SPITE_BAD_ARG;
    if (b->n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    // 128 threads hold a query latent of up to 2,048 elements: two loads of a thread on their way instead of one, and
    // twice the blocks a multiprocessor
    const int threads = (p->q_rank <= 2048 && p->kv_rank <= 512) ? 128 : 256;
    const bool vec = p->q_rank % 4 == 0 && p->kv_rank % 4 == 0 && p->down_stride % 4 == 0 && p->q_rank <= 16 * threads &&
                     p->kv_rank <= 4 * threads && (((uintptr_t)p->down | (uintptr_t)p->cq_out | (uintptr_t)p->q_gain) & 15) == 0;
    if (dtype == SPITE_DT_F32) {
        if (vec) SPITE_LAUNCH((latent_prepare_kernel<float, true>), b->n_tokens, threads, 0, st, *p, *b, *c);
        else SPITE_LAUNCH((latent_prepare_kernel<float, false>), b->n_tokens, threads, 0, st, *p, *b, *c);
    } else if (dtype == SPITE_DT_BF16) {
        if (vec) SPITE_LAUNCH((latent_prepare_kernel<__nv_bfloat16, true>), b->n_tokens, threads, 0, st, *p, *b, *c);
        else SPITE_LAUNCH((latent_prepare_kernel<__nv_bfloat16, false>), b->n_tokens, threads, 0, st, *p, *b, *c);
    } else return SPITE_BAD_ARG;
    return spite_launch_status();
}

SPITE_API int spite_latent_queries(int dtype, const LatentQueryParams* p, void* stream) {
    if (!p || !p->q || !p->q_out || !p->inv_freq || !p->positions || !p->rows_out || !p->offsets_out) return SPITE_BAD_ARG;
    if (p->num_heads < 1 || p->head_dim < 1 || p->kv_rank < 1 || p->rot_dim < 2 || p->rot_dim % 2 || p->n_tokens < 0) return SPITE_BAD_ARG;
    if (p->row < p->kv_rank + p->rot_dim) return SPITE_BAD_ARG;
    if (p->pairing != SPITE_PAIR_NEIGHBOURS && p->pairing != SPITE_PAIR_HALVES) return SPITE_BAD_ARG;
    if (p->rot_dim > 8192) return SPITE_UNSUPPORTED;
    if (p->n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)p->rot_dim * sizeof(float);
    const bool wide = p->head_dim % 4 == 0 && p->rot_dim % 4 == 0 && p->kv_rank % 2 == 0 && p->row % 2 == 0 &&
                      (((uintptr_t)p->q | (uintptr_t)p->q_out | (uintptr_t)p->q_sorted_out) & 15) == 0;
    if (dtype == SPITE_DT_F32) {
        if (wide) SPITE_LAUNCH((latent_queries_kernel<float, true>), p->n_tokens, 128, smem, st, *p);
        else SPITE_LAUNCH((latent_queries_kernel<float, false>), p->n_tokens, 128, smem, st, *p);
    } else if (dtype == SPITE_DT_BF16) {
        if (wide) SPITE_LAUNCH((latent_queries_kernel<__nv_bfloat16, true>), p->n_tokens, 128, smem, st, *p);
        else SPITE_LAUNCH((latent_queries_kernel<__nv_bfloat16, false>), p->n_tokens, 128, smem, st, *p);
    } else return SPITE_BAD_ARG;
    return spite_launch_status();
}
