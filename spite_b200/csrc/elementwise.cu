// Embedding gather and RMS norm.  Both are bound by memory traffic: one read of
// the row, one write.  The residual stream is float32; the norm writes the
// model's activation type.
#include "common.cuh"

// h[m, :] = table[token[m], :] * scale    (crates/spite-models/src/llama/llama4.rs:118-119; scale 1 there)
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ h, int d, int vocab, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x;
    const int tok = tokens[m];
    float* out = h + (size_t)m * d;
    if (tok < 0 || tok >= vocab) {          // the host rejects such ids before the launch
        for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)tok * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

// Four elements with one store.
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *(float4*)p = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2*)p = make_uint2(*(unsigned*)&lo, *(unsigned*)&hi);
}

// h[m, :] = table[token[m], :] * scale + pos_table[positions[m], :]: learned position vectors (the factor applies to the
// token's row only); the sum is float32
template <typename T>
__global__ void embed_positions_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                       const T* __restrict__ pos_table, const int* __restrict__ positions,
                                       float* __restrict__ h, int d, int vocab, int n_positions, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x;
    const int tok = tokens[m], pos = positions[m];
    float* out = h + (size_t)m * d;
    if (tok < 0 || tok >= vocab || pos < 0 || pos >= n_positions) {   // the host rejects such steps before the launch
        for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)tok * d;
    const T* pv = pos_table + (size_t)pos * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = to_f32(row[i]) * scale + to_f32(pv[i]);
}

// The same with four elements a thread: widths that are multiples of four.
__device__ __forceinline__ float4 load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 v = *(const uint2*)p;
    const __nv_bfloat162 lo = *(const __nv_bfloat162*)&v.x, hi = *(const __nv_bfloat162*)&v.y;
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
template <typename T>
__global__ void embed_positions_vec_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                           const T* __restrict__ pos_table, const int* __restrict__ positions,
                                           float* __restrict__ h, int d, int vocab, int n_positions, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x;
    const int tok = tokens[m], pos = positions[m];
    float* out = h + (size_t)m * d;
    const bool ok = tok >= 0 && tok < vocab && pos >= 0 && pos < n_positions;     // the host rejects other steps before the launch
    const T* row = table + (size_t)(ok ? tok : 0) * d;
    const T* pv = pos_table + (size_t)(ok ? pos : 0) * d;
    for (int i = 4 * threadIdx.x; i < d; i += 4 * blockDim.x) {
        const float4 e = load4(row + i), q = load4(pv + i);
        *(float4*)(out + i) = ok ? make_float4(e.x * scale + q.x, e.y * scale + q.y, e.z * scale + q.z, e.w * scale + q.w)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// out[m, :] = [a[m, :]; b[m, :]] in the activation type, for two float32 streams of width d; with `refill` every
// row of a becomes that vector afterwards (a thread overwrites what it has just read itself)
template <typename T>
__global__ void pack_pair_kernel(float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ refill,
                                 T* __restrict__ out, int d) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t m = blockIdx.x;
    float* ar = a + m * d;
    const float* br = b + m * d;
    T* o = out + m * 2 * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        o[i] = from_f32<T>(ar[i]);
        o[d + i] = from_f32<T>(br[i]);
        if (refill) ar[i] = refill[i];
    }
}

// The same with four elements a thread (16-byte loads of the two streams): widths that are multiples of four.
template <typename T>
__global__ void pack_pair_vec_kernel(float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ refill,
                                     T* __restrict__ out, int d4) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t m = blockIdx.x;
    float4* ar = (float4*)a + m * d4;
    const float4* br = (const float4*)b + m * d4;
    T* o = out + m * 8 * d4;
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        const float4 x = ar[i], y = br[i];
        store4(o + 4 * i, x.x, x.y, x.z, x.w);
        store4(o + 4 * (d4 + i), y.x, y.y, y.z, y.w);
        if (refill) ar[i] = ((const float4*)refill)[i];
    }
}

// y[i, :] = x[r, :] * rsqrt(mean(x[r]^2) + eps) * gain      r = rows ? rows[i] : i
// (crates/spite-models/src/dense.rs:175-181; the sum runs in float32)
// One block per row.  The row stays in registers between the sum and the scaling: every thread
// holds up to VPT groups of four elements, loaded with one 16-byte read each.
template <typename T, int VPT>
__global__ void rms_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                    const int* __restrict__ rows, T* __restrict__ y, int d, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const float4* in = (const float4*)(x + (size_t)r * d);
    const int d4 = d >> 2;
    float4 v[VPT];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = c < d4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) s += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)d + eps);
    T* out = y + (size_t)i * d;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < d4) {
            const float4 g = ((const float4*)gain)[c];
            store4(out + 4 * c, v[k].x * scale * g.x, v[k].y * scale * g.y, v[k].z * scale * g.z, v[k].w * scale * g.w);
        }
    }
}

// The same for widths that are no multiple of four, or too wide for the registers: two passes over the row.
template <typename T>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                const int* __restrict__ rows, T* __restrict__ y, int d, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const float* in = x + (size_t)r * d;
    float s = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { float v = in[c]; s += v * v; }
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)d + eps);
    T* out = y + (size_t)i * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[c] = from_f32<T>(in[c] * scale * gain[c]);
}

// logits = cap * tanh(logits * scale / cap), or logits * scale without a cap (cap <= 0)
__global__ void transform_logits_kernel(float* __restrict__ logits, long long n, float scale, float cap) {
    pdl_wait();
    pdl_launch_dependents();
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = logits[i] * scale;
        logits[i] = cap > 0.f ? cap * tanhf(v * inv_cap) : v;
    }
}

// dst[i, :] = src[idx[i], :]   (rows of activations brought into expert order), 16 bytes per thread and step
__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ idx,
                                   uint4* __restrict__ dst, int row_vecs) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = blockIdx.x;
    const uint4* in = src + (size_t)idx[i] * row_vecs;
    uint4* out = dst + i * row_vecs;
    for (int c = threadIdx.x; c < row_vecs; c += blockDim.x) out[c] = in[c];
}

SPITE_API int spite_gather_rows(const void* src, const int* idx, void* dst, int n_rows, long long row_bytes,
                                void* stream) {
    if (!src || !idx || !dst || n_rows < 0 || row_bytes <= 0) return SPITE_BAD_ARG;
    if (row_bytes % 16 || (((uintptr_t)src | (uintptr_t)dst) & 15)) return SPITE_UNSUPPORTED;
    if (n_rows == 0) return SPITE_OK;
    SPITE_LAUNCH(gather_rows_kernel, n_rows, 128, 0, (cudaStream_t)stream, (const uint4*)src, idx, (uint4*)dst,
                 (int)(row_bytes / 16));
    return spite_launch_status();
}

// Zero pages of a paged cache: `base` holds `n_outer` blocks of `outer_stride` bytes (one per cache of a
// group and per keys / values), each with pages of `page_bytes`.  grid (pages to clear, n_outer).
struct PageList { int n; int ids[60]; };
template <typename Word>
__global__ void clear_pages_kernel(unsigned char* __restrict__ base, long long outer_stride, long long page_bytes,
                                   const PageList pages) {
    pdl_wait();
    pdl_launch_dependents();
    Word* dst = (Word*)(base + (size_t)blockIdx.y * outer_stride + (size_t)pages.ids[blockIdx.x] * page_bytes);
    const long long n = page_bytes / (long long)sizeof(Word);
    Word zero;
    memset(&zero, 0, sizeof(Word));
    for (long long i = threadIdx.x; i < n; i += blockDim.x) dst[i] = zero;
}

// `page_ids` is host memory (the ids are passed to the kernel by value, 60 a launch).
SPITE_API int spite_clear_pages(void* base, long long n_outer, long long outer_stride, long long page_bytes,
                                int n_pages_total, const int* page_ids, int n_ids, void* stream) {
    if (!base || n_outer < 1 || outer_stride < 1 || page_bytes < 1 || n_pages_total < 1 || n_ids < 0) return SPITE_BAD_ARG;
    if (n_ids > 0 && !page_ids) return SPITE_BAD_ARG;
    if (page_bytes % 4 || outer_stride % 4 || ((uintptr_t)base & 3) || n_outer > 65535) return SPITE_UNSUPPORTED;
    const bool wide = page_bytes % 16 == 0 && outer_stride % 16 == 0 && ((uintptr_t)base & 15) == 0;
    for (int i = 0; i < n_ids; ++i)
        if (page_ids[i] < 0 || page_ids[i] >= n_pages_total) return SPITE_BAD_ARG;
    for (int at = 0; at < n_ids; at += 60) {
        PageList list;
        list.n = n_ids - at < 60 ? n_ids - at : 60;
        for (int i = 0; i < list.n; ++i) list.ids[i] = page_ids[at + i];
        if (wide)
            SPITE_LAUNCH(clear_pages_kernel<uint4>, dim3(list.n, (unsigned)n_outer), 256, 0, (cudaStream_t)stream,
                         (unsigned char*)base, outer_stride, page_bytes, list);
        else
            SPITE_LAUNCH(clear_pages_kernel<unsigned>, dim3(list.n, (unsigned)n_outer), 256, 0, (cudaStream_t)stream,
                         (unsigned char*)base, outer_stride, page_bytes, list);
        if (spite_launch_status() != SPITE_OK) return SPITE_LAUNCH_FAILED;
    }
    return SPITE_OK;
}

SPITE_API int spite_transform_logits(float* logits, long long n, float scale, float softcap, void* stream) {
    if (!logits || n < 0 || !(scale == scale) || !(softcap == softcap)) return SPITE_BAD_ARG;
    if (n == 0) return SPITE_OK;
    const long long blocks = (n + 255) / 256;
    SPITE_LAUNCH(transform_logits_kernel, (int)(blocks < 4096 ? blocks : 4096), 256, 0, (cudaStream_t)stream, logits, n,
                 scale, softcap);
    return spite_launch_status();
}

SPITE_API int spite_embed(int dtype, const void* table, const int* tokens, float* h,
                          int n_tokens, int d, int vocab, float scale, void* stream) {
    if (!table || !tokens || !h || n_tokens < 0 || d <= 0 || vocab <= 0 || !(scale == scale)) return SPITE_BAD_ARG;
    if (n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == SPITE_DT_F32)
        SPITE_LAUNCH(embed_kernel<float>, n_tokens, threads, 0, st, (const float*)table, tokens, h, d, vocab, scale);
    else if (dtype == SPITE_DT_BF16)
        SPITE_LAUNCH(embed_kernel<__nv_bfloat16>, n_tokens, threads, 0, st, (const __nv_bfloat16*)table, tokens, h, d, vocab, scale);
    else
        return SPITE_BAD_ARG;
    return spite_launch_status();
}

SPITE_API int spite_embed_positions(int dtype, const void* table, const int* tokens, const void* pos_table,
                                    const int* positions, float* h, int n_tokens, int d, int vocab, int n_positions,
                                    float scale, void* stream) {
    if (!table || !tokens || !pos_table || !positions || !h || n_tokens < 0 || d <= 0 || vocab <= 0 || n_positions <= 0 ||
        !(scale == scale))
        return SPITE_BAD_ARG;
    if (dtype != SPITE_DT_F32 && dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (d % 4 == 0 && ((((uintptr_t)table | (uintptr_t)pos_table | (uintptr_t)h) & 15) == 0)) {
        if (dtype == SPITE_DT_F32)
            SPITE_LAUNCH(embed_positions_vec_kernel<float>, n_tokens, threads, 0, st, (const float*)table, tokens,
                         (const float*)pos_table, positions, h, d, vocab, n_positions, scale);
        else
            SPITE_LAUNCH(embed_positions_vec_kernel<__nv_bfloat16>, n_tokens, threads, 0, st, (const __nv_bfloat16*)table, tokens,
                         (const __nv_bfloat16*)pos_table, positions, h, d, vocab, n_positions, scale);
        return spite_launch_status();
    }
    if (dtype == SPITE_DT_F32)
        SPITE_LAUNCH(embed_positions_kernel<float>, n_tokens, threads, 0, st, (const float*)table, tokens,
                     (const float*)pos_table, positions, h, d, vocab, n_positions, scale);
    else
        SPITE_LAUNCH(embed_positions_kernel<__nv_bfloat16>, n_tokens, threads, 0, st, (const __nv_bfloat16*)table, tokens,
                     (const __nv_bfloat16*)pos_table, positions, h, d, vocab, n_positions, scale);
    return spite_launch_status();
}

// `a` and `b` float32 [n_rows, d] -> `out` [n_rows, 2 d] of `out_dtype`; `refill` [d] float32 or null
SPITE_API int spite_pack_pair(int out_dtype, float* a, const float* b, const float* refill, void* out, int n_rows, int d,
                              void* stream) {
    if (!a || !b || !out || n_rows < 0 || d <= 0) return SPITE_BAD_ARG;
    if (out_dtype != SPITE_DT_F32 && out_dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (n_rows == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    const bool f32 = out_dtype == SPITE_DT_F32;
    if (d % 4 == 0 && ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)refill | (uintptr_t)out) & 15) == 0)) {
        if (f32) SPITE_LAUNCH(pack_pair_vec_kernel<float>, n_rows, threads, 0, st, a, b, refill, (float*)out, d / 4);
        else SPITE_LAUNCH(pack_pair_vec_kernel<__nv_bfloat16>, n_rows, threads, 0, st, a, b, refill, (__nv_bfloat16*)out, d / 4);
        return spite_launch_status();
    }
    if (f32) SPITE_LAUNCH(pack_pair_kernel<float>, n_rows, threads, 0, st, a, b, refill, (float*)out, d);
    else SPITE_LAUNCH(pack_pair_kernel<__nv_bfloat16>, n_rows, threads, 0, st, a, b, refill, (__nv_bfloat16*)out, d);
    return spite_launch_status();
}

SPITE_API int spite_rms_norm(int out_dtype, const float* x, const float* gain, const int* rows,
                             void* y, int n_rows, int d, float eps, void* stream) {
    if (!x || !gain || !y || n_rows < 0 || d <= 0 || !(eps > 0.f)) return SPITE_BAD_ARG;
    if (n_rows == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype != SPITE_DT_F32 && out_dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    const bool f32 = out_dtype == SPITE_DT_F32;
    const bool aligned = d % 4 == 0 && ((((uintptr_t)x | (uintptr_t)gain | (uintptr_t)y) & 15) == 0);
    if (aligned && d <= 256 * 4 * 8) {
        // threads and groups per thread so that every thread has work: 128 x 1 up to 256 x 8
        const int d4 = d / 4;
        const int threads = d4 <= 128 ? 128 : 256;
        const int vpt = (d4 + threads - 1) / threads;
#define SPITE_RMS(V)                                                                                              \
        if (f32) SPITE_LAUNCH((rms_norm_vec_kernel<float, V>), n_rows, threads, 0, st, x, gain, rows, (float*)y, d, eps); \
        else SPITE_LAUNCH((rms_norm_vec_kernel<__nv_bfloat16, V>), n_rows, threads, 0, st, x, gain, rows, (__nv_bfloat16*)y, d, eps)
        if (vpt <= 1) { SPITE_RMS(1); }
        else if (vpt <= 2) { SPITE_RMS(2); }
        else if (vpt <= 4) { SPITE_RMS(4); }
        else if (vpt <= 5) { SPITE_RMS(5); }
        else { SPITE_RMS(8); }
#undef SPITE_RMS
        return spite_launch_status();
    }
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    if (f32)
        SPITE_LAUNCH(rms_norm_kernel<float>, n_rows, threads, 0, st, x, gain, rows, (float*)y, d, eps);
    else
        SPITE_LAUNCH(rms_norm_kernel<__nv_bfloat16>, n_rows, threads, 0, st, x, gain, rows, (__nv_bfloat16*)y, d, eps);
    return spite_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// A sublayer whose output is normed before it joins the residual stream:
//     h[m, :] += mult * y[m, :] * rsqrt(mean(y[m]^2) + eps) * gain
// and, if `next_out` is given, the norm that the next sublayer reads, of the row just made:
//     next_out[m, :] = h[m, :] * rsqrt(mean(h[m]^2) + eps) * next_gain
// (without `next_gain`: the row itself in the output type, for a sublayer that reads the stream unnormed)
// One block per row; the row (y, then h) stays in registers between the sums and the scalings, VPT groups of four
// elements a thread.  All sums float32.
template <typename T, int VPT>
__global__ void rms_norm_residual_vec_kernel(const float* __restrict__ y, const float* __restrict__ gain, float* __restrict__ h,
                                             const float* __restrict__ next_gain, T* __restrict__ next_out, int d, float eps,
                                             float mult) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const size_t m = blockIdx.x;
    const float4* in = (const float4*)(y + m * d);
    float4* hr = (float4*)(h + m * d);
    const int d4 = d >> 2;
    float4 v[VPT], r[VPT];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = c < d4 ? in[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        r[k] = c < d4 ? hr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) s += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)d + eps);
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < d4) {
            const float4 g = ((const float4*)gain)[c];
            r[k].x += mult * (v[k].x * scale * g.x); r[k].y += mult * (v[k].y * scale * g.y);
            r[k].z += mult * (v[k].z * scale * g.z); r[k].w += mult * (v[k].w * scale * g.w);
            hr[c] = r[k];
            s2 += (r[k].x * r[k].x + r[k].y * r[k].y) + (r[k].z * r[k].z + r[k].w * r[k].w);
        }
    }
    if (!next_out) return;
    T* out = next_out + m * d;
    if (!next_gain) {                                          // the next sublayer reads the row itself, not its norm
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < d4) store4(out + 4 * c, r[k].x, r[k].y, r[k].z, r[k].w);
        }
        return;
    }
    s2 = block_sum(s2, scratch);
    const float scale2 = 1.0f / sqrtf(s2 / (float)d + eps);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < d4) {
            const float4 g = ((const float4*)next_gain)[c];
            store4(out + 4 * c, r[k].x * scale2 * g.x, r[k].y * scale2 * g.y, r[k].z * scale2 * g.z, r[k].w * scale2 * g.w);
        }
    }
}

// The same for any width: passes over the rows in global memory.
template <typename T>
__global__ void rms_norm_residual_kernel(const float* __restrict__ y, const float* __restrict__ gain, float* __restrict__ h,
                                         const float* __restrict__ next_gain, T* __restrict__ next_out, int d, float eps,
                                         float mult) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const size_t m = blockIdx.x;
    const float* in = y + m * d;
    float* hr = h + m * d;
    float s = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { const float v = in[c]; s += v * v; }
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)d + eps);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const float v = hr[c] + mult * (in[c] * scale * gain[c]);
        hr[c] = v;                                             // (read again below by the thread that wrote it)
        s2 += v * v;
    }
    if (!next_out) return;
    T* out = next_out + m * d;
    if (!next_gain) {                                          // the next sublayer reads the row itself, not its norm
        for (int c = threadIdx.x; c < d; c += blockDim.x) out[c] = from_f32<T>(hr[c]);
        return;
    }
    s2 = block_sum(s2, scratch);
    const float scale2 = 1.0f / sqrtf(s2 / (float)d + eps);
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[c] = from_f32<T>(hr[c] * scale2 * next_gain[c]);
}

SPITE_API int spite_rms_norm_residual(int out_dtype, const float* y, const float* gain, float* h, const float* next_gain,
                                      void* next_out, int n_rows, int d, float eps, float mult, void* stream) {
    if (!y || !gain || !h || n_rows < 0 || d <= 0 || !(eps > 0.f) || !(mult == mult)) return SPITE_BAD_ARG;
    if (next_gain && !next_out) return SPITE_BAD_ARG;          // (an output without a gain: the row itself, not its norm)
    if (out_dtype != SPITE_DT_F32 && out_dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (n_rows == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool f32 = out_dtype == SPITE_DT_F32;
    const bool aligned = d % 4 == 0 &&
        ((((uintptr_t)y | (uintptr_t)gain | (uintptr_t)h | (uintptr_t)next_gain | (uintptr_t)next_out) & 15) == 0);
    if (aligned && d <= 256 * 4 * 4) {
        const int d4 = d / 4;
        const int threads = d4 <= 128 ? 128 : 256;
        const int vpt = (d4 + threads - 1) / threads;
#define SPITE_RMSR(V)                                                                                                      \
        if (f32) SPITE_LAUNCH((rms_norm_residual_vec_kernel<float, V>), n_rows, threads, 0, st, y, gain, h, next_gain,     \
                              (float*)next_out, d, eps, mult);                                                             \
        else SPITE_LAUNCH((rms_norm_residual_vec_kernel<__nv_bfloat16, V>), n_rows, threads, 0, st, y, gain, h, next_gain, \
                          (__nv_bfloat16*)next_out, d, eps, mult)
        if (vpt <= 1) { SPITE_RMSR(1); }
        else if (vpt <= 2) { SPITE_RMSR(2); }
        else { SPITE_RMSR(4); }
#undef SPITE_RMSR
        return spite_launch_status();
    }
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    if (f32) SPITE_LAUNCH(rms_norm_residual_kernel<float>, n_rows, threads, 0, st, y, gain, h, next_gain, (float*)next_out, d, eps, mult);
    else SPITE_LAUNCH(rms_norm_residual_kernel<__nv_bfloat16>, n_rows, threads, 0, st, y, gain, h, next_gain,
                      (__nv_bfloat16*)next_out, d, eps, mult);
    return spite_launch_status();
}

// out[m, :] (=|+=) vec: a bias that a product then adds its rows to (float32 [n_rows, d]).
__global__ void fill_rows_kernel(float* __restrict__ out, const float* __restrict__ vec, long long n, int d, int accumulate) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float b = vec[i % d];
        out[i] = accumulate ? out[i] + b : b;
    }
}

SPITE_API int spite_fill_rows(float* out, const float* vec, int n_rows, int d, int accumulate, void* stream) {
    if (!out || !vec || n_rows < 0 || d <= 0) return SPITE_BAD_ARG;
    if (n_rows == 0) return SPITE_OK;
    const long long n = (long long)n_rows * d;
    const long long blocks = (n + 255) / 256;
    SPITE_LAUNCH(fill_rows_kernel, (int)(blocks < 8192 ? blocks : 8192), 256, 0, (cudaStream_t)stream, out, vec, n, d, accumulate);
    return spite_launch_status();
}

// What stands between a mixer's heads and its output projection:
//     out[m, h * size + j] = x[m, h * size + j] * r_mh * gain[h * size + j] * sigmoid(gates[m, h * size + j])
// (`gate_silu`: times z sigmoid(z) of the gate column z instead; without `gain_per_head` the gain has `size` elements
// that all heads share)
// r_mh = rsqrt(mean_j(x[m, h, :]^2) + eps) if eps > 0, else 1; gain and gates may be null (a factor of one).
// `gates` has rows of `gate_stride` elements (the gate columns of a wider product).  One warp per (token, head); the
// head's elements stay in registers between the sum and the scaling while they are few enough.
template <typename TX, typename TO>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const TX* __restrict__ x, const TX* __restrict__ gates,
                                                             long long gate_stride, const float* __restrict__ gain,
                                                             TO* __restrict__ out, int n_tokens, int heads, int size, float eps,
                                                             int gate_silu, int gain_per_head) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= (long long)n_tokens * heads) return;
    const long long m = row / heads;
    const int h = (int)(row % heads);
    const size_t base = (size_t)m * heads * size + (size_t)h * size;
    const TX* in = x + base;
    float mul = 1.f;
    if (eps > 0.f) {
        float s = 0.f;
        for (int j = lane; j < size; j += 32) { const float v = to_f32(in[j]); s += v * v; }
        s = warp_sum(s);
        mul = 1.0f / sqrtf(s / (float)size + eps);
    }
    const TX* g = gates ? gates + (size_t)m * gate_stride + (size_t)h * size : nullptr;
    const float* w = gain ? gain + (gain_per_head ? (size_t)h * size : 0) : nullptr;
    TO* o = out + base;
    for (int j = lane; j < size; j += 32) {
        float v = to_f32(in[j]) * mul;
        if (w) v *= w[j];
        if (g) {
            const float z = to_f32(g[j]), sg = 1.0f / (1.0f + expf(-z));
            v *= gate_silu ? z * sg : sg;
        }
        o[j] = from_f32<TO>(v);
    }
}

// x_dtype: type of x and gates; out_dtype: type of out (x may be the float32 result of a recurrence while out feeds a
// bfloat16 product); out may be x.
SPITE_API int spite_head_norm_gate(int x_dtype, int out_dtype, const void* x, const void* gates, long long gate_stride,
                                   const float* gain, void* out, int n_tokens, int heads, int size, float eps, int gate_silu,
                                   int gain_per_head, void* stream) {
    if (!x || !out || n_tokens < 0 || heads < 1 || size < 1 || !(eps == eps) || eps < 0.f) return SPITE_BAD_ARG;
    if (gates && gate_stride < (long long)heads * size) return SPITE_BAD_ARG;
    if (x_dtype != SPITE_DT_F32 && x_dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (out_dtype != SPITE_DT_F32 && out_dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (x_dtype == SPITE_DT_BF16 && out_dtype == SPITE_DT_F32) return SPITE_UNSUPPORTED;
    if (n_tokens == 0) return SPITE_OK;
    const long long rows = (long long)n_tokens * heads;
    const long long blocks = (rows + 3) / 4;
    if (blocks > 0x7fffffffLL) return SPITE_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == SPITE_DT_F32 && out_dtype == SPITE_DT_F32)
        SPITE_LAUNCH((head_norm_gate_kernel<float, float>), (int)blocks, 128, 0, st, (const float*)x, (const float*)gates,
                     gate_stride, gain, (float*)out, n_tokens, heads, size, eps, gate_silu, gain_per_head);
    else if (x_dtype == SPITE_DT_F32)
        SPITE_LAUNCH((head_norm_gate_kernel<float, __nv_bfloat16>), (int)blocks, 128, 0, st, (const float*)x, (const float*)gates,
                     gate_stride, gain, (__nv_bfloat16*)out, n_tokens, heads, size, eps, gate_silu, gain_per_head);
    else
        SPITE_LAUNCH((head_norm_gate_kernel<__nv_bfloat16, __nv_bfloat16>), (int)blocks, 128, 0, st, (const __nv_bfloat16*)x,
                     (const __nv_bfloat16*)gates, gate_stride, gain, (__nv_bfloat16*)out, n_tokens, heads, size, eps, gate_silu, gain_per_head);
    return spite_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// out (T) = x (float32), element by element: the copy of the residual stream that a sublayer without a norm in front
// of it reads.
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long n4, long long n) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const float4 v = ((const float4*)x)[i];
        store4(out + 4 * i, v.x, v.y, v.z, v.w);
    }
    if (blockIdx.x == 0)
        for (long long i = 4 * n4 + threadIdx.x; i < n; i += blockDim.x) out[i] = from_f32<T>(x[i]);
}

SPITE_API int spite_cast_rows(int out_dtype, const float* x, void* out, long long n, void* stream) {
    if (!x || !out || n < 0) return SPITE_BAD_ARG;
    if (out_dtype != SPITE_DT_F32 && out_dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (n == 0) return SPITE_OK;
    const bool aligned = (((uintptr_t)x | (uintptr_t)out) & 15) == 0;
    const long long n4 = aligned ? n / 4 : 0;
    const long long blocks = (n4 + 255) / 256;
    const int grid = (int)(blocks < 1 ? 1 : (blocks < 4096 ? blocks : 4096));
    if (out_dtype == SPITE_DT_F32) SPITE_LAUNCH(cast_rows_kernel<float>, grid, 256, 0, (cudaStream_t)stream, x, (float*)out, n4, n);
    else SPITE_LAUNCH(cast_rows_kernel<__nv_bfloat16>, grid, 256, 0, (cudaStream_t)stream, x, (__nv_bfloat16*)out, n4, n);
    return spite_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// A short causal convolution over time on every channel of a projection's output, carried from step to step:
//     y[t, c] = act( sum_j w[c, j] * u[t - taps + 1 + j, c] ),   u = 0 before the sequence's first token
// u is the float32 output of the projection; the last taps - 1 rows of u of every request live in its state slot
// (float32 [taps - 1, channels], oldest first; all zeros: the start of a sequence) and are renewed by the step.
// Columns behind the channels (`copy_columns` of them) are passed on unchanged (gate columns of the same product).
// A thread owns one column of one block of CONV_TB tokens of one segment; only the thread of a segment's first block
// reads or writes the slot.  Sums in float32 in the order of the taps.
struct ShortConvParams {
    const float* x;             // [tokens, x_stride]
    long long x_stride;
    const float* w;             // [channels, taps]
    void* out;                  // [tokens, out_stride] (T or float32)
    long long out_stride;
    float* state;               // state + slot * slot_stride: [taps - 1, channels]
    long long slot_stride;
    const int* cu_seqlens;      // [segments + 1]
    const int* slots;           // [segments]
    int n_segments, channels, taps, copy_columns;
    int activation;             // 0: none, 1: silu
    int max_seg_len;
};

constexpr int CONV_TB = 16;
constexpr int CONV_MAX_TAPS = 8;

template <typename T>
__global__ void __launch_bounds__(128) short_conv_kernel(const ShortConvParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= p.channels + p.copy_columns) return;
    const int s = blockIdx.y;
    const int t0 = p.cu_seqlens[s], n = p.cu_seqlens[s + 1] - t0;
    const int i0 = blockIdx.z * CONV_TB;
    if (i0 >= n) return;
    const int slot = p.slots[s];
    // A captured step pads its rows with copies of its first row.  A copy must come out as the first row does (its
    // keys go to the same place of the cache), but it would read a slot that the first row's thread may have renewed
    // already: so the first row's thread writes the copies' rows as well, and the copies' threads do nothing.
    if (s > 0 && slot == p.slots[0]) return;
    const int i1 = min(i0 + CONV_TB, n);
    T* out = (T*)p.out;
    float y[CONV_TB];
    if (c >= p.channels) {
        for (int i = i0; i < i1; ++i) {
            y[i - i0] = p.x[(size_t)(t0 + i) * p.x_stride + c];
            out[(size_t)(t0 + i) * p.out_stride + c] = from_f32<T>(y[i - i0]);
        }
    } else {
        const int taps = p.taps;
        float w[CONV_MAX_TAPS], win[CONV_MAX_TAPS - 1], old[CONV_MAX_TAPS - 1];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)               // the taps right-aligned: w[CONV_MAX_TAPS - 1] is the current token's
            w[j] = j >= CONV_MAX_TAPS - taps ? p.w[(size_t)c * taps + j - (CONV_MAX_TAPS - taps)] : 0.f;
        float* st = p.state + (size_t)slot * p.slot_stride + c;
#pragma unroll
        for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) old[k] = (i0 == 0 && k < taps - 1) ? st[(size_t)k * p.channels] : 0.f;
        // win[CONV_MAX_TAPS - 1 - d] is the input d tokens back
#pragma unroll
        for (int d = 1; d < CONV_MAX_TAPS; ++d) {
            float v = 0.f;
            if (d < taps) {
                const int idx = i0 - d;
                if (idx >= 0) v = p.x[(size_t)(t0 + idx) * p.x_stride + c];
                else if (taps - 1 + idx >= 0) {
#pragma unroll
                    for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) if (k == taps - 1 + idx) v = old[k];
                }
            }
            win[CONV_MAX_TAPS - 1 - d] = v;
        }
        for (int i = i0; i < i1; ++i) {
            const float cur = p.x[(size_t)(t0 + i) * p.x_stride + c];
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) acc = fmaf(w[j], win[j], acc);
            acc = fmaf(w[CONV_MAX_TAPS - 1], cur, acc);
            if (p.activation == 1) acc = acc / (1.0f + expf(-acc));
            y[i - i0] = acc;
            out[(size_t)(t0 + i) * p.out_stride + c] = from_f32<T>(acc);
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS - 2; ++j) win[j] = win[j + 1];
            win[CONV_MAX_TAPS - 2] = cur;
        }
        if (i0 == 0) {
            // the slot's next content: the last taps - 1 inputs of the sequence so far
            for (int k = 0; k < taps - 1; ++k) {
                const int idx = n - (taps - 1) + k;
                float v = 0.f;
                if (idx >= 0) v = p.x[(size_t)(t0 + idx) * p.x_stride + c];
                else {
#pragma unroll
                    for (int kk = 0; kk < CONV_MAX_TAPS - 1; ++kk) if (kk == taps - 1 + idx) v = old[kk];
                }
                st[(size_t)k * p.channels] = v;
            }
        }
    }
    if (s == 0 && i0 == 0) {
        for (int s2 = 1; s2 < p.n_segments; ++s2) {
            if (p.slots[s2] != slot) continue;
            const int u0 = p.cu_seqlens[s2], m = min(p.cu_seqlens[s2 + 1] - u0, i1);
            for (int i = 0; i < m; ++i) out[(size_t)(u0 + i) * p.out_stride + c] = from_f32<T>(y[i]);
        }
    }
}

SPITE_API int spite_short_conv(int out_dtype, const ShortConvParams* p, void* stream) {
    if (!p || !p->x || !p->w || !p->out || !p->state || !p->cu_seqlens || !p->slots) return SPITE_BAD_ARG;
    if (p->n_segments < 0 || p->channels < 1 || p->taps < 1 || p->copy_columns < 0 || p->max_seg_len < 0) return SPITE_BAD_ARG;
    if (p->x_stride < p->channels + p->copy_columns || p->out_stride < p->channels + p->copy_columns) return SPITE_BAD_ARG;
    if (p->taps > 1 && p->slot_stride < (long long)(p->taps - 1) * p->channels) return SPITE_BAD_ARG;
    if (p->activation != 0 && p->activation != 1) return SPITE_BAD_ARG;
    if (out_dtype != SPITE_DT_F32 && out_dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (p->taps > CONV_MAX_TAPS || p->n_segments > 65535) return SPITE_UNSUPPORTED;
    if (p->n_segments == 0 || p->max_seg_len == 0) return SPITE_OK;
    const int cols = p->channels + p->copy_columns;
    const int zb = (p->max_seg_len + CONV_TB - 1) / CONV_TB;
    if (zb > 65535) return SPITE_UNSUPPORTED;
    dim3 grid((cols + 127) / 128, p->n_segments, zb);
    if (out_dtype == SPITE_DT_F32) SPITE_LAUNCH(short_conv_kernel<float>, grid, 128, 0, (cudaStream_t)stream, *p);
    else SPITE_LAUNCH(short_conv_kernel<__nv_bfloat16>, grid, 128, 0, (cudaStream_t)stream, *p);
    return spite_launch_status();
}
