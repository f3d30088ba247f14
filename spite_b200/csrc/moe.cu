// Router of a mixture-of-experts feed-forward and the ordering of tokens by expert.
//
// logits: l = Wr x in float32 (crates/spite-models/src/moe.rs:65-66).
// select: the k largest raw logits are chosen, equal logits preferring the lower expert
//   id (moe.rs:110-116, a stable descending sort); the weight is sigmoid(logit)
//   (moe.rs:120).  No softmax, no renormalisation.  A second scoring rule, SCORE_SOFTMAX_RENORM: the weight
//   of a choice is its share of the softmax over all experts divided by the sum of the chosen shares
//   (+ 1e-20), all float32; the order of the experts is the same (the softmax is monotonic).
//   A third, SCORE_SOFTMAX_BIASED: the experts are ordered by their softmax share plus a per-expert constant
//   (`choice_bias`), and the weight of a choice is its share alone, not renormalised.
//   Choices are stored slot-major: expert_ids[slot][token], weights[slot][token].
// sort: for every choice slot a stable counting sort of the tokens by expert:
//   offsets[slot][e] .. offsets[slot][e+1] are the places of expert e's tokens in
//   sorted_rows[slot][:], in ascending token order; sorted_weights[slot][i], if asked for, is the
//   weight of the token at place i (for a product that scales its rows in the sorted order).
//   No host round trip: the grouped products read these arrays on the device.
//
// Two kernels.  The first computes the logits (8 tokens x 2 experts at a time, the block's 8
// warps splitting the width), one pair of experts a block, so that a few tokens still spread over
// several multiprocessors.  The second, one block per choice slot, selects and sorts.
// A logit is summed in an order fixed by the width alone.
#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 1024;
constexpr int TB = 8;                  // tokens per block of the logits kernel
constexpr int EB = 2;                  // experts per block
constexpr int WARPS = 8;
constexpr int SCORE_SIGMOID = 0, SCORE_SOFTMAX_RENORM = 1, SCORE_SOFTMAX_BIASED = 2;

__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 t = *(const float4*)p;
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *(const uint2*)p;
    const __nv_bfloat162 a = *(const __nv_bfloat162*)&t.x, b = *(const __nv_bfloat162*)&t.y;
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

// grid (ceil(tokens / TB), ceil(experts / experts_per_block)), block 256.  A block computes the logits
// of TB tokens for experts_per_block experts, EB at a time; from the second pair on its tokens come
// out of the first-level cache.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32) route_logits_kernel(const T* __restrict__ x, const float* __restrict__ wr,
                                                                 int n_tokens, int d, int n_experts, int experts_per_block,
                                                                 float* __restrict__ logits) {
    __shared__ float part[WARPS][EB * TB];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * TB;
    const int e_end = min(n_experts, (int)(blockIdx.y + 1) * experts_per_block);
    const bool vec = (d % 4 == 0) && (((uintptr_t)wr & 15) == 0) && (((uintptr_t)x & 15) == 0);
    for (int e0 = blockIdx.y * experts_per_block; e0 < e_end; e0 += EB) {
        float acc[EB][TB];
#pragma unroll
        for (int e = 0; e < EB; ++e)
#pragma unroll
            for (int t = 0; t < TB; ++t) acc[e][t] = 0.f;

        if (vec) {
            const int n4 = d >> 2;                            // groups of four elements
            const int lo = (int)((long long)n4 * warp / WARPS), hi = (int)((long long)n4 * (warp + 1) / WARPS);
            for (int k4 = lo + lane; k4 < hi; k4 += 32) {
                float w[EB][4];
#pragma unroll
                for (int e = 0; e < EB; ++e) {
                    if (e0 + e < e_end) load4(wr + (size_t)(e0 + e) * d + 4 * k4, w[e]);
                    else w[e][0] = w[e][1] = w[e][2] = w[e][3] = 0.f;
                }
#pragma unroll
                for (int t = 0; t < TB; ++t) {
                    if (t0 + t < n_tokens) {
                        float xv[4];
                        load4(x + (size_t)(t0 + t) * d + 4 * k4, xv);
#pragma unroll
                        for (int e = 0; e < EB; ++e)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[e][t] = fmaf(xv[i], w[e][i], acc[e][t]);
                    }
                }
            }
        } else {
            const int lo = (int)((long long)d * warp / WARPS), hi = (int)((long long)d * (warp + 1) / WARPS);
            for (int k = lo + lane; k < hi; k += 32) {
#pragma unroll
                for (int t = 0; t < TB; ++t) {
                    if (t0 + t < n_tokens) {
                        const float xv = to_f32(x[(size_t)(t0 + t) * d + k]);
#pragma unroll
                        for (int e = 0; e < EB; ++e)
                            if (e0 + e < e_end) acc[e][t] = fmaf(xv, wr[(size_t)(e0 + e) * d + k], acc[e][t]);
                    }
                }
            }
        }
        __syncthreads();                                      // the sums of the pair before have been read
#pragma unroll
        for (int e = 0; e < EB; ++e)
#pragma unroll
            for (int t = 0; t < TB; ++t) {
                const float s = warp_sum(acc[e][t]);
                if (lane == 0) part[warp][e * TB + t] = s;
            }
        __syncthreads();
        if (threadIdx.x < EB * TB) {
            const int e = threadIdx.x / TB, t = threadIdx.x % TB;
            if (e0 + e < e_end && t0 + t < n_tokens) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) s += part[w][threadIdx.x];
                logits[(size_t)(t0 + t) * n_experts + e0 + e] = s;
            }
        }
    }
}

// grid top_k, block 1024: block `slot` picks every token's slot-th expert and sorts the tokens by it.
__global__ void __launch_bounds__(1024) select_and_sort_kernel(const float* __restrict__ logits, int n_tokens,
                                                               int n_experts, int top_k,
                                                               int* __restrict__ expert_ids, float* __restrict__ weights,
                                                               int* __restrict__ offsets,
                                                               int* __restrict__ sorted_rows, int scoring,
                                                               float* __restrict__ sorted_weights,
                                                               const float* __restrict__ choice_bias) {
    __shared__ int counts[MAX_EXPERTS + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int slot = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    int* ids = expert_ids + (size_t)slot * n_tokens;
    for (int t = threadIdx.x; t < n_tokens; t += blockDim.x) {
        // the slot-th element in the order (logit descending, expert id ascending)
        const float* l = logits + (size_t)t * n_experts;
        if (scoring == SCORE_SOFTMAX_BIASED) {
            // share_e = exp(l_e - max) / Z; the slot-th expert in the order (share + bias descending, expert id ascending)
            float mx = -INFINITY, z = 0.f;
            for (int e = 0; e < n_experts; ++e) mx = fmaxf(mx, l[e]);
            for (int e = 0; e < n_experts; ++e) z += expf(l[e] - mx);
            const float inv_z = 1.0f / z;                    // (one rounding for every share of the token, choice and weight alike)
            float pv = INFINITY, bv = 0.f;
            int pe = -1, be = 0;
            for (int s = 0; s <= slot; ++s) {
                bv = -INFINITY;
                be = -1;
                for (int e = 0; e < n_experts; ++e) {
                    const float v = expf(l[e] - mx) * inv_z + choice_bias[e];
                    const bool after_prev = v < pv || (v == pv && e > pe);
                    if (after_prev && (be < 0 || v > bv)) { bv = v; be = e; }
                }
                if (be < 0) { be = 0; bv = 0.f; }
                pv = bv;
                pe = be;
            }
            ids[t] = be;
            weights[(size_t)slot * n_tokens + t] = expf(l[be] - mx) * inv_z;
            atomicAdd(&counts[be + 1], 1);
            continue;
        }
        float prev_v = INFINITY;
        int prev_e = -1;
        float best_v = 0.f, mine_v = 0.f;
        int best_e = 0, mine_e = 0;
        float chosen_max = 0.f, chosen_sum = 0.f;            // of exp(logit - largest logit) over the chosen experts
        const int picks = scoring == SCORE_SOFTMAX_RENORM ? top_k : slot + 1;
        for (int s = 0; s < picks; ++s) {
            best_v = -INFINITY;
            best_e = -1;
            for (int e = 0; e < n_experts; ++e) {
                const float v = l[e];
                const bool after_prev = v < prev_v || (v == prev_v && e > prev_e);
                if (after_prev && (best_e < 0 || v > best_v)) { best_v = v; best_e = e; }
            }
            if (best_e < 0) { best_e = 0; best_v = l[0]; }    // logits that do not compare (NaN): still a valid id
            prev_v = best_v;
            prev_e = best_e;
            if (s == 0) chosen_max = best_v;                 // the largest logit of all
            chosen_sum += expf(best_v - chosen_max);
            if (s == slot) { mine_v = best_v; mine_e = best_e; }
        }
        ids[t] = mine_e;
        float w;
        if (scoring == SCORE_SOFTMAX_RENORM) {
            // share_e = exp(l_e - max) / Z with Z over all experts; w = share / (sum of chosen shares + 1e-20)
            float z = 0.f;
            for (int e = 0; e < n_experts; ++e) z += expf(l[e] - chosen_max);
            w = (expf(mine_v - chosen_max) / z) / (chosen_sum / z + 1e-20f);
        } else {
            w = 1.0f / (1.0f + expf(-mine_v));
        }
        weights[(size_t)slot * n_tokens + t] = w;
        atomicAdd(&counts[mine_e + 1], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int e = 0; e < n_experts; ++e) counts[e + 1] += counts[e];
    __syncthreads();
    int* off = offsets + (size_t)slot * (n_experts + 1);
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) off[e] = counts[e];
    int* rows = sorted_rows + (size_t)slot * n_tokens;
    for (int e = warp; e < n_experts; e += nwarps) {
        int base = counts[e];
        if (counts[e + 1] == base) continue;
        for (int t0 = 0; t0 < n_tokens; t0 += 32) {
            const int t = t0 + lane;
            const bool mine = t < n_tokens && ids[t] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int at = base + __popc(mask & ((1u << lane) - 1u));
                rows[at] = t;
                if (sorted_weights) sorted_weights[(size_t)slot * n_tokens + at] = weights[(size_t)slot * n_tokens + t];
            }
            base += __popc(mask);
        }
    }
}

}  // namespace

// `logits` [tokens, experts] float32 is always written (the caller owns it).
SPITE_API int spite_moe_route(int dtype, const void* x, const float* w_router, int n_tokens, int d,
                              int n_experts, int top_k, int* expert_ids, float* weights,
                              float* logits, int* offsets, int* sorted_rows, int scoring, float* sorted_weights,
                              const float* choice_bias, void* stream) {
    if (!x || !w_router || !expert_ids || !weights || !logits || !offsets || !sorted_rows) return SPITE_BAD_ARG;
    if (scoring != SCORE_SIGMOID && scoring != SCORE_SOFTMAX_RENORM && scoring != SCORE_SOFTMAX_BIASED) return SPITE_BAD_ARG;
    if (scoring == SCORE_SOFTMAX_BIASED && !choice_bias) return SPITE_BAD_ARG;
    if (n_tokens < 0 || d <= 0 || n_experts < 1 || top_k < 1 || top_k > n_experts) return SPITE_BAD_ARG;
    if (n_experts > MAX_EXPERTS) return SPITE_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_tokens > 0) {
        // one pair of experts a block: measured faster than blocks that take several pairs and reuse
        // their tokens from the first-level cache (31 us against 40 and 53 us for 2048 tokens, 16 experts)
        const int per_block = EB;
        dim3 grid((n_tokens + TB - 1) / TB, (n_experts + per_block - 1) / per_block);
        if (grid.y > 65535) return SPITE_UNSUPPORTED;
        if (dtype == SPITE_DT_F32)
            SPITE_LAUNCH(route_logits_kernel<float>, grid, WARPS * 32, 0, st, (const float*)x, w_router, n_tokens, d,
                         n_experts, per_block, logits);
        else if (dtype == SPITE_DT_BF16)
            SPITE_LAUNCH(route_logits_kernel<__nv_bfloat16>, grid, WARPS * 32, 0, st, (const __nv_bfloat16*)x, w_router,
                         n_tokens, d, n_experts, per_block, logits);
        else
            return SPITE_BAD_ARG;
        if (cudaGetLastError() != cudaSuccess) return SPITE_LAUNCH_FAILED;
    }
    SPITE_LAUNCH(select_and_sort_kernel, top_k, 1024, 0, st, (const float*)logits, n_tokens, n_experts, top_k,
                 expert_ids, weights, offsets, sorted_rows, scoring, sorted_weights, choice_bias);
    return spite_launch_status();
}

namespace {

// Experts that return their input: out[t, :] (=|+=) sum over the choice slots whose expert id is `first_identity` or
// above of weights[slot][t] * x[t, :], the slots in ascending order.  With `accumulate` 0 every row of `out` is written
// (zeros where no such expert was chosen), so the kernel also starts the sum that the real experts then add to.
template <typename T>
__global__ void __launch_bounds__(256) moe_identity_kernel(const T* __restrict__ x, const int* __restrict__ expert_ids,
                                                           const float* __restrict__ weights, int n_tokens, int d, int top_k,
                                                           int first_identity, float* __restrict__ out, int accumulate) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    bool any = false;
    for (int s = 0; s < top_k; ++s)
        if (expert_ids[(size_t)s * n_tokens + t] >= first_identity) any = true;
    if (!any && accumulate) return;
    const T* in = x + (size_t)t * d;
    float* o = out + (size_t)t * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        // (the slots' terms are weights times the same element: their sum is the element times the sum of the weights,
        // added slot by slot so that one identity expert gives w * x exactly)
        float v = 0.f;
        if (any) {
            const float xv = to_f32(in[c]);
            for (int s = 0; s < top_k; ++s)
                if (expert_ids[(size_t)s * n_tokens + t] >= first_identity) v = fmaf(weights[(size_t)s * n_tokens + t], xv, v);
        }
        o[c] = accumulate ? o[c] + v : v;
    }
}

}  // namespace

SPITE_API int spite_moe_identity(int dtype, const void* x, const int* expert_ids, const float* weights, int n_tokens, int d,
                                 int top_k, int first_identity, float* out, int accumulate, void* stream) {
    if (!x || !expert_ids || !weights || !out) return SPITE_BAD_ARG;
    if (n_tokens < 0 || d <= 0 || top_k < 1 || first_identity < 0) return SPITE_BAD_ARG;
    if (dtype != SPITE_DT_F32 && dtype != SPITE_DT_BF16) return SPITE_BAD_ARG;
    if (n_tokens == 0) return SPITE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == SPITE_DT_F32)
        SPITE_LAUNCH(moe_identity_kernel<float>, n_tokens, threads, 0, st, (const float*)x, expert_ids, weights, n_tokens, d, top_k,
                     first_identity, out, accumulate);
    else
        SPITE_LAUNCH(moe_identity_kernel<__nv_bfloat16>, n_tokens, threads, 0, st, (const __nv_bfloat16*)x, expert_ids, weights,
                     n_tokens, d, top_k, first_identity, out, accumulate);
    return spite_launch_status();
}
