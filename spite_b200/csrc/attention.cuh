// Argument blocks of the attention kernels.
#pragma once
#include "common.cuh"

#define SPITE_WINDOW_FULL 0      // keys 0..pos
#define SPITE_WINDOW_CHUNK 1     // keys of the query's chunk: floor(pos/size)*size .. pos
#define SPITE_WINDOW_SLIDING 2   // the last `size` keys: max(0, pos-size+1) .. pos

// The tokens of one step, flattened.  Token t belongs to segment seg_of_token[t]
// (one segment per request in the step) and sits at absolute position positions[t].
// block_table[seg * table_width + p / page_size] is the page that holds position p.
struct StepTokens {
    const int* positions;
    const int* seg_of_token;
    const int* block_table;
    int table_width;
    int n_tokens;
};

// One cache: keys at kv, values at kv + v_offset (elements); a page holds, for every
// kv head, page_size rows of head_dim elements: [pages][kv heads][page_size][head_dim].
// v_offset 0: the cache has keys only and a position's value is its key row.
struct PagedCache {
    void* kv;
    long long v_offset;
    int n_pages;
    int page_size;
    int num_kv_heads;
    int head_dim;
};

#define SPITE_PAIR_NEIGHBOURS 0   // pair i of a head is elements (2i, 2i+1)
#define SPITE_PAIR_HALVES 1       // pair i is elements (i, i + rotary_dim/2)

struct QkPrepareParams {
    const void* qkv;            // [tokens, (nq + 2 nkv) * head_dim]: q heads, k heads, v heads
    void* q_out;                // [tokens, nq * head_dim]
    const float* inv_freq;      // [rotary_dim / 2] rotation frequencies, or null: no rotation
    const float* q_gain;        // [head_dim] gain of the norm of q heads, or null (weightless)
    const float* k_gain;        // [head_dim] the same for k heads
    float qk_norm_eps;          // > 0: RMS norm of every q and k head
    int norm_before_rotation;   // the norm runs before the rotation instead of after it
    int pairing;                // SPITE_PAIR_*
    int rotary_dim;             // the first rotary_dim elements of a head rotate (even, <= head_dim)
    int temperature_floor;      // > 0: q *= ln(floor((pos+1)/floor) + 1) * temperature_scale + 1
    float temperature_scale;
    int num_heads;
    int write_cache;            // append k and v to the cache
    long long qkv_stride;       // elements between two tokens' rows of qkv (>= (nq + 2 nkv) * head_dim; 0: exactly that)
    float rot_amplitude;        // cos and sin of the rotation are multiplied by this (1, or 0 for unset: a pure rotation)
    // value blending: element i < v_mix_dim of kv head g's value becomes (1 - v_mix) v + v_mix * v_other[t * v_other_stride +
    // g * v_other_head + i] before it is cached (v_other null: no blending)
    const void* v_other;
    long long v_other_stride;
    int v_other_head;
    int v_mix_dim;
    float v_mix;
    // gates_out[t * nq + h] = sigmoid(qkv[t * qkv_stride + (nq + 2 nkv) * head_dim + h]) (null: no gate columns)
    float* gates_out;
    // bias[column] (float32, the columns of a token's row of qkv up to the last head's) is added to the projection's
    // output before anything else happens to it (null: none)
    const float* bias;
    int q_only;                 // the rows of qkv hold the q heads alone: this layer reads keys and values that another layer cached
    int norm_dim;               // > 0: a q or k head has this many elements (the rest of its head_dim are padding zeros): the
                                // per-head norm's mean is taken over them (0: over head_dim)
};

struct AttentionParams {
    const void* q;              // [tokens, nq * head_dim]
    void* out;                  // [tokens, nq * head_dim]
    int num_heads;
    int window_kind;
    int window_size;
    float softmax_scale;
    int has_sink;               // the softmax's denominator also holds exp(sink_logit): a key every query sees
    float sink_logit;           // and that adds nothing to the output (a score of 0 puts exp(0) = 1 into the sum)
    const float* head_sinks;    // [num_heads] or null: with has_sink, head h's sink has the score head_sinks[h] instead
    const float* head_slopes;   // [num_heads] or null: head_slopes[h] * (query position - key position) is taken off a score
    const float* head_gates;    // [tokens, num_heads] or null: head h's output of token t is multiplied by head_gates[t * nq + h]
    int out_by_head_tokens;     // 0: out is [tokens, num_heads, head_dim]; n > 0: out is [num_heads, n, head_dim], head by head
                                // (n the tokens of the step), the order in which a product per head reads its rows
    float score_softcap;        // > 0: a scaled score s becomes cap * tanh(s / cap) before bias, mask and softmax
};

// Where the output row of (token, head) starts, in rows of head_dim elements.
__device__ __forceinline__ size_t out_row_of(const AttentionParams& p, int token, int head) {
    return p.out_by_head_tokens > 0 ? (size_t)head * p.out_by_head_tokens + token : (size_t)token * p.num_heads + head;
}

// The score of head `head`'s sink (only meaningful with has_sink).
__device__ __forceinline__ float sink_of(const AttentionParams& p, int head) {
    return p.head_sinks ? p.head_sinks[head] : p.sink_logit;
}
// What is taken off the score of a key `distance` positions before the query.
__device__ __forceinline__ float slope_of(const AttentionParams& p, int head) {
    return p.head_slopes ? p.head_slopes[head] : 0.f;
}
// A scaled score squashed into (-cap, cap), or itself without a cap.  The tensor-core kernels are compiled in both
// forms (CAP): with the choice made per score at run time, the decode kernel took a tenth longer without any cap.
__device__ __forceinline__ float capped(const AttentionParams& p, float s) {
    return p.score_softcap > 0.f ? p.score_softcap * tanhf(s / p.score_softcap) : s;
}
template <bool CAP> __device__ __forceinline__ float capped_if(const AttentionParams& p, float s) {
    if constexpr (CAP) return p.score_softcap * tanhf(s / p.score_softcap);
    else return s;
}
// The factor on a finished output row.
__device__ __forceinline__ float gate_of(const AttentionParams& p, int token, int head) {
    return p.head_gates ? p.head_gates[(size_t)token * p.num_heads + head] : 1.f;
}

// The sink folded into a finished softmax state: `m` and `l` are the maximum and the sum of exp(s - m) over the
// real keys (natural-log units).  Afterwards l is the whole denominator relative to max(m, sink); the return
// value is the factor by which the accumulated values shrink to the same reference.
__device__ __forceinline__ float fold_sink(const AttentionParams& p, int head, float m, float& l) {
    if (!p.has_sink) return 1.f;
    const float sink = sink_of(p, head);
    const float m2 = fmaxf(m, sink);
    const float f = (m == -INFINITY) ? 0.f : expf(m - m2);
    l = l * f + expf(sink - m2);
    return f;
}

// What the tensor-core attention kernels need beyond the above.  Two kernels share a step:
// segments of few tokens (decode) go to the one that splits the keys among blocks, segments
// of many tokens (prompt portions) to the one that gives every warp its own rows; each kernel
// serves the segments whose token count lies in [seg_min_tokens, seg_max_tokens].
struct AttnMmaExtra {
    const int* cu_seqlens;       // [segments + 1]
    float* o_part;               // [tokens, heads, splits, head_dim]   (splits > 1)
    float* ml_part;              // [tokens, heads, splits, 2]          running maximum, sum
    int n_segments;
    int tokens_per_block;        // tokens whose (token, head) rows fill one block
    int n_splits;
    int seg_min_tokens;
    int seg_max_tokens;
};

// The same for the decode kernel whose last-arriving block merges the key splits itself.
struct AttnDecodeExtra {
    const int* cu_seqlens;       // [segments + 1]
    float* partial;              // [blocks, kv heads, splits, 16, head_dim + 4]   (splits > 1)
    int* tickets;                // [blocks, kv heads], zero between launches      (splits > 1)
    int n_segments;
    int tokens_per_block;
    int n_splits;
    int seg_min_tokens;
    int seg_max_tokens;
    int cache_settled;           // the cache rows of positions before each request's first token of this step were
                                 // written at least two launches ago on this stream: they may be read before the wait
};

__device__ __forceinline__ int window_lowest(int kind, int size, int pos) {
    if (kind == SPITE_WINDOW_CHUNK) return (pos / size) * size;
    if (kind == SPITE_WINDOW_SLIDING) return max(0, pos - size + 1);
    return 0;
}
