"""The contract between the layer parts and the kernels.

A `KernelSet` is bound to one activation type (bfloat16 or float32).  The
residual stream, norm gains, router weights, softmax statistics and logits are
float32 in both sets.  Parts call these methods and nothing else to touch the
device; a kernel set never learns which model or layer it serves.

Shapes use M for the tokens of the step, d for the model width, T for the
activation type.  All tensors are contiguous and live on the set's device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class KernelError(RuntimeError):
    """A kernel refused its arguments or could not be launched."""


class KernelTimeout(KernelError):
    """A kernel gave up a bounded wait and left its output incomplete: the results of the steps
    since the last check cannot be trusted (ExecutorError in crates/spite-executor/src/lib.rs:88-100
    is the counterpart: a typed error instead of wrong logits)."""


@dataclass
class Routing:
    """Result of `moe_route` for M tokens, E experts and k choices per token."""
    expert_ids: torch.Tensor     # [k, M] int32
    weights: torch.Tensor        # [k, M] float32, sigmoid of the chosen logits
    offsets: torch.Tensor        # [k, E + 1] int32: places of each expert's tokens in sorted_rows
    sorted_rows: torch.Tensor    # [k, M] int32: token indices ordered by expert, ascending within one
    logits: Optional[torch.Tensor] = None   # [M, E] float32 if asked for
    sorted_weights: Optional[torch.Tensor] = None   # [k, M] float32: weights[slot][sorted_rows[slot][i]] at place i


class KernelSet:
    """Interface; see `CudaKernels` for the product implementation."""

    dtype: torch.dtype
    device: torch.device

    def errors(self) -> dict:
        """{kernel library: code} for every library one of whose kernels gave up a bounded wait since
        the last call; reading clears.  Does not wait for the device: call it after a point at
        which the host has waited for the step's results."""
        return {}

    # ---- elementwise
    def embed(self, table, token_ids, out_h, *, scale=1.0, position_table=None, positions=None):
        """out_h[m, :] (float32) = table[token_ids[m], :] (T) * scale; with a `position_table` [P, d] (T)
        and `positions` [M] int32, + position_table[positions[m], :] (the factor applies to the token's row only)."""
        raise NotImplementedError

    def pack_pair(self, a, b, out, *, refill=None):
        """out[m, :] (T) = [a[m, :]; b[m, :]] for two float32 streams [M, d]; with `refill` [d] float32 every
        row of `a` becomes that vector afterwards (the stream is restarted for a product that adds into it)."""
        raise NotImplementedError

    def transform_logits(self, logits, *, scale=1.0, softcap=None):
        """In place: logits *= scale; then, with a cap, logits = cap * tanh(logits / cap)."""
        raise NotImplementedError

    def rms_norm(self, h, gain, eps, out, rows=None):
        """out[i, :] (T or float32) = h[r] * rsqrt(mean(h[r]^2) + eps) * gain, r = rows[i] if rows else i.
        h float32 [*, d], gain float32 [d]."""
        raise NotImplementedError

    def rms_norm_residual(self, y, gain, eps, mult, h, *, next_gain=None, next_out=None):
        """A sublayer's output is normed before it joins the residual stream:
        h[m, :] += mult * y[m, :] * rsqrt(mean(y[m]^2) + eps) * gain (y, h float32 [M, d]); with `next_out` [M, d]
        (T) also the norm the next sublayer reads, of the row just made: next_out = h * rsqrt(mean(h^2) + eps) * next_gain;
        `next_out` without `next_gain`: the row itself in next_out's type (the next sublayer reads the stream unnormed)."""
        raise NotImplementedError

    def cast_rows(self, h, out):
        """out (T) = h (float32), element by element: what a sublayer without a norm in front of it reads."""
        raise NotImplementedError

    def short_conv(self, x, w, out, batch, state, *, channels, activation=None, state_offset=0):
        """A short causal convolution over time on the first `channels` columns of a projection's float32 output x
        [M, >= channels + c]: out[t, ch] = act(sum_j w[ch, j] * x[t - taps + 1 + j, ch]) within each segment, w float32
        [channels, taps]; rows before a segment's first token come from the request's slot, state[slot, state_offset :
        state_offset + (taps - 1) * channels] (float32 [taps - 1, channels], oldest first; zeros at the start of a
        sequence), which then receives the sequence's last taps - 1 rows of x.  The c = out.shape[1] - channels columns behind
        the channels are passed on unchanged.  out [M, channels + c] is T or float32; `activation` None or "silu".
        With one tap nothing is carried and `state` may be None."""
        raise NotImplementedError

    def fill_rows(self, out, vec, *, accumulate=False):
        """out[m, :] (float32 [M, d]) = vec (float32 [d]), or += vec: a bias laid down for a product that adds to it."""
        raise NotImplementedError

    def head_norm_gate(self, x, out, *, heads, size, gates=None, gate_column=0, gain=None, eps=None, gate_activation="sigmoid"):
        """What stands between a mixer's heads and its output projection.  x [M, heads * size] (T, or float32: the
        result of a recurrence), out [M, heads * size] (T; may be x):
        out[m, h, j] = x[m, h, j] * r * gain[h * size + j] * sigmoid(gates[m, gate_column + h * size + j]) with
        r = rsqrt(mean_j x[m, h, :]^2 + eps) if `eps` is given (a norm of every head without a gain of its own), else 1;
        `gates` (a 2-D tensor of x's type, the gate columns of a wider product) and `gain` (float32) may be left out.
        `gate_activation` "silu": the factor is z * sigmoid(z) of the gate column z instead of sigmoid(z)."""
        raise NotImplementedError

    # ---- matrix products: y = x W^T with W [out, in]
    def linear(self, x, w, out, *, accumulate=False, row_scale=None, activation=None):
        """out[M, N] = x[M, K] @ w[N, K]^T.  `out` is T, or float32 (logits); with
        `accumulate` it is float32 and the product is added to it (residual stream).
        `row_scale` [M] float32 multiplies the product's rows.  `activation` (with an output of type T):
        "relu2": out = relu(s y)^2; "gelu_tanh": out = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), z = s y."""
        raise NotImplementedError

    def linear_swiglu(self, x, w_gate_up, out, *, row_scale=None):
        """out[M, F] (T) = silu(s g) * (s u) with g = x @ w[:F]^T, u = x @ w[F:]^T, s = row_scale or 1."""
        raise NotImplementedError

    def grouped_linear_swiglu(self, x, w_gate_up, sorted_rows, offsets, row_scale, out):
        """Row i of `out` [M, F] (sorted order) is the SwiGLU of token sorted_rows[i] through the
        expert whose range of `offsets` holds i; w_gate_up [E, 2F, K]; row_scale [M] by token."""
        raise NotImplementedError

    def grouped_linear_act(self, x, w_up, sorted_rows, offsets, row_scale, out, *, activation="relu2"):
        """Row i of `out` [M, F] (sorted order) is act(s * (x[sorted_rows[i]] @ w_up[e]^T)) for the expert e whose
        range of `offsets` holds i; w_up [E, F, K]; row_scale [M] by token; "relu2": act(y) = relu(y)^2."""
        raise NotImplementedError

    def grouped_linear_accumulate(self, a, w_down, sorted_rows, offsets, h, *, row_scale=None):
        """h[sorted_rows[i], :] (float32) += s_i * (a[i, :] @ w_down[expert of i]^T); w_down [E, d, F];
        `row_scale` [M] float32 by place i in the sorted order (s_i = 1 without it)."""
        raise NotImplementedError

    def grouped_linear_rows(self, a, w, rows, offsets, out, *, a_sorted=False):
        """out[rows[i], :N] (T) = a[rows[i], :K] @ w[g]^T for every place i of group g's range of `offsets`;
        a [R, lda >= K], w [G, N, K], out [R, ldc >= N].  Rows of `a` and `out` that no place names, and columns
        beyond K and N, are neither read nor written (a product per head: the rows are (token, head) pairs).
        With `a_sorted`, `a` lies in the list's order already: place i reads a[i, :K]."""
        raise NotImplementedError

    # ---- cache
    def clear_pages(self, kv, page_ids):
        """Zero the pages `page_ids` (a list of ints) of every cache of a group; `kv` is the group's tensor
        [caches, 2, pages, kv heads, page_size, head_dim].  The engine does this when it hands a page out,
        so that a request never multiplies a masked key's zero weight with what another request left there."""
        raise NotImplementedError

    # ---- attention
    def qk_prepare(self, qkv, q_out, batch, cache, *, num_heads, rotation, qk_norm, temperature,
                   value_mix=None, gates_out=None, bias=None, q_only=False, norm_dim=None):
        """Encode positions of q and k, normalise, scale q, append k and v to the cache.
        `bias` float32 [(nq + 2 nkv) hd]: added to the projection's columns before anything else.  `q_only`: a row of
        qkv holds the q heads alone (and `bias` theirs): the layer reads keys and values that another layer cached.
        qkv [M, >= (nq + 2 nkv) hd] T -> q_out [M, nq hd] T; `cache` is a `LayerCache`.
        `rotation`: a `parts.Rotation` or None; `qk_norm`: a `parts.QkNorm` or None (RMS norm of
        every q and k head, after the rotation unless it says before); `temperature`:
        (floor, scale) or None: q *= ln(floor((pos + 1) / floor) + 1) * scale + 1.
        `value_mix` = (other [M, *] T, column, head stride, value size, lam): element i < value size of kv head g's
        value becomes (1 - lam) v + lam * other[m, column + g * head stride + i] before it is cached.
        `gates_out` float32 [M, nq]: receives sigmoid(qkv[m, (nq + 2 nkv) hd + h]), the columns after the heads.
        `norm_dim`: a q or k head has this many elements and zeros behind them up to hd (a cache row wider than the key):
        the per-head norm takes its mean over them."""
        raise NotImplementedError

    def paged_attention(self, q, out, batch, cache, *, num_heads, window, softmax_scale, cache_settled=False,
                        sink_logit=None, head_sinks=None, head_slopes=None, head_gates=None, out_by_head=False,
                        score_softcap=None):
        """out[M, nq hd] = softmax(q K^T * scale over the visible cached keys) V.
        `score_softcap` c: a scaled score s becomes c * tanh(s / c) before anything else happens to it.
        `out_by_head`: the result is laid out head by head instead, out[nq, M, hd] (the order in which a product per
        head reads its rows).
        `sink_logit`: the softmax's denominator also holds exp(sink_logit), a key without a value;
        `head_sinks` float32 [nq]: the same with a score of its own for every head.
        `head_slopes` float32 [nq]: slope_h * (query position - key position) is taken off head h's scores.
        `head_gates` float32 [M, nq]: head h's output for token m is multiplied by head_gates[m, h].
        A cache with one plane (`cache.kv.shape[0] == 1`) holds keys only, and the value of a position is its key row.
        `cache_settled`: the caller promises that the cache rows of positions before each request's first
        token of this step were written by earlier steps (not by the one or two kernels launched just
        before this call), so a kernel may fetch them while the kernel before still runs."""
        raise NotImplementedError

    # ---- attention through latents
    def latent_prepare(self, down, cq_out, batch, cache, *, q_rank, kv_rank, rotation, q_gain, kv_gain, eps,
                       num_gates=0, gates_out=None):
        """One row of `down` (float32 [M, >= q_rank + kv_rank + rot + num_gates]) holds a token's query latent, its
        key/value latent, the key part that all heads share and the gate columns.  cq_out [M, q_rank] (T) =
        RMS norm of the query latent * q_gain; the cache row of the token's position becomes [RMS norm of the
        key/value latent * kv_gain; the shared part rotated by `rotation` (either pairing, times its amplitude);
        zeros up to the row's size]; gates_out [M, num_gates] float32 = sigmoid of the gate columns."""
        raise NotImplementedError

    def latent_queries(self, q, q_out, batch, *, num_heads, head_dim, kv_rank, rotation, rows_out, offsets_out,
                       sorted_out=None):
        """q [M, nq (head_dim + rot)] (T): every head's last `rot` elements are rotated (as in `latent_prepare`) into
        q_out[m, h, kv_rank : kv_rank + rot], and q_out's elements behind them become zero (q_out [M, nq, row] T; its
        first kv_rank elements are left for the product that follows).  Also lists the (token, head) rows head by
        head: rows_out[h M + m] = m nq + h, offsets_out[h] = h M (int32 [nq M] and [nq + 1]); `sorted_out` [nq M, head_dim]
        (T), if given, receives the heads' unrotated parts in that order: sorted_out[h M + m] = q[m, h, :head_dim]."""
        raise NotImplementedError

    # ---- recurrent mixers
    def mlstm_scan(self, proj, out, batch, state, *, heads, dim, vdim, gate_cap, q_scale, columns, i_bias, f_bias,
                   chunked=None):
        """Matrix memory with exponential gates, token by token, for every segment of the step from the state its
        request's slot holds (all zeros: the start of a sequence); the slot receives the state after the segment's
        last token.  proj float32 [M, *] holds, from the columns `columns` = (q, k, v, i, f) on, q and k
        [heads * dim], v [heads * vdim] and the gates' pre-activations [heads]; out float32 [M, heads * vdim];
        state float32 [slots, heads, `mlstm_state_size(dim, vdim)`].
        i = cap tanh((a + i_bias) / cap), f = logsigmoid(cap tanh((c + f_bias) / cap)), m' = max(f + m, i),
        S' = exp(f + m - m') S + exp(i - m') k v^T, n' alike with k, out = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6),
        q times `q_scale`.  All float32.  `chunked`: walk the segments 32 tokens at a time (the same sums in another
        order) instead of token by token; None leaves the choice to the kernel set."""
        raise NotImplementedError

    @staticmethod
    def mlstm_state_size(dim: int, vdim: int) -> int:
        """Floats of one head's state: S [dim, vdim], then one copy of (n [dim], m) for every 32 value columns, each
        rounded up to a multiple of four floats."""
        return dim * vdim + -(-vdim // 32) * (-(-(dim + 1) // 4) * 4)

    def delta_scan(self, x, out, batch, state, *, heads, kv_heads, dim, vdim, columns, a_log, dt_bias, q_scale,
                   unit_eps=1e-6, state_offset=0, split_rows=None):
        """The gated delta rule, token by token, for every segment of the step from the matrix its request's slot holds
        (zeros: the start of a sequence); the slot receives the matrix after the segment's last token.  x float32 [M, *]
        holds, from the columns `columns` = (q, k, v, b, a) on, q and k [kv_heads * dim], v [heads * vdim] and two
        numbers a head; out float32 [M, heads * vdim]; state float32 [slots, *], head h's S [dim, vdim] row-major at
        state[slot, state_offset + h * dim * vdim].  Head h reads q/k head h // (heads / kv_heads).
        k <- k / sqrt(|k|^2 + unit_eps), q <- q / sqrt(|q|^2 + unit_eps) * q_scale, beta = sigmoid(b),
        g = exp(-exp(a_log[h]) * softplus(a + dt_bias[h])); S <- g S; u = beta (v - S^T k); S <- S + k u^T; out = S^T q.
        All float32.  `split_rows`: more lanes share a value column's key rows (the same sums in another order; for steps
        with long segments); None leaves the choice to the kernel set."""
        raise NotImplementedError

    # ---- mixture of experts
    def moe_identity(self, x, routing, first_identity, out, *, accumulate=True):
        """Experts that return their input: out[m, :] (float32) (+)= sum over the choice slots s whose expert id
        routing.expert_ids[s, m] >= first_identity of routing.weights[s, m] * x[m, :] (x is T).  Without `accumulate`
        every row of out is written (zeros where no such expert was chosen)."""
        raise NotImplementedError

    def moe_route(self, x, w_router, top_k, want_logits=False, scoring="sigmoid", choice_bias=None) -> Routing:
        """Router logits in float32, the `top_k` largest per token (equal ones: the lower expert first), the
        tokens sorted by expert for every choice slot.  `scoring` "sigmoid": the weight of a choice is the sigmoid
        of its logit; "softmax_renorm": its share of the softmax over all experts, divided by the sum of the
        chosen shares (+ 1e-20); `sorted_weights` is filled for it.  "softmax_biased": the experts are ordered by their
        softmax share plus `choice_bias` (float32 [E]), and the weight of a choice is its share alone (not renormalised);
        `sorted_weights` is filled."""
        raise NotImplementedError

    # ---- sampling
    def argmax(self, logits):
        """[R] int32: index of the maximum of each row, the highest index among equals."""
        raise NotImplementedError

    def sample(self, logits, *, temperature, top_k, top_p, min_p, repetition_penalty,
               context, context_offsets, rng_state):
        """[R] int32 tokens; `rng_state` [R] int64 is advanced in place for rows that draw."""
        raise NotImplementedError
