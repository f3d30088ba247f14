"""Grouped-query attention over the paged cache.

One part serves every attention layer: the window rule (all keys, the keys of
the query's chunk, the last W keys), the position encoding, the per-head norm of
q and k (after or before the rotation, with gains or without), the
temperature factor, a value size that differs from the key size, a sink in
the softmax (an extra term exp(sink) in the sum, with nothing behind it; one score for all heads or a learned
one per head), a bias that grows with the distance between query and key, a gate on every head's output (one
number a head, or one for every element of the concatenated heads), biases on the four projections, the
blending of the values with those of another layer, and keys and values that are not the layer's own but those
another layer cached are constructor parameters.

Formulas: crates/spite-models/src/llama/llama4.rs:126-207 (projections, rotation
then norm, temperature factor on layers without rotation, append to the cache,
attention, output projection added to the residual stream) and
crates/spite-compute/src/flash_attn.rs:111-156 (scores, mask, softmax, values).
"""
from __future__ import annotations

import math

import torch

from ..cache import FixedState, PagedKV, Window
from ..config.specs import ConfigError, PartSpec
from .base import Mixer, ParamSpec, QkNorm, build_part, register_mixer


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    graph_safe = True
    can_store = True
    kernel_libraries = ("gemm_simt", "attention", "attention_mma", "attention_rows", "attention_tc", "attention_decode")

    def __init__(self, ctx, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, window=("full", 0), qk_norm_eps=None, qk_norm_gain=False,
                 qk_norm_before_rotation=False, temperature_tuning=None, softmax_scale=None,
                 value_dim=None, sink_logit=None, head_sinks=False, distance_slopes=None, head_gate=False,
                 value_mix=None, bias=False, output_gate=False, kv_shared=False, conv_taps=None, score_softcap=None):
        """`head_dim` is the size of a query and a key head, `value_dim` that of a value head (default: the
        same).  `sink_logit`, if given, is the score of a sink: a term exp(sink) in every softmax's sum that adds
        nothing to the output, p_j = exp(s_j) / (exp(sink) + sum exp(s_j')); with `head_sinks` the score is a
        learned parameter per head (`sinks` [heads]).  `distance_slopes` (one number per head): slope_h * (i - j)
        is taken off the score of query position i and key position j.  `head_gate`: head h's output is multiplied by
        sigmoid(w_h . x), w the rows of `gate_proj` [heads, hidden], x the mixer's input.  `value_mix`: "source"
        marks the layer whose values of the step's tokens later layers blend in; "blend" makes this layer's
        values (1 - lam) v + lam v_source before they are cached, lam the scalar parameter `value_mix`.
        `bias`: the projections of q, k, v and the output projection add a bias each (`q_bias`, `k_bias`, `v_bias`,
        `o_bias`).  `output_gate`: the concatenated heads are multiplied element by element by sigmoid(W x), W the
        parameter `out_gate_proj` [heads * value size, hidden], x the mixer's input, before the output projection.
        `kv_shared`: the layer has no key and value projections; it reads the cache another layer of the run order
        writes (keys after that layer's rotation) with its own queries, window and everything else.
        `conv_taps` n: q, k and v pass a causal convolution over time of n taps per channel (`q_conv`, `k_conv`, `v_conv`
        [channels, n], the last column the current token's) directly behind their projections, before norm and
        rotation; a request's last n - 1 projected rows are kept in its state slot.  `score_softcap` c: a scaled score s
        becomes c tanh(s / c) before the softmax."""
        super().__init__(ctx)
        self.conv_taps = None if conv_taps is None else int(conv_taps)
        if self.conv_taps is not None and (self.conv_taps < 1 or self.conv_taps > 8):
            raise ConfigError(f"conv_taps {conv_taps} must lie in 1..8")
        if self.conv_taps is not None and kv_shared:
            raise ConfigError("a layer that reads another layer's keys and values keeps no convolution state of its own")
        self.score_softcap = None if score_softcap is None else float(score_softcap)
        if self.score_softcap is not None and not self.score_softcap > 0:
            raise ConfigError("score_softcap must be positive")
        self.has_bias, self.output_gate, self.kv_shared = bool(bias), bool(output_gate), bool(kv_shared)
        if self.kv_shared and value_mix:
            raise ConfigError("a layer that reads another layer's keys and values has no values to blend")
        if self.output_gate and head_gate:
            raise ConfigError("a gate per head and a gate per element exclude each other")
        if num_heads % num_kv_heads:
            raise ConfigError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads evenly")
        if head_dim < 1 or head_dim > 256:
            raise ConfigError(f"head_dim {head_dim} must lie in 1..256")
        self.d, self.nq, self.nkv = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.kd = int(head_dim)
        self.vd = int(value_dim) if value_dim else self.kd
        if self.vd < 1 or self.vd > 256:
            raise ConfigError(f"value_dim {self.vd} must lie in 1..256")
        self.sink_logit = None if sink_logit is None else float(sink_logit)
        self.has_head_sinks = bool(head_sinks)
        if self.has_head_sinks and self.sink_logit is not None:
            raise ConfigError("a sink is either one score for all heads or a learned one per head")
        if distance_slopes is not None and len(distance_slopes) != num_heads:
            raise ConfigError(f"{len(distance_slopes)} distance slopes for {num_heads} heads")
        self._slopes = None if distance_slopes is None else torch.tensor(
            [float(s) for s in distance_slopes], dtype=torch.float64).to(torch.float32).to(ctx.device)
        self.head_gate = bool(head_gate)
        if value_mix not in (None, "source", "blend"):
            raise ConfigError(f"value_mix {value_mix!r} is unknown (source, blend)")
        self.value_mix = value_mix
        self.head_sinks = self.value_lambda = None
        self.window = window if isinstance(window, Window) else Window(window[0], int(window[1]))
        self.position = build_part("position", position, ctx)
        # Keys and values share the cache's pages and the attention kernels' tiles, which have one row size.  Where
        # the two sizes differ it is the larger one, in bfloat16 rounded up to the tensor-core kernels' step of 16.  The projection
        # matrices get zero rows (and the output projection zero columns) for the padding, so the padded
        # elements are exact zeros: they add nothing to a score and come out of the attention as zeros.
        # A rotation or a per-head norm would have to know which elements of a row are padding: a layer
        # with either keeps its rows as they are.
        # (A rotation of the leading elements alone leaves the padding, which follows the key's last element, alone too.)
        rot = self.position.rotation()
        if rot is not None and (rot.rotary_dim or self.kd) > self.kd:
            raise ConfigError(f"{rot.rotary_dim} rotating elements in a head of {self.kd}")
        # (the per-head norm is told the key's own size and takes its mean over that)
        may_pad = rot is None or rot.rotary_dim is not None
        if self.kd % 2 and not may_pad:
            raise ConfigError(f"head_dim {head_dim} must be even where heads rotate or are normed")
        hd = max(self.kd, self.vd)
        step = 16 if self.vd != self.kd and ctx.dtype == torch.bfloat16 and hd <= 128 else 2
        self.hd = -(-hd // step) * step
        if self.hd != self.kd and not may_pad:
            raise ConfigError(f"a value size {self.vd} other than the key size {self.kd} cannot be combined "
                              f"with a rotation of the whole head")
        # only the attention kernels that these sizes can reach are compiled for the model
        libs = ["gemm_simt", "attention"]
        if ctx.dtype == torch.bfloat16 and self.hd % 16 == 0 and self.hd <= 128 and self.nq // self.nkv <= 16:
            libs += ["attention_mma", "attention_rows"]
            if self.hd in (64, 128):
                libs += ["attention_tc", "attention_decode"]
        self.kernel_libraries = tuple(libs)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.qk_norm_gain = bool(qk_norm_gain) and self.qk_norm_eps is not None
        self.qk_norm_before_rotation = bool(qk_norm_before_rotation)
        self.qk_norm = None if self.qk_norm_eps is None else QkNorm(self.qk_norm_eps, self.qk_norm_before_rotation)
        if temperature_tuning is not None:
            floor, scale = temperature_tuning
            if float(floor) != int(floor) or int(floor) < 1:
                raise ConfigError(f"temperature floor_scale {floor} must be a positive integer")
            temperature_tuning = (int(floor), float(scale))
        self.temperature = temperature_tuning
        self.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.kd)
        self.wqkv = self.wo = None

    def param_specs(self):
        d, nq, nkv, kd, vd = self.d, self.nq, self.nkv, self.kd, self.vd
        specs = {"q_proj": ParamSpec((nq * kd, d)), "o_proj": ParamSpec((d, nq * vd))}
        if not self.kv_shared:
            specs.update({"k_proj": ParamSpec((nkv * kd, d)), "v_proj": ParamSpec((nkv * vd, d))})
        if self.has_bias:
            specs.update({"q_bias": ParamSpec((nq * kd,)), "o_bias": ParamSpec((d,))})
            if not self.kv_shared:
                specs.update({"k_bias": ParamSpec((nkv * kd,)), "v_bias": ParamSpec((nkv * vd,))})
        if self.output_gate:
            specs["out_gate_proj"] = ParamSpec((nq * vd, d))
        if self.qk_norm_gain:
            specs.update({"q_norm": ParamSpec((kd,), "ones"), "k_norm": ParamSpec((kd,), "ones")})
        if self.has_head_sinks:
            specs["sinks"] = ParamSpec((nq,))
        if self.head_gate:
            specs["gate_proj"] = ParamSpec((nq, d))
        if self.value_mix:
            specs["value_mix"] = ParamSpec(())          # (the source layer's own is in the file too, and unused)
        if self.conv_taps is not None:
            specs.update({"q_conv": ParamSpec((nq * kd, self.conv_taps)), "k_conv": ParamSpec((nkv * kd, self.conv_taps)),
                          "v_conv": ParamSpec((nkv * vd, self.conv_taps))})
        return specs

    def _pad_heads(self, w, heads, size):
        """[heads * size, d] -> [heads * hd, d]: every head's rows followed by zero rows up to the cache's row size."""
        if size == self.hd:
            return w
        out = torch.zeros((heads, self.hd, w.shape[1]), dtype=w.dtype, device=w.device)
        out[:, :size] = w.view(heads, size, w.shape[1])
        return out.view(heads * self.hd, w.shape[1])

    def bind(self, params):
        dt = self.ctx.dtype
        # q, k and v rows in one matrix: one product per layer instead of three
        rows = [self._pad_heads(params["q_proj"].to(dt), self.nq, self.kd)]
        if not self.kv_shared:
            rows += [self._pad_heads(params["k_proj"].to(dt), self.nkv, self.kd),
                     self._pad_heads(params["v_proj"].to(dt), self.nkv, self.vd)]
        self.head_columns = sum(r.shape[0] for r in rows)       # the gates' columns of the product follow the heads'
        self.conv_w = None
        if self.conv_taps is not None:
            # one tap vector per column of the product, in the columns' order (zeros for the padding, which stays zero)
            self.conv_w = torch.cat([self._pad_heads(params["q_conv"].to(torch.float32), self.nq, self.kd),
                                     self._pad_heads(params["k_conv"].to(torch.float32), self.nkv, self.kd),
                                     self._pad_heads(params["v_conv"].to(torch.float32), self.nkv, self.vd)], 0).contiguous()
        self.qkv_bias = self.o_bias = None
        if self.has_bias:
            # added in float32 to the product's columns by the prepare kernel (zeros for the padding), and laid down
            # in the output buffer before the output projection adds to it
            def column(name, heads, size):
                return self._pad_heads(params[name].to(torch.float32).reshape(-1, 1), heads, size).reshape(-1)
            cols = [column("q_bias", self.nq, self.kd)]
            if not self.kv_shared:
                cols += [column("k_bias", self.nkv, self.kd), column("v_bias", self.nkv, self.vd)]
            self.qkv_bias = torch.cat(cols).contiguous()
            self.o_bias = params["o_bias"].to(torch.float32).contiguous()
        if self.output_gate:
            # a gate per element of the concatenated heads: its rows ride in the same product, laid out like the
            # attention's result (zero rows for the padding: they meet zeros there)
            rows.append(self._pad_heads(params["out_gate_proj"].to(dt), self.nq, self.vd))
        if self.head_gate:
            # the gates' rows ride in the same product: one more column per head, then zero rows up to a multiple of 8
            g = params["gate_proj"].to(dt)
            rows += [g, torch.zeros((-self.nq % 8, self.d), dtype=dt, device=g.device)]
        self.wqkv = torch.cat(rows, 0).contiguous()
        if self.has_head_sinks:
            self.head_sinks = params["sinks"].to(torch.float32).contiguous()
        if self.value_mix == "blend":
            self.value_lambda = float(params["value_mix"].to(torch.float32))
        # the output projection's columns, head by head, with zero columns for the padding
        self.wo = self._pad_heads(params["o_proj"].to(dt).t().contiguous(), self.nq, self.vd).t().contiguous()
        if self.qk_norm_gain:
            def gain(name):                                      # (zeros for the padding of a head)
                g = torch.zeros((self.hd,), dtype=torch.float32, device=params[name].device)
                g[:self.kd] = params[name].to(torch.float32)
                return g.contiguous()
            self.qk_norm = QkNorm(self.qk_norm_eps, self.qk_norm_before_rotation, gain("q_norm"), gain("k_norm"))

    def weight_bytes(self):
        return (self.wqkv.numel() + self.wo.numel()) * self.wqkv.element_size()

    def cache_request(self):
        state = None
        if self.conv_taps is not None and self.conv_taps > 1:
            state = FixedState(((self.conv_taps - 1) * (self.nq + 2 * self.nkv) * self.hd,), torch.float32)
        return PagedKV(self.window, self.nkv, self.hd), state

    def forward(self, x, h, batch, cache, accumulate=True):
        M = x.shape[0]
        k = self.k
        qkv = torch.empty((M, self.wqkv.shape[0]), dtype=x.dtype, device=x.device)
        if self.conv_w is None:
            k.linear(x, self.wqkv, qkv)
        else:
            # the projection's float32 sums pass the convolution over time; the gates' columns behind them pass unchanged
            proj = torch.empty((M, self.wqkv.shape[0]), dtype=torch.float32, device=x.device)
            k.linear(x, self.wqkv, proj)
            k.short_conv(proj, self.conv_w, qkv, batch, cache.state, channels=self.head_columns)
        q = torch.empty((M, self.nq * self.hd), dtype=x.dtype, device=x.device)
        extra = {}
        gates = None
        if self.head_gate:
            gates = extra["gates_out"] = torch.empty((M, self.nq), dtype=torch.float32, device=x.device)
        v_column = (self.nq + self.nkv) * self.hd
        if self.value_mix == "source":
            # the step's values as this layer projects them, for the layers that blend them in (the step keeps
            # the product's output alive until it ends)
            batch.shared["value_mix_source"] = (qkv, v_column, self.hd, self.nkv)
        elif self.value_mix == "blend":
            src = batch.shared.get("value_mix_source")
            if src is None or src[3] != self.nkv:
                raise ConfigError("a layer blends values in, but no layer before it in the run order is their source")
            extra["value_mix"] = (src[0], src[1], src[2], self.vd, self.value_lambda)
        if self.qkv_bias is not None:
            extra["bias"] = self.qkv_bias
        if self.qk_norm is not None and self.hd != self.kd:
            extra["norm_dim"] = self.kd
        if self.kv_shared:
            if cache.write:
                raise ConfigError("a layer without keys and values of its own was given a cache to write")
            extra["q_only"] = True
        k.qk_prepare(qkv, q, batch, cache, num_heads=self.nq, rotation=self.position.rotation(),
                     qk_norm=self.qk_norm, temperature=self.temperature, **extra)
        o = torch.empty_like(q)
        # keys and values of earlier positions were cached by earlier steps; this step's own were written by
        # the prepare kernel just before, which is what the attention kernel waits for
        more = {}
        if self.head_sinks is not None:
            more["head_sinks"] = self.head_sinks
        if self._slopes is not None:
            more["head_slopes"] = self._slopes
        if gates is not None:
            more["head_gates"] = gates
        if self.score_softcap is not None:
            more["score_softcap"] = self.score_softcap
        k.paged_attention(q, o, batch, cache, num_heads=self.nq, window=self.window,
                          softmax_scale=self.softmax_scale, cache_settled=True, sink_logit=self.sink_logit, **more)
        if self.output_gate:
            k.head_norm_gate(o, o, heads=self.nq, size=self.hd, gates=qkv, gate_column=self.head_columns)
        if self.o_bias is not None:
            k.fill_rows(h, self.o_bias, accumulate=accumulate)
            accumulate = True
        k.linear(o, self.wo, h, accumulate=accumulate)
