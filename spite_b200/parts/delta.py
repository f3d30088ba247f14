"""The gated delta rule as a mixer: a matrix per head that decays, is corrected towards the value along the key, and is
read by the query.

Per head a matrix S [dim, vdim], zero at the start of a sequence, carried from token to token in float32 in the
request's state slot:

    q = silu(conv(W_q x)),  k = silu(conv(W_k x))        (kv_heads x dim)        v = silu(conv(W_v x))   (heads x vdim)
    q <- q / sqrt(|q|^2 + 1e-6) * q_scale,   k <- k / sqrt(|k|^2 + 1e-6)          (per head; q_scale default dim^-1/2)
    beta = sigmoid(W_b x),   g = exp(-exp(A_log) * softplus(W_a x + dt_bias))     (one number a head each)
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q               (the read-out sees the token's own write)
    out = W_o [ o_h / rms(o_h) * gain * silu(W_g x)_h  for every head, concatenated ]

`conv` is a causal convolution over time of `conv_taps` taps per channel; the last taps - 1 projected rows of a
sequence live in the slot beside the matrices.  Head h reads q/k head h // (heads / kv_heads).

One product makes q, k, v, the output gate's columns and the two numbers a head as float32 sums; `short_conv` passes
q, k, v through the convolution and silu (the other columns unchanged); `delta_scan` walks every segment of the step
from its slot's matrices (unit vectors, beta and the decay are computed there, in float32); `head_norm_gate` norms
the heads and applies gain and gate; the output projection adds into (or fills) the float32 stream.
"""
from __future__ import annotations

import torch

from ..cache import FixedState
from ..config.specs import ConfigError
from .base import Mixer, ParamSpec, register_mixer


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    graph_safe = True
    can_store = True
    kernel_libraries = ("gemm_simt", "delta")

    def __init__(self, ctx, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 conv_taps: int, norm_eps: float, q_scale: float | None = None, unit_eps: float = 1e-6):
        """`num_heads` value heads on `num_kv_heads` query/key heads; `head_dim`: size of a q and k head, `value_dim`: of
        a v head and of a head's output; `conv_taps`: taps of the convolution over time; `norm_eps`: of the heads'
        norm; `unit_eps`: inside the root that makes q and k unit vectors."""
        super().__init__(ctx)
        self.d, self.H, self.G = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.kd, self.vd, self.taps = int(head_dim), int(value_dim), int(conv_taps)
        if min(self.d, self.H, self.G, self.kd, self.vd) < 1 or self.H % self.G:
            raise ConfigError("gated_delta: sizes must be positive and the heads a multiple of the kv heads")
        if self.kd > 512:
            raise ConfigError(f"gated_delta: head_dim {self.kd} exceeds the scan kernel's 512")
        if not 1 <= self.taps <= 8:
            raise ConfigError(f"gated_delta: conv_taps {conv_taps} must lie in 1..8")
        if not float(norm_eps) > 0 or not float(unit_eps) >= 0:
            raise ConfigError("gated_delta: norm_eps must be positive")
        self.eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.q_scale = float(q_scale) if q_scale is not None else self.kd ** -0.5
        H, G, kd, vd = self.H, self.G, self.kd, self.vd
        # columns of the one product: q, k, v (the convolution's channels), the output gate, b, a (then padding)
        self.channels = 2 * G * kd + H * vd
        self.columns = (0, G * kd, 2 * G * kd, self.channels + H * vd, self.channels + H * vd + H)
        self.gate_column = self.channels
        self.n_columns = -(-(self.channels + H * vd + 2 * H) // 8) * 8
        self.state_matrices = H * kd * vd
        self.w_in = self.w_out = self.conv_w = self.gain = self.a_log = self.dt_bias = None

    def param_specs(self):
        d, H, G, kd, vd, n = self.d, self.H, self.G, self.kd, self.vd, self.taps
        return {"q_proj": ParamSpec((G * kd, d)), "k_proj": ParamSpec((G * kd, d)), "v_proj": ParamSpec((H * vd, d)),
                "q_conv": ParamSpec((G * kd, n)), "k_conv": ParamSpec((G * kd, n)), "v_conv": ParamSpec((H * vd, n)),
                "beta_proj": ParamSpec((H, d)), "decay_proj": ParamSpec((H, d)), "a_log": ParamSpec((H,)),
                "dt_bias": ParamSpec((H,)), "gate_proj": ParamSpec((H * vd, d)), "norm": ParamSpec((vd,), "ones"),
                "o_proj": ParamSpec((d, H * vd))}

    def bind(self, params):
        dt = self.ctx.dtype
        rows = [params[n].to(dt) for n in ("q_proj", "k_proj", "v_proj", "gate_proj", "beta_proj", "decay_proj")]
        have = sum(r.shape[0] for r in rows)
        rows.append(torch.zeros((self.n_columns - have, self.d), dtype=dt, device=rows[0].device))
        self.w_in = torch.cat(rows, 0).contiguous()
        self.w_out = params["o_proj"].to(dt).contiguous()
        self.conv_w = torch.cat([params[n].to(torch.float32) for n in ("q_conv", "k_conv", "v_conv")], 0).contiguous()
        self.gain = params["norm"].to(torch.float32).repeat(self.H).contiguous()      # one gain vector, shared by the heads
        self.a_log = params["a_log"].to(torch.float32).contiguous()
        self.dt_bias = params["dt_bias"].to(torch.float32).contiguous()

    def weight_bytes(self):
        return (self.w_in.numel() + self.w_out.numel()) * self.w_in.element_size() + self.conv_w.numel() * 4

    def cache_request(self):
        # the heads' matrices, then the convolution's rows
        return None, FixedState((self.state_matrices + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, h, batch, cache, accumulate=True):
        k = self.k
        M = x.shape[0]
        proj = torch.empty((M, self.n_columns), dtype=torch.float32, device=x.device)
        k.linear(x, self.w_in, proj)                              # float32 sums: nothing that enters the recurrence is rounded
        u = torch.empty_like(proj)
        k.short_conv(proj, self.conv_w, u, batch, cache.state, channels=self.channels, activation="silu",
                     state_offset=self.state_matrices)
        o = torch.empty((M, self.H * self.vd), dtype=torch.float32, device=x.device)
        k.delta_scan(u, o, batch, cache.state, heads=self.H, kv_heads=self.G, dim=self.kd, vdim=self.vd,
                     columns=self.columns, a_log=self.a_log, dt_bias=self.dt_bias, q_scale=self.q_scale,
                     unit_eps=self.unit_eps)
        a = torch.empty((M, self.H * self.vd), dtype=x.dtype, device=x.device)
        k.head_norm_gate(o, a, heads=self.H, size=self.vd, gates=u, gate_column=self.gate_column, gain=self.gain,
                         eps=self.eps, gate_activation="silu")
        k.linear(a, self.w_out, h, accumulate=accumulate)
