"""Matrix memory with exponential gates (the mLSTM cell of xLSTM) as a mixer.

Per head a matrix S [dim, vdim], a vector n [dim] and a running maximum m, all zero at the start of a sequence
and carried from token to token in float32 in the request's state slot:

    q = W_q x * q_scale,  k = W_k x,  v = W_v x                                (heads x dim, heads x vdim)
    i = cap tanh((W_i x + b_i) / cap),  f = logsigmoid(cap tanh((W_f x + b_f) / cap))      (one number a head)
    m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' = exp(f + m - m') n + exp(i - m') k
    o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
    out = W_o [ (o_h / rms(o_h)) for every head, concatenated, * gain * sigmoid(W_g x) ]

One product makes q, k, v, the gate's columns and the two gates' pre-activations as float32 sums; the scan walks
every segment of the step from its slot's state (token by token in decode steps, 32 tokens at a time where the step
has prompt portions: the same recurrence unrolled over a chunk, see `csrc/recurrent.cu`); one kernel norms the heads
and applies gain and gate; the output projection adds into (or fills) the float32 stream.
"""
from __future__ import annotations

import torch

from ..cache import FixedState
from ..config.specs import ConfigError
from ..kernels.api import KernelSet
from .base import Mixer, ParamSpec, register_mixer


@register_mixer("mlstm")
class MatrixLstm(Mixer):
    graph_safe = True
    can_store = True
    kernel_libraries = ("gemm_simt", "recurrent")

    def __init__(self, ctx, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, gate_cap: float,
                 norm_eps: float, q_scale: float | None = None):
        """`head_dim`: size of a head's q and k; `value_dim`: of its v and its output; `gate_cap`: the gates'
        pre-activations are squashed to cap tanh(z / cap); `norm_eps`: of the heads' norm; `q_scale`: factor on q
        (default head_dim^-1/2)."""
        super().__init__(ctx)
        self.d, self.H, self.kd, self.vd = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        if min(self.d, self.H, self.kd, self.vd) < 1:
            raise ConfigError("mlstm: sizes must be positive")
        if self.kd > 512:
            raise ConfigError(f"mlstm: head_dim {self.kd} exceeds the scan kernel's 512")
        if not float(gate_cap) > 0 or not float(norm_eps) > 0:
            raise ConfigError("mlstm: gate_cap and norm_eps must be positive")
        self.cap, self.eps = float(gate_cap), float(norm_eps)
        self.q_scale = float(q_scale) if q_scale is not None else self.kd ** -0.5
        H, kd, vd = self.H, self.kd, self.vd
        # columns of the one product: q, k, v, the output gate, the input gates, the forget gates (then padding)
        self.columns = (0, H * kd, 2 * H * kd, 2 * H * kd + 2 * H * vd, 2 * H * kd + 2 * H * vd + H)
        self.gate_column = 2 * H * kd + H * vd
        self.n_columns = -(-(2 * H * kd + 2 * H * vd + 2 * H) // 8) * 8
        self.w_in = self.w_out = self.gain = self.i_bias = self.f_bias = None

    def param_specs(self):
        d, H, kd, vd = self.d, self.H, self.kd, self.vd
        return {"q_proj": ParamSpec((H * kd, d)), "k_proj": ParamSpec((H * kd, d)), "v_proj": ParamSpec((H * vd, d)),
                "gate_proj": ParamSpec((H * vd, d)), "o_proj": ParamSpec((d, H * vd)), "norm": ParamSpec((H * vd,), "ones"),
                "igate_proj": ParamSpec((H, d)), "igate_bias": ParamSpec((H,)),
                "fgate_proj": ParamSpec((H, d)), "fgate_bias": ParamSpec((H,))}

    def bind(self, params):
        dt = self.ctx.dtype
        rows = [params[n].to(dt) for n in ("q_proj", "k_proj", "v_proj", "gate_proj", "igate_proj", "fgate_proj")]
        have = sum(r.shape[0] for r in rows)
        rows.append(torch.zeros((self.n_columns - have, self.d), dtype=dt, device=rows[0].device))
        self.w_in = torch.cat(rows, 0).contiguous()
        self.w_out = params["o_proj"].to(dt).contiguous()
        self.gain = params["norm"].to(torch.float32).contiguous()
        self.i_bias = params["igate_bias"].to(torch.float32).contiguous()
        self.f_bias = params["fgate_bias"].to(torch.float32).contiguous()

    def weight_bytes(self):
        return (self.w_in.numel() + self.w_out.numel()) * self.w_in.element_size()

    def cache_request(self):
        return None, FixedState((self.H, KernelSet.mlstm_state_size(self.kd, self.vd)), torch.float32)

    def forward(self, x, h, batch, cache, accumulate=True):
        k = self.k
        M = x.shape[0]
        proj = torch.empty((M, self.n_columns), dtype=torch.float32, device=x.device)
        k.linear(x, self.w_in, proj)                              # float32 sums: nothing that enters the recurrence is rounded
        o = torch.empty((M, self.H * self.vd), dtype=torch.float32, device=x.device)
        q, kk, v, i, f = self.columns
        k.mlstm_scan(proj, o, batch, cache.state, heads=self.H, dim=self.kd, vdim=self.vd, gate_cap=self.cap,
                     q_scale=self.q_scale, columns=(q, kk, v, i, f), i_bias=self.i_bias, f_bias=self.f_bias)
        a = torch.empty((M, self.H * self.vd), dtype=x.dtype, device=x.device)
        k.head_norm_gate(o, a, heads=self.H, size=self.vd, gates=proj, gate_column=self.gate_column, gain=self.gain,
                         eps=self.eps)
        k.linear(a, self.w_out, h, accumulate=accumulate)
