"""Attention through low-rank latents over the paged cache.

A token's keys and values of all heads are functions of one short vector, the latent c = norm(W_dkv x)
(`kv_rank` elements), plus one rotated key part k_r (`rotary_dim` elements) that every head shares:

    k_h = [W_uk,h c ; k_r]      v_h = W_uv,h c      q_h = [q_n,h ; q_r,h] = W_uq norm(W_dq x), q_r rotated

Only [c ; k_r] is cached, one row per position (a cache of one kv head and one plane: the value of a
position is its key row).  The heads' own matrices move to the query's side, where they are applied to the
step's tokens only:

    score_h(i, j) = (W_uk,h^T q_n,h(i)) . c(j) + q_r,h(i) . k_r(j)
    out_h(i)      = W_uv,h sum_j p_h(i, j) c(j)

so the attention kernels see `num_heads` query heads on one key head whose rows are [c ; k_r], and the products
with W_uk,h^T before and W_uv,h after them are products per head over the (token, head) rows.  The score's scale
is a parameter, and so is the window (every earlier position, the query's chunk, or the last W positions).  An
optional gate multiplies head h's output by sigmoid(w_h . x); it is applied to the attention's result before W_uv,h,
which is the same product.  An optional learned sink per head adds exp(sink_h) to the softmax's sum.

Steps of `forward`: one product for W_dq, W_dkv and the gates' rows (float32 sums kept); `latent_prepare` (both
norms in float32, the rotation of k_r, the cache row, the gates); W_uq; `latent_queries` (rotation of q_r into
the query rows, the unrotated parts laid out head by head) and the product per head with W_uk^T; attention, its
result laid out head by head; the product per head with W_uv; W_o into the residual stream.
"""
from __future__ import annotations

import torch

from ..cache import PagedKV, Window
from ..config.specs import ConfigError, PartSpec
from .base import Mixer, ParamSpec, build_part, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True
    can_store = True

    def __init__(self, ctx, hidden_size: int, num_heads: int, head_dim: int, rotary_dim: int, value_dim: int,
                 q_rank: int, kv_rank: int, softmax_scale: float, norm_eps: float, position: PartSpec,
                 head_gate: bool = False, window=("full", 0), head_sinks: bool = False):
        """`head_dim` is the unrotated part of a query/key head, `rotary_dim` the rotated part, `value_dim` a value
        head; `q_rank` and `kv_rank` are the sizes of the two latents, both RMS-normed (gains `q_latent_norm`,
        `kv_latent_norm`, eps `norm_eps`).  `position` must rotate exactly `rotary_dim` elements (either pairing).
        `window`: which earlier positions a query sees.  `head_sinks`: a learned score per head (`sinks` [heads]) whose
        exponential joins the softmax's denominator and nothing else."""
        super().__init__(ctx)
        self.d, self.nq = int(hidden_size), int(num_heads)
        self.dn, self.dr, self.dv = int(head_dim), int(rotary_dim), int(value_dim)
        self.rq, self.rkv = int(q_rank), int(kv_rank)
        if min(self.nq, self.dn, self.dr, self.dv, self.rq, self.rkv) < 1 or self.dr % 2:
            raise ConfigError("latent attention needs positive sizes and an even rotary_dim")
        self.softmax_scale, self.eps = float(softmax_scale), float(norm_eps)
        self.head_gate = bool(head_gate)
        self.has_head_sinks = bool(head_sinks)
        self.window = window if isinstance(window, Window) else Window(window[0], int(window[1]))
        self.position = build_part("position", position, ctx)
        rot = self.position.rotation()
        if rot is None or (rot.rotary_dim or self.dr) != self.dr or 2 * rot.inv_freq.numel() != self.dr:
            raise ConfigError(f"latent attention needs a rotation over exactly its {self.dr} rotating elements")
        # a cache row is [latent ; shared key part], in bfloat16 rounded up to the tensor-core kernels' step of 16
        # (the padding is zeros on both sides of every score); the general kernels take even sizes
        row = self.rkv + self.dr
        step = 16 if ctx.dtype == torch.bfloat16 and row <= 128 else 2
        self.row = -(-row // step) * step
        if self.row > 640:
            raise ConfigError(f"a latent row of {row} elements exceeds the 640 that the attention kernels take")
        libs = ["gemm_simt", "attention", "latent"]
        if ctx.dtype == torch.bfloat16 and self.row % 16 == 0 and self.row <= 128 and self.nq <= 16:
            libs += ["attention_mma", "attention_rows"]
            if self.row in (64, 128):
                libs += ["attention_tc", "attention_decode"]
        self.kernel_libraries = tuple(libs)
        self.down_cols = self.rq + self.rkv + self.dr + (self.nq if self.head_gate else 0)
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.wo = self.q_gain = self.kv_gain = self.sinks = None

    def param_specs(self):
        d, nq = self.d, self.nq
        specs = {"q_down": ParamSpec((self.rq, d)), "q_latent_norm": ParamSpec((self.rq,), "ones"),
                 "q_up": ParamSpec((nq * (self.dn + self.dr), self.rq)),
                 "kv_down": ParamSpec((self.rkv + self.dr, d)), "kv_latent_norm": ParamSpec((self.rkv,), "ones"),
                 "k_up": ParamSpec((nq * self.dn, self.rkv)), "v_up": ParamSpec((nq * self.dv, self.rkv)),
                 "o_proj": ParamSpec((d, nq * self.dv))}
        if self.head_gate:
            specs["gate_proj"] = ParamSpec((nq, d))
        if self.has_head_sinks:
            specs["sinks"] = ParamSpec((nq,))
        return specs

    def bind(self, params):
        dt = self.ctx.dtype
        rows = [params["q_down"].to(dt), params["kv_down"].to(dt)]
        if self.head_gate:
            rows.append(params["gate_proj"].to(dt))
        pad = -self.down_cols % 8
        if pad:
            rows.append(torch.zeros((pad, self.d), dtype=dt, device=rows[0].device))
        self.w_down = torch.cat(rows, 0).contiguous()          # one product: both latents, the shared key part, the gates
        self.w_uq = params["q_up"].to(dt).contiguous()
        # W_uk,h is [head_dim, kv_rank]; the query's side needs its transpose as an [out, in] matrix per head
        self.w_uk_t = params["k_up"].to(dt).view(self.nq, self.dn, self.rkv).transpose(1, 2).contiguous()
        self.w_uv = params["v_up"].to(dt).view(self.nq, self.dv, self.rkv).contiguous()
        self.wo = params["o_proj"].to(dt).contiguous()
        self.q_gain = params["q_latent_norm"].to(torch.float32).contiguous()
        self.kv_gain = params["kv_latent_norm"].to(torch.float32).contiguous()
        if self.has_head_sinks:
            self.sinks = params["sinks"].to(torch.float32).contiguous()

    def weight_bytes(self):
        n = sum(t.numel() for t in (self.w_down, self.w_uq, self.w_uk_t, self.w_uv, self.wo))
        return n * self.wo.element_size() + (self.q_gain.numel() + self.kv_gain.numel()) * 4

    def cache_request(self):
        return PagedKV(self.window, 1, self.row, planes=1), None

    def forward(self, x, h, batch, cache, accumulate=True):
        M, k, dev = x.shape[0], self.k, x.device
        nq, row = self.nq, self.row
        down = torch.empty((M, self.w_down.shape[0]), dtype=torch.float32, device=dev)
        k.linear(x, self.w_down, down)
        cq = torch.empty((M, self.rq), dtype=x.dtype, device=dev)
        gates = torch.empty((M, nq), dtype=torch.float32, device=dev) if self.head_gate else None
        rotation = self.position.rotation()
        k.latent_prepare(down, cq, batch, cache, q_rank=self.rq, kv_rank=self.rkv, rotation=rotation,
                         q_gain=self.q_gain, kv_gain=self.kv_gain, eps=self.eps,
                         num_gates=nq if self.head_gate else 0, gates_out=gates)
        q = torch.empty((M, nq * (self.dn + self.dr)), dtype=x.dtype, device=dev)
        k.linear(cq, self.w_uq, q)
        qa = torch.empty((M, nq * row), dtype=x.dtype, device=dev)
        rows = torch.empty((nq * M,), dtype=torch.int32, device=dev)
        offsets = torch.empty((nq + 1,), dtype=torch.int32, device=dev)
        qn = torch.empty((nq * M, self.dn), dtype=x.dtype, device=dev)      # the unrotated parts, head by head
        k.latent_queries(q, qa, batch, num_heads=nq, head_dim=self.dn, kv_rank=self.rkv, rotation=rotation,
                         rows_out=rows, offsets_out=offsets, sorted_out=qn)
        # q_n,h -> W_uk,h^T q_n,h, written in front of the rotated part of the same (token, head) row
        k.grouped_linear_rows(qn, self.w_uk_t, rows, offsets, qa.view(M * nq, row), a_sorted=True)
        ol = torch.empty((nq * M, row), dtype=x.dtype, device=dev)           # head by head, as the next product reads it
        more = {"head_gates": gates} if gates is not None else {}
        if self.sinks is not None:
            more["head_sinks"] = self.sinks
        k.paged_attention(qa, ol, batch, cache, num_heads=nq, window=self.window,
                          softmax_scale=self.softmax_scale, cache_settled=True, out_by_head=True, **more)
        o = torch.empty((M, nq * self.dv), dtype=x.dtype, device=dev)
        k.grouped_linear_rows(ol, self.w_uv, rows, offsets, o.view(M * nq, self.dv), a_sorted=True)
        k.linear(o, self.wo, h, accumulate=accumulate)
