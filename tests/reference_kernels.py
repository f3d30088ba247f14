"""Plain torch restatement of every kernel's contract (`spite_b200.kernels.api`).

Two uses, both in tests only:
  * the reference each CUDA kernel is compared with, op by op;
  * a stand-in kernel set with which the engine's host logic (cache, batches,
    scheduler, trace replay) is exercised on a machine without a GPU.
It is slow on purpose: loops over tokens and heads, float32 arithmetic (float64
on request), no fusion.  It is not part of the package and nothing in the
package imports it.
"""
from __future__ import annotations

import math

import torch

from spite_b200.kernels.api import KernelSet, Routing


class TorchReferenceKernels(KernelSet):
    def __init__(self, dtype=torch.float32, device="cpu", acc=torch.float32):
        self.dtype = dtype
        self.device = torch.device(device)
        self.acc = acc

    # ---- elementwise
    def embed(self, table, token_ids, out_h, *, scale=1.0, position_table=None, positions=None):
        x = table[token_ids.long()].to(self.acc) * scale
        if position_table is not None:
            x = x + position_table[positions.long()].to(self.acc)
        out_h.copy_(x.to(out_h.dtype))

    def pack_pair(self, a, b, out, *, refill=None):
        out.copy_(torch.cat([a, b], -1).to(out.dtype))
        if refill is not None:
            a.copy_(refill.to(a.dtype)[None, :].expand_as(a))

    def clear_pages(self, kv, page_ids):
        if page_ids:
            kv[:, :, torch.tensor(page_ids, dtype=torch.long)] = 0

    def transform_logits(self, logits, *, scale=1.0, softcap=None):
        logits.mul_(scale)
        if softcap:
            logits.copy_(softcap * torch.tanh(logits / softcap))

    def rms_norm(self, h, gain, eps, out, rows=None):
        x = h if rows is None else h[rows.long()]
        x = x.to(self.acc)
        y = x * (1.0 / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)) * gain.to(self.acc)
        out.copy_(y.to(out.dtype))

    def rms_norm_residual(self, y, gain, eps, mult, h, *, next_gain=None, next_out=None):
        v = y.to(self.acc)
        v = v * (1.0 / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)) * gain.to(self.acc)
        h.add_((mult * v).to(h.dtype))
        if next_out is not None and next_gain is None:
            next_out.copy_(h.to(next_out.dtype))
        elif next_out is not None:
            self.rms_norm(h, next_gain, eps, next_out)

    def cast_rows(self, h, out):
        out.copy_(h.to(out.dtype))

    def short_conv(self, x, w, out, batch, state, *, channels, activation=None, state_offset=0):
        taps = w.shape[1]
        cu = batch.cu_seqlens.tolist()
        slots = batch.slots.tolist()
        xv, wv = x.to(self.acc), w.to(self.acc)
        out[:, channels:] = x[:, channels:out.shape[1]].to(out.dtype)
        for s in range(len(cu) - 1):
            if s > 0 and slots[s] == slots[0]:                  # a padding copy of the first row comes out as that row does
                n = min(cu[s + 1] - cu[s], cu[1] - cu[0])
                out[cu[s]:cu[s] + n] = out[cu[0]:cu[0] + n]
                continue
            if taps > 1:
                st = state[slots[s]].reshape(-1)[state_offset:state_offset + (taps - 1) * channels].view(taps - 1, channels)
            else:
                st = xv.new_zeros((0, channels))
            hist = torch.cat([st.to(self.acc), xv[cu[s]:cu[s + 1], :channels]], 0)       # rows -(taps-1) .. n-1
            for i in range(cu[s + 1] - cu[s]):
                y = torch.zeros(channels, dtype=self.acc)
                for j in range(taps):
                    y = y + wv[:, j] * hist[i + j]
                if activation == "silu":
                    y = y * torch.sigmoid(y)
                out[cu[s] + i, :channels] = y.to(out.dtype)
            if taps > 1:
                st.copy_(hist[hist.shape[0] - (taps - 1):].to(st.dtype))

    def delta_scan(self, x, out, batch, state, *, heads, kv_heads, dim, vdim, columns, a_log, dt_bias, q_scale,
                   unit_eps=1e-6, state_offset=0, split_rows=None):
        qc, kc, vc, bc, ac = columns
        xv = x.to(self.acc)
        cu = batch.cu_seqlens.tolist()
        slots = batch.slots.tolist()
        for s in range(len(cu) - 1):
            if s > 0 and slots[s] == slots[0]:                  # a padding copy of the first row
                out[cu[s]:cu[s + 1]] = 0
                continue
            flat = state[slots[s]].reshape(-1)
            for a in range(heads):
                g = a // (heads // kv_heads)
                st = flat[state_offset + a * dim * vdim:state_offset + (a + 1) * dim * vdim]
                S = st.to(self.acc).reshape(dim, vdim).clone()
                for t in range(cu[s], cu[s + 1]):
                    q = xv[t, qc + g * dim:qc + (g + 1) * dim]
                    k = xv[t, kc + g * dim:kc + (g + 1) * dim]
                    v = xv[t, vc + a * vdim:vc + (a + 1) * vdim]
                    q = q / torch.sqrt((q * q).sum() + unit_eps) * q_scale
                    k = k / torch.sqrt((k * k).sum() + unit_eps)
                    beta = torch.sigmoid(xv[t, bc + a])
                    decay = torch.exp(-torch.exp(a_log[a].to(self.acc)) *
                                      torch.nn.functional.softplus(xv[t, ac + a] + dt_bias[a].to(self.acc)))
                    S = decay * S
                    u = beta * (v - S.T @ k)
                    S = S + torch.outer(k, u)
                    out[t, a * vdim:(a + 1) * vdim] = (S.T @ q).to(out.dtype)
                st.copy_(S.reshape(-1).to(st.dtype))

    def fill_rows(self, out, vec, *, accumulate=False):
        if accumulate:
            out.add_(vec[None, :].to(out.dtype))
        else:
            out.copy_(vec[None, :].to(out.dtype).expand_as(out))

    def head_norm_gate(self, x, out, *, heads, size, gates=None, gate_column=0, gain=None, eps=None, gate_activation="sigmoid"):
        M = x.shape[0]
        v = x.to(self.acc).reshape(M, heads, size)
        if eps is not None:
            v = v * (1.0 / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps))
        v = v.reshape(M, heads * size)
        if gain is not None:
            v = v * gain.to(self.acc)
        if gates is not None:
            z = gates[:, gate_column:gate_column + heads * size].to(self.acc)
            v = v * (torch.sigmoid(z) * z if gate_activation == "silu" else torch.sigmoid(z))
        out.copy_(v.to(out.dtype))

    # ---- recurrent mixers
    def mlstm_scan(self, proj, out, batch, state, *, heads, dim, vdim, gate_cap, q_scale, columns, i_bias, f_bias, chunked=None):
        qc, kc, vc, ic, fc = columns
        x = proj.to(self.acc)
        cu = batch.cu_seqlens.tolist()
        slots = batch.slots.tolist()
        nm = -(-(dim + 1) // 4) * 4
        for s in range(len(cu) - 1):
            if s > 0 and slots[s] == slots[0]:                  # a padding copy of the first row
                out[cu[s]:cu[s + 1]] = 0
                continue
            for a in range(heads):
                st = state[slots[s], a]
                S = st[:dim * vdim].to(self.acc).reshape(dim, vdim).clone()
                n = st[dim * vdim:dim * vdim + dim].to(self.acc).clone()
                m = st[dim * vdim + dim].to(self.acc).clone()
                for t in range(cu[s], cu[s + 1]):
                    q = x[t, qc + a * dim:qc + (a + 1) * dim] * q_scale
                    k = x[t, kc + a * dim:kc + (a + 1) * dim]
                    v = x[t, vc + a * vdim:vc + (a + 1) * vdim]
                    ig = gate_cap * torch.tanh((x[t, ic + a] + i_bias[a].to(self.acc)) / gate_cap)
                    fg = torch.nn.functional.logsigmoid(gate_cap * torch.tanh((x[t, fc + a] + f_bias[a].to(self.acc)) / gate_cap))
                    m_new = torch.maximum(fg + m, ig)
                    keep, take = torch.exp(fg + m - m_new), torch.exp(ig - m_new)
                    S = keep * S + take * torch.outer(k, v)
                    n = keep * n + take * k
                    m = m_new
                    den = torch.maximum((n @ q).abs(), torch.exp(-m)) + 1e-6
                    out[t, a * vdim:(a + 1) * vdim] = ((S.T @ q) / den).to(out.dtype)
                st[:dim * vdim] = S.reshape(-1).to(st.dtype)
                for b in range(-(-vdim // 32)):                  # every block of 32 value columns keeps its own n and m
                    o = dim * vdim + b * nm
                    st[o:o + dim] = n.to(st.dtype)
                    st[o + dim] = m.to(st.dtype)

    # ---- matrix products
    def _mm(self, x, w):
        return x.to(self.acc) @ w.to(self.acc).T

    def linear(self, x, w, out, *, accumulate=False, row_scale=None, activation=None):
        y = self._mm(x, w)
        if row_scale is not None:
            y = y * row_scale.to(self.acc)[:, None]
        if activation is not None:
            assert activation in ("relu2", "gelu_tanh") and not accumulate
            if activation == "relu2":
                y = torch.relu(y) ** 2
            else:
                y = 0.5 * y * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (y + 0.044715 * y ** 3)))
        if accumulate:
            out.add_(y.to(out.dtype))
        else:
            out.copy_(y.to(out.dtype))

    @staticmethod
    def _silu(g):
        return g / (1.0 + torch.exp(-g))

    def linear_swiglu(self, x, w_gate_up, out, *, row_scale=None):
        F = w_gate_up.shape[0] // 2
        y = self._mm(x, w_gate_up)
        if row_scale is not None:
            y = y * row_scale.to(self.acc)[:, None]
        out.copy_((self._silu(y[:, :F]) * y[:, F:]).to(out.dtype))

    def grouped_linear_swiglu(self, x, w_gate_up, sorted_rows, offsets, row_scale, out):
        E, F2, _ = w_gate_up.shape
        F = F2 // 2
        off = offsets.tolist()
        rows = sorted_rows.long()
        for e in range(E):
            lo, hi = off[e], off[e + 1]
            if hi == lo:
                continue
            tok = rows[lo:hi]
            y = self._mm(x[tok], w_gate_up[e])
            if row_scale is not None:
                y = y * row_scale[tok].to(self.acc)[:, None]
            out[lo:hi] = (self._silu(y[:, :F]) * y[:, F:]).to(out.dtype)

    def grouped_linear_act(self, x, w_up, sorted_rows, offsets, row_scale, out, *, activation="relu2"):
        assert activation == "relu2"
        off = offsets.tolist()
        rows = sorted_rows.long()
        for e in range(w_up.shape[0]):
            lo, hi = off[e], off[e + 1]
            if hi == lo:
                continue
            tok = rows[lo:hi]
            y = self._mm(x[tok], w_up[e])
            if row_scale is not None:
                y = y * row_scale[tok].to(self.acc)[:, None]
            out[lo:hi] = (torch.relu(y) ** 2).to(out.dtype)

    def grouped_linear_accumulate(self, a, w_down, sorted_rows, offsets, h, *, row_scale=None):
        E = w_down.shape[0]
        off = offsets.tolist()
        rows = sorted_rows.long()
        for e in range(E):
            lo, hi = off[e], off[e + 1]
            if hi == lo:
                continue
            y = self._mm(a[lo:hi], w_down[e])
            if row_scale is not None:
                y = y * row_scale[lo:hi].to(self.acc)[:, None]
            h[rows[lo:hi]] += y.to(h.dtype)

    def grouped_linear_rows(self, a, w, rows, offsets, out, *, a_sorted=False):
        G, N, K = w.shape
        off = offsets.tolist()
        idx = rows.long()
        for g in range(G):
            r = idx[off[g]:off[g + 1]]
            if r.numel():
                src = a[off[g]:off[g + 1], :K] if a_sorted else a[r, :K]
                out[r, :N] = self._mm(src, w[g]).to(out.dtype)

    # ---- attention
    def qk_prepare(self, qkv, q_out, batch, cache, *, num_heads, rotation, qk_norm, temperature,
                   value_mix=None, gates_out=None, bias=None, q_only=False, norm_dim=None):
        kv = cache.kv
        nkv, P, hd = kv.shape[2], kv.shape[3], kv.shape[4]
        nq = num_heads
        M = qkv.shape[0]
        cols = (nq + (0 if q_only else 2 * nkv)) * hd
        x = qkv[:, :cols].to(self.acc)
        if bias is not None:
            x = x + bias.to(self.acc)[None, :]
        x = x.reshape(M, -1, hd)
        q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]
        if q_only:
            assert not cache.write
            k = q[:, :0]
        pos = batch.positions.long()
        if gates_out is not None:
            gates_out.copy_(torch.sigmoid(qkv[:, cols:cols + nq].to(torch.float32)))
        if value_mix is not None:
            other, col, stride, vd, lam = value_mix
            v = v.clone()
            for g in range(nkv):
                o = other[:, col + g * stride: col + g * stride + vd].to(self.acc)
                v[:, g, :vd] = (1.0 - lam) * v[:, g, :vd] + lam * o

        def norm(t, gain):
            t = t * (1.0 / torch.sqrt(t.pow(2).sum(-1, keepdim=True) / (norm_dim or hd) + qk_norm.eps))
            return t if gain is None else t * gain.to(t.device, self.acc)

        if qk_norm is not None and qk_norm.before_rotation:
            q, k = norm(q, qk_norm.q_gain), norm(k, qk_norm.k_gain)
        if rotation is not None:
            inv_freq = rotation.inv_freq.to(q.device)
            rd = rotation.rotary_dim or hd
            ang = (pos.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)).to(self.acc)
            cos, sin = torch.cos(ang)[:, None, :] * rotation.amplitude, torch.sin(ang)[:, None, :] * rotation.amplitude

            def rot(t):
                o = t.clone()
                if rotation.pairing == "neighbours":
                    a, b = t[..., 0:rd:2], t[..., 1:rd:2]
                    o[..., 0:rd:2] = a * cos - b * sin
                    o[..., 1:rd:2] = a * sin + b * cos
                else:
                    a, b = t[..., :rd // 2], t[..., rd // 2:rd]
                    o[..., :rd // 2] = a * cos - b * sin
                    o[..., rd // 2:rd] = a * sin + b * cos
                return o
            q, k = rot(q), rot(k)
        if qk_norm is not None and not qk_norm.before_rotation:
            q, k = norm(q, qk_norm.q_gain), norm(k, qk_norm.k_gain)
        if temperature:
            floor, scale = temperature
            fl = torch.div(pos + 1, int(floor), rounding_mode="floor").to(self.acc)
            q = q * (torch.log(fl + 1.0) * scale + 1.0)[:, None, None]
        q_out.copy_(q.reshape(M, nq * hd).to(q_out.dtype))
        if cache.write:
            bt = batch.block_tables[cache.group]
            seg = batch.seg_of_token.long()
            for t in range(M):
                p = int(pos[t])
                page = int(bt[seg[t], p // P])
                assert page >= 0, "write into a page that is not held"
                kv[0, page, :, p % P, :] = k[t].to(kv.dtype)
                kv[1, page, :, p % P, :] = v[t].to(kv.dtype)

    def _rotate_pairs(self, t, pos, rotation):
        """t [M, ..., rot]: neighbouring pairs (or element i with i + rot/2) turn by pos * inv_freq, times the amplitude."""
        ang = (pos.to(torch.float32)[:, None] * rotation.inv_freq.to(t.device, torch.float32)[None, :]).to(self.acc)
        shape = [t.shape[0]] + [1] * (t.dim() - 2) + [ang.shape[1]]
        cos, sin = (torch.cos(ang) * rotation.amplitude).view(shape), (torch.sin(ang) * rotation.amplitude).view(shape)
        o = torch.empty_like(t)
        if rotation.pairing == "halves":
            half = t.shape[-1] // 2
            a, b = t[..., :half], t[..., half:]
            o[..., :half] = a * cos - b * sin
            o[..., half:] = a * sin + b * cos
            return o
        a, b = t[..., 0::2], t[..., 1::2]
        o[..., 0::2] = a * cos - b * sin
        o[..., 1::2] = a * sin + b * cos
        return o

    def latent_prepare(self, down, cq_out, batch, cache, *, q_rank, kv_rank, rotation, q_gain, kv_gain, eps,
                       num_gates=0, gates_out=None):
        kv = cache.kv
        P, row = kv.shape[3], kv.shape[4]
        rot = rotation.inv_freq.numel() * 2
        x = down.to(self.acc)
        pos = batch.positions.long()

        def norm(t, gain):
            return t * (1.0 / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + eps)) * gain.to(self.acc)
        cq_out.copy_(norm(x[:, :q_rank], q_gain).to(cq_out.dtype))
        c = norm(x[:, q_rank:q_rank + kv_rank], kv_gain)
        kr = self._rotate_pairs(x[:, q_rank + kv_rank:q_rank + kv_rank + rot], pos, rotation)
        if gates_out is not None:
            g0 = q_rank + kv_rank + rot
            gates_out.copy_(torch.sigmoid(down[:, g0:g0 + num_gates].to(torch.float32)))
        if cache.write:
            bt = batch.block_tables[cache.group]
            seg = batch.seg_of_token.long()
            for t in range(x.shape[0]):
                p = int(pos[t])
                page = int(bt[seg[t], p // P])
                assert page >= 0, "write into a page that is not held"
                kv[0, page, 0, p % P, :] = 0
                kv[0, page, 0, p % P, :kv_rank] = c[t].to(kv.dtype)
                kv[0, page, 0, p % P, kv_rank:kv_rank + rot] = kr[t].to(kv.dtype)

    def latent_queries(self, q, q_out, batch, *, num_heads, head_dim, kv_rank, rotation, rows_out, offsets_out,
                       sorted_out=None):
        M = q.shape[0]
        rot = rotation.inv_freq.numel() * 2
        qv = q.to(self.acc).view(M, num_heads, head_dim + rot)
        out = q_out.view(M, num_heads, -1)
        out[:, :, kv_rank:] = 0
        out[:, :, kv_rank:kv_rank + rot] = self._rotate_pairs(qv[:, :, head_dim:], batch.positions.long(), rotation).to(out.dtype)
        m = torch.arange(M, dtype=torch.int32, device=q.device)
        for h in range(num_heads):
            rows_out[h * M:(h + 1) * M] = m * num_heads + h
        offsets_out.copy_(torch.arange(num_heads + 1, dtype=torch.int32, device=q.device) * M)
        if sorted_out is not None:
            sorted_out.copy_(q.view(M, num_heads, head_dim + rot)[:, :, :head_dim].transpose(0, 1).reshape(num_heads * M, head_dim))

    def paged_attention(self, q, out, batch, cache, *, num_heads, window, softmax_scale, cache_settled=False,
                        sink_logit=None, head_sinks=None, head_slopes=None, head_gates=None, out_by_head=False,
                        score_softcap=None):
        kv = cache.kv
        nkv, P, hd = kv.shape[2], kv.shape[3], kv.shape[4]
        nq = num_heads
        group = nq // nkv
        M = q.shape[0]
        bt = batch.block_tables[cache.group]
        pos = batch.positions.tolist()
        seg = batch.seg_of_token.tolist()
        qf = q.to(self.acc).view(M, nq, hd)
        for t in range(M):
            p = pos[t]
            lo = window.lowest_visible(p)
            js = torch.arange(lo, p + 1)
            pages = bt[seg[t]].long()[torch.div(js, P, rounding_mode="floor")]
            assert bool((pages >= 0).all()), "read from a page that was given back"
            K = kv[0, pages, :, js % P, :].to(self.acc)          # [n, nkv, hd]
            V = kv[kv.shape[0] - 1, pages, :, js % P, :].to(self.acc)     # (one plane: the key rows are the values)
            for h in range(nq):
                s = (K[:, h // group, :] @ qf[t, h]) * softmax_scale
                if score_softcap is not None:
                    s = score_softcap * torch.tanh(s / score_softcap)
                if head_slopes is not None:
                    s = s - float(head_slopes[h]) * (p - js).to(self.acc)
                sink = sink_logit if head_sinks is None else float(head_sinks[h])
                if sink is None:
                    w = torch.softmax(s, dim=0)
                else:                                            # a key of that score and no value
                    w = torch.softmax(torch.cat([s, s.new_tensor([sink])]), dim=0)[:-1]
                o = w @ V[:, h // group, :]
                if head_gates is not None:
                    o = o * head_gates[t, h].to(self.acc)
                if out_by_head:
                    out.view(nq, M, hd)[h, t] = o.to(out.dtype)
                else:
                    out[t, h * hd:(h + 1) * hd] = o.to(out.dtype)

    # ---- mixture of experts
    def moe_identity(self, x, routing, first_identity, out, *, accumulate=True):
        w = (routing.weights * (routing.expert_ids >= first_identity)).sum(0).to(self.acc)      # [M]
        y = w[:, None] * x.to(self.acc)
        if accumulate:
            out.add_(y.to(out.dtype))
        else:
            out.copy_(y.to(out.dtype))

    def moe_route(self, x, w_router, top_k, want_logits=False, scoring="sigmoid", choice_bias=None) -> Routing:
        logits = (x.to(torch.float32) @ w_router.to(torch.float32).T)
        order = torch.sort(logits, dim=-1, descending=True, stable=True)
        if scoring == "softmax_biased":
            share = torch.softmax(logits, -1)
            order = torch.sort(share + choice_bias.to(torch.float32)[None, :], dim=-1, descending=True, stable=True)
        ids = order.indices[:, :top_k].T.contiguous().to(torch.int32)        # [k, M]
        if scoring == "sigmoid":
            w = (1.0 / (1.0 + torch.exp(-order.values[:, :top_k]))).T.contiguous()
        elif scoring == "softmax_biased":
            w = share.gather(1, order.indices[:, :top_k]).T.contiguous()
        else:
            assert scoring == "softmax_renorm"
            share = torch.softmax(logits, -1).gather(1, order.indices[:, :top_k])
            w = (share / (share.sum(-1, keepdim=True) + 1e-20)).T.contiguous()
        M, E = logits.shape
        offsets = torch.zeros((top_k, E + 1), dtype=torch.int32, device=x.device)
        rows = torch.zeros((top_k, M), dtype=torch.int32, device=x.device)
        for s in range(top_k):
            srt = torch.sort(ids[s].long(), stable=True)
            rows[s] = srt.indices.to(torch.int32)
            counts = torch.bincount(ids[s].long(), minlength=E)
            offsets[s, 1:] = torch.cumsum(counts, 0).to(torch.int32)
        sorted_w = torch.stack([w[s][rows[s].long()] for s in range(top_k)], 0)
        return Routing(ids, w, offsets, rows, logits if want_logits else None, sorted_w)

    # ---- sampling
    def argmax(self, logits):
        V = logits.shape[1]
        flipped = torch.flip(logits, dims=[1])
        return (V - 1 - torch.argmax(flipped, dim=1)).to(torch.int32)

    def sample(self, logits, *, temperature, top_k=None, top_p=None, min_p=None, repetition_penalty=None,
               context=None, context_offsets=None, rng_state):
        from plain_llama4 import sample_plain
        out = torch.zeros(logits.shape[0], dtype=torch.int32)
        for r in range(logits.shape[0]):
            ctx = []
            if context is not None:
                ctx = context[int(context_offsets[r]):int(context_offsets[r + 1])].tolist()
            tok, st = sample_plain(
                logits[r].cpu(), ctx, temperature=float(temperature[r]),
                top_k=int(top_k[r]) if top_k is not None else 0,
                top_p=float(top_p[r]) if top_p is not None else 1.0,
                min_p=float(min_p[r]) if min_p is not None else 0.0,
                repetition_penalty=float(repetition_penalty[r]) if repetition_penalty is not None else 1.0,
                repeat_last_n=0, state=int(rng_state[r]) & ((1 << 64) - 1))
            out[r] = tok
            rng_state[r] = st - (1 << 64) if st >= (1 << 63) else st
        return out.to(logits.device)
