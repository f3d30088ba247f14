"""Plain implementation of the Gapevik decoder: whole sequences, no cache, CPU, one function per mechanism, loops where a
loop is the clearest statement.  It shares no code with the package (its own safetensors reader included) and is the
oracle of the Gapevik tests.

The model.  x_0 = E[token] * s_emb.  Layer: x += mu * N1(mixer(x)); x += mu * N2(ff(x)); both sublayers read x itself
(no norm in front), N(y) = y / sqrt(mean(y^2) + eps) * gain.  Mixers: `attention` (grouped-query attention: a short
causal convolution over time on q, k and v, per-head RMS norm of q and k with a gain, rotation of neighbouring pairs of
the first rot.dims elements, scores * scale squashed to cap tanh(s / cap), sight limited to the query's chunk, a gate
sigmoid(w_h . x) per head), `latent_attention` (queries through a normed latent, keys and values of all heads from one
normed latent per position plus one rotated key part that the heads share, element i paired with i + dims/2, a sliding
window, a learned sink per head in the softmax's sum, the same gate per head) and `delta` (the gated delta rule: a matrix
state per head that decays, is corrected towards the value by the key and read by the query).  Feed-forward: a mixture
of gated SiLU experts chosen by softmax score plus a correction, weighted by the score alone, the last `identity`
router outputs standing for experts that return their input.  Output: N(x) E^T.
"""
from __future__ import annotations

import json
import math
import struct

import torch

_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path) -> dict:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=_DTYPES[info["dtype"]]).reshape(info["shape"]).clone()
    return out


def load_folder(folder):
    with open(f"{folder}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{folder}/model.safetensors")


_round = None      # set by `forward(round_inputs=...)`: what an engine that keeps activations in 16 bits does to them


def _in(x):
    """An input of a matrix product (or an attention's q, k, v), rounded the way `forward` was told to."""
    return x if _round is None else _round(x)


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the first token."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotate_neighbours(x, dims, base, positions):
    """x [T, heads, size]: pair (2i, 2i+1) of the first `dims` elements turns by p * base^(-2i/dims)."""
    out = x.clone()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        a = positions.to(x.dtype) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def rotate_halves(x, dims, base, positions):
    """x [T, heads, size]: pair (i, i + dims/2) of the first `dims` elements turns by p * base^(-2i/dims)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        f = base ** (-2.0 * i / dims)
        a = positions.to(x.dtype) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def chunk_visible(T, size):
    """[T, T] bool: query i sees key j <= i of its own chunk, chunks counted from position 0."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))


def window_visible(T, size):
    """[T, T] bool: query i sees itself and the size - 1 keys before it."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def attention(h, w, mx, eps):
    T = h.shape[0]
    H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = torch.arange(T)
    h = _in(h)
    conv = (lambda u, name: short_conv(u, w[name])) if mx.get("conv") else (lambda u, name: u)
    q = conv(h @ w["q"].T, "q.conv").view(T, H, dim)
    k = conv(h @ w["k"].T, "k.conv").view(T, G, dim)
    v = conv(h @ w["v"].T, "v.conv").view(T, G, vdim)
    q = rms_norm(q, w["q.norm"], eps)
    k = rms_norm(k, w["k.norm"], eps)
    rot = mx["rot"]
    q = _in(rotate_neighbours(q, rot["dims"], rot["base"], pos))
    k = _in(rotate_neighbours(k, rot["dims"], rot["base"], pos))
    v = _in(v)
    gate = torch.sigmoid(h @ w["g"].T)                       # [T, H]
    cap, size = mx.get("softcap"), (mx["mask"]["size"] if mx.get("mask") else T)
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    sees = chunk_visible(T, size)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * mx["scale"]             # [queries, keys]
        if cap is not None:
            s = cap * torch.tanh(s / cap)
        p = torch.softmax(s.masked_fill(~sees, -math.inf), -1)
        out[:, hd] = (p @ v[:, g]) * gate[:, hd:hd + 1]
    return _in(out.reshape(T, H * vdim)) @ w["o"].T


def latent_attention(h, w, mx, eps):
    T = h.shape[0]
    H, dim, rd, vdim, r = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    pos = torch.arange(T)
    h = _in(h)
    cq = _in(rms_norm(h @ w["dq"].T, w["dq.norm"], eps))
    q = (cq @ w["uq"].T).view(T, H, dim + rd)
    qn, qr = q[..., :dim], q[..., dim:]
    d = h @ w["dkv"].T
    c = _in(rms_norm(d[:, :r], w["dkv.norm"], eps))
    kr = d[:, r:].view(T, 1, rd)
    rot = mx["rot"]
    qr = rotate_halves(qr, rot["dims"], rot["base"], pos)
    kr = _in(rotate_halves(kr, rot["dims"], rot["base"], pos)[:, 0])
    kn = (c @ w["uk"].T).view(T, H, dim)
    v = (c @ w["uv"].T).view(T, H, vdim)
    gate = torch.sigmoid(h @ w["g"].T)
    size = mx["mask"]["size"] if mx.get("mask") else T
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    sees = window_visible(T, size)
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * mx["scale"]
        s = s.masked_fill(~sees, -math.inf)
        sink = w["sink"][hd].to(h.dtype)
        m = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - m)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))          # the sink: in the sum, nowhere else
        out[:, hd] = (p @ v[:, hd]) * gate[:, hd:hd + 1]
    return _in(out.reshape(T, H * vdim)) @ w["o"].T


def delta(h, w, mx, eps):
    T = h.shape[0]
    H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    h = _in(h)
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).view(T, G, dim)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).view(T, G, dim)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).view(T, H, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)                                                    # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(h @ w["a"].T + w["dt_bias"]))
    z = silu(h @ w["g"].T).view(T, H, vdim)
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w["norm"] * z
    return _in(out.reshape(T, H * vdim)) @ w["o"].T


def moe(h, w, ff):
    r = ff["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    h = _in(h)
    s = torch.softmax(h @ w["router"].T, -1)                 # [T, E + I]
    choice = s + w["correction"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E + I), key=lambda e: (-float(choice[t, e]), e))[:top]
        for e in order:
            if e >= E:
                out[t] += s[t, e] * h[t]
            else:
                a = _in(silu(h[t] @ w[f"e{e}.gate"].T) * (h[t] @ w[f"e{e}.up"].T))
                out[t] += s[t, e] * (a @ w[f"e{e}.down"].T)
    return out


MIXERS = {"attention": attention, "latent_attention": latent_attention, "delta": delta}


def _sub(tensors, prefix, dtype):
    return {k[len(prefix):]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, dtype=torch.float32, taps=None, round_inputs=None):
    """Logits [T, vocab] of one sequence; `taps`, a list, receives the residual stream after every layer;
    `round_inputs`, a function, is applied to every input of a matrix product and to attention's q, k and v."""
    global _round
    _round = round_inputs
    try:
        return _forward(cfg, tensors, tokens, dtype, taps)
    finally:
        _round = None


def _forward(cfg, tensors, tokens, dtype, taps):
    eps, mu = cfg["norm"]["eps"], cfg["residual_mult"]
    E = tensors["embed"].to(dtype)
    x = E[torch.tensor(tokens, dtype=torch.long)] * cfg.get("embedding", {}).get("scale", 1.0)
    for i, L in enumerate(cfg["layers"]):
        src = L.get("weights_of", i)
        p = f"l{src}."
        mix = MIXERS[L["type"]](x, _sub(tensors, p + "mix.", dtype), L["mixer"], eps)
        x = x + mu * rms_norm(mix, tensors[p + "norm1"].to(dtype), eps)
        if L.get("mlp") is not None:
            y = moe(x, _sub(tensors, p + "mlp.", dtype), L["mlp"])
            x = x + mu * rms_norm(y, tensors[p + "norm2"].to(dtype), eps)
        if taps is not None:
            taps.append(x.clone())
    return _in(rms_norm(x, tensors["final.norm"].to(dtype), eps)) @ E.T
