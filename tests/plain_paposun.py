"""Plain, slow implementation of the Paposun decoder: whole sequences, no cache, float32 (or float64) on the
CPU, one function per mechanism, written from the design's equations.  It shares no code with the package: it
has its own safetensors reader and takes the parsed config.json as a dict.

Notation: x is the residual stream [T, d] of one sequence, h a sublayer's input, p a position (from 0).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ---------------------------------------------------------------------------------- files
def read_safetensors(path) -> dict:
    """8-byte little-endian header length, JSON header (name -> dtype, shape, data_offsets), data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = memoryview(raw)[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
    return out


def load_folder(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# ---------------------------------------------------------------------------------- mechanisms
_round = None        # `forward(round_inputs=...)`: applied to the activations that enter every matrix product and to what attention reads and writes


def _in(x):
    return x if _round is None else _round(x)


def rms_norm(x, w, eps):
    """y = x / sqrt(mean(x^2) + eps) * w; the epsilon stands inside the root."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotation_frequencies(rot):
    """f_i = base^(-2i/dims), i < dims/2, then the rescaling by wavelength l = 2 pi / f: short waves (l <
    original/high) stay, long ones (l > original/low) are divided by `factor`, those between are blended with
    s = (original/l - low) / (high - low): (1 - s) f / factor + s f."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            factor, low, high, orig = (float(sc[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x, rot, start=0):
    """x [T, heads, dim]: among the first `dims` elements of a head, element i pairs with i + dims/2;
    (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p f_i.  The other elements pass."""
    T = x.shape[0]
    dims = int(rot["dims"])
    half = dims // 2
    f = torch.tensor(rotation_frequencies(rot), dtype=torch.float64)
    p = torch.arange(start, start + T, dtype=torch.float64)
    a = p[:, None] * f[None, :]                        # [T, half]
    cos, sin = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def chunk_mask(T, size):
    """[T, T] True where row i may see column j: j <= i and both in the same chunk of `size` positions (no size: j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) if size is None else (j <= i) & (i // size == j // size)


def attention_keys_values(h, w, mx):
    """The layer's own rotated keys and its values: ([T, G, dim], [T, G, vdim])."""
    T = h.shape[0]
    h = _in(h)
    G, dim, vdim = int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, dim)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, vdim)
    return _in(rotate(k, mx["rot"])), _in(v)


def gated_attention(h, w, mx, keys, values):
    """Grouped-query attention over the given (rotated) keys and values, softmax over the keys of the query's chunk,
    the concatenated heads times sigmoid(W_g h), then the output projection with its bias."""
    T = h.shape[0]
    h = _in(h)
    H, G, dim, vdim = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    q = _in(rotate((h @ w["q"].T + w["q.b"]).reshape(T, H, dim), mx["rot"]))
    see = chunk_mask(T, int(mx["mask"]["size"]) if mx.get("mask") else None)
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ keys[:, g].T) * float(mx["scale"])
        s = s.masked_fill(~see, -math.inf)
        out[:, a] = torch.softmax(s, -1) @ values[:, g]
    gate = torch.sigmoid(h @ w["g"].T)
    return _in(_in(out.reshape(T, H * vdim)) * gate) @ w["o"].T + w["o.b"]


def mlstm(h, w, mx, eps):
    """Matrix memory per head, token by token.  q = W_q h / sqrt(dim), k = W_k h, v = W_v h;
    i = cap tanh((W_i h + b_i) / cap), f = logsigmoid(cap tanh((W_f h + b_f) / cap));
    m_t = max(f + m_(t-1), i) with m_(-1) = 0; S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T, n_t alike with k;
    o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6); every head's o over its root mean square, all heads times
    `norm`, times sigmoid(W_g h), then W_o."""
    T = h.shape[0]
    h = _in(h)
    H, dim, vdim, cap = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"]), float(mx["gate_cap"])
    q = (h @ w["q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ w["k"].T).reshape(T, H, dim)
    v = (h @ w["v"].T).reshape(T, H, vdim)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)                       # [T, H]
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        n = torch.zeros(dim, dtype=h.dtype)
        m = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            m_new = torch.maximum(gf[t, a] + m, gi[t, a])
            keep, take = torch.exp(gf[t, a] + m - m_new), torch.exp(gi[t, a] - m_new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            m = m_new
            den = torch.maximum((n @ q[t, a]).abs(), torch.exp(-m)) + 1e-6
            out[t, a] = (S.T @ q[t, a]) / den
    out = rms_norm(out, None, eps).reshape(T, H * vdim) * w["norm"]
    return _in(out * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def dense_ff(h, w):
    return _in(gelu_tanh(_in(h) @ w["up"].T)) @ w["down"].T


# ---------------------------------------------------------------------------------- the model
def _sub(tensors, prefix, dtype):
    return {k[len(prefix):]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, dtype=torch.float32, taps=None, round_inputs=None):
    """Logits [T, vocab] of one whole sequence.  `taps`, a list, receives the residual stream after every layer.
    `round_inputs`, a function, is applied to the activations that enter every matrix product, to queries, keys and
    values as attention reads them and to the heads it puts out (and to nothing else): with a rounding to 16 bits it
    shows how far that rounding alone moves the logits."""
    global _round
    _round = round_inputs
    try:
        return _forward(cfg, tensors, tokens, dtype, taps)
    finally:
        _round = None


def _forward(cfg, tensors, tokens, dtype, taps):
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = tensors["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    kept = {}                                           # layer -> its rotated keys and its values
    for i, layer in enumerate(cfg["layers"]):
        name = f"l{i}."
        w = _sub(tensors, name + "mix.", dtype)
        mx = layer["mixer"]
        h = rms_norm(x, tensors[name + "norm1"].to(dtype), eps)
        if layer["type"] == "attention":
            if mx.get("kv_from") is not None:
                keys, values = kept[int(mx["kv_from"])]
            else:
                keys, values = kept[i] = attention_keys_values(h, w, mx)
            y = gated_attention(h, w, mx, keys, values)
        elif layer["type"] == "mlstm":
            y = mlstm(h, w, mx, eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + mult * rms_norm(y, tensors[name + "norm1b"].to(dtype), eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, tensors[name + "norm2"].to(dtype), eps)
            y = dense_ff(h, _sub(tensors, name + "mlp.", dtype))
            x = x + mult * rms_norm(y, tensors[name + "norm2b"].to(dtype), eps)
        if taps is not None:
            taps.append(x.clone())
    x = _in(rms_norm(x, tensors["final.norm"].to(dtype), eps))
    return (x @ tensors["embed"].to(dtype).T) * float(cfg["logit_scale"])
