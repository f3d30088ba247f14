"""Small Gapevik configurations for the tests (none has the sizes of a published model), model folders with random
weights, and the comparison with the plain implementation (`plain_gapevik`)."""
from __future__ import annotations

import functools
from pathlib import Path

import torch

import plain_gapevik as plain
from helpers import note_error
from spite_b200.config import GapevikConfig
from spite_b200.weights import save_file, write_random_model


def _attn(heads, kv, dim, vdim, scale, rot_dims, rot_base, chunk=None, softcap=None, conv=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": rot_base}}
    if chunk is not None:
        d["mask"] = {"size": chunk}
    if softcap is not None:
        d["softcap"] = softcap
    if conv is not None:
        d["conv"] = conv
    return d


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot_base, window=None):
    d = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": rot_base}}
    if window is not None:
        d["mask"] = {"size": window}
    return d


def _delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(ff, experts, identity, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def _layer(kind, mixer, mlp=None, weights_of=None):
    d = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def _model(vocab, width, eps, mult, emb, layers):
    return {"architecture": "Gapevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"scale": emb}, "layers": layers}


# awkward sizes: value heads smaller and larger than key heads, a rotation of 6 of 24 elements, chunks and windows
# shorter than a page, convolutions of 2 and 3 taps, a latent row of 24 elements, a delta layer of three heads on one
# q/k head whose value columns fill no block of 32, three experts and one identity expert, one expert a token
# elsewhere, a layer without feed-forward, layers that borrow weights
_A0 = _layer("attention", _attn(4, 2, 24, 16, 0.2, 6, 50.0, chunk=20, softcap=5.0, conv=3), _moe(40, 3, 1, 2))
_A2 = _layer("delta", _delta(3, 1, 20, 12, 2), _moe(24, 4, 0, 1))
CONFIG_A = _model(211, 72, 1e-5, 0.5, 3.0, [
    _A0,
    _layer("latent_attention", _latent(3, 12, 6, 20, 10, 18, 0.25, 100.0, window=7), None),
    _A2,
    dict(_A0, weights_of=0),
    _layer("attention", _attn(3, 3, 16, 32, 0.25, 16, 10000.0, chunk=33, softcap=2.0, conv=2), _moe(32, 2, 2, 3)),
    dict(_A2, weights_of=2),
    _layer("latent_attention", _latent(2, 8, 4, 8, 7, 11, 0.3, 10.0, window=40), _moe(16, 1, 1, 1)),
])

# rows of 64 and 128 elements and a width of 128: the tcgen05 and TMA kernels; a chunk and a window that cross pages;
# six delta heads of 64 x 64 on three q/k heads and two of 136 x 40; conv of 4 taps
_B1 = _layer("latent_attention", _latent(8, 32, 32, 32, 64, 96, 0.12, 20000.0, window=100), _moe(64, 6, 2, 2))
CONFIG_B = _model(520, 128, 1e-6, 0.5, 11.3, [
    _layer("attention", _attn(4, 2, 64, 64, 0.125, 32, 5e5, chunk=150, softcap=30.0, conv=4), _moe(80, 6, 3, 2)),
    _B1,
    _layer("delta", _delta(6, 3, 64, 64, 4), _moe(64, 4, 1, 2)),
    _layer("latent_attention", _latent(4, 16, 16, 48, 40, 48, 0.15, 1e4, window=64), None),
    dict(_B1, weights_of=1),
    _layer("delta", _delta(2, 2, 136, 40, 4), None),
    _layer("attention", _attn(2, 1, 128, 96, 0.09, 128, 500.0, chunk=64, softcap=50.0, conv=4), _moe(128, 2, 0, 2)),
])

# values that may hide a fault by being one: one head everywhere, one expert a token, a window of one (a token sees
# itself alone), a chunk of one, a convolution of one tap, factors of one
CONFIG_C = _model(97, 40, 1e-3, 1.0, 1.0, [
    _layer("delta", _delta(1, 1, 8, 8, 1), _moe(24, 1, 1, 1)),
    _layer("attention", _attn(1, 1, 8, 8, 0.4, 2, 10.0, chunk=1, softcap=1.0, conv=1), _moe(24, 2, 1, 1)),
    _layer("latent_attention", _latent(1, 4, 2, 6, 3, 5, 0.5, 10.0, window=1), None),
    _layer("attention", _attn(2, 2, 10, 10, 0.3, 10, 10.0, chunk=3, softcap=8.0, conv=8), None),
    _layer("delta", _delta(2, 1, 33, 5, 8), _moe(8, 3, 0, 3)),
])

CONFIGS = {"A": (CONFIG_A, 0.12, 5), "B": (CONFIG_B, 0.09, 6), "C": (CONFIG_C, 0.2, 7)}


def write_model(folder, name: str, dtype=torch.bfloat16, settled_routing=False) -> Path:
    """A model folder with random weights.  Norm gains are drawn around one so that a lost gain shows; the sinks, the
    routers' corrections and the decays' constants get sizes at which leaving one out changes the logits.
    `settled_routing`: the routers' weights are small and the corrections lie 0.3 apart in a random order, so that every
    token's choice of experts is clear of rounding (for comparisons in bfloat16, where a choice that rounding decides
    makes two correct implementations differ by an expert's output, at that position and, through keys, values and
    recurrent state, at every later one); the shares still differ from token to token, and with them the weights."""
    cfg, std, seed = CONFIGS[name]
    config = GapevikConfig.from_dict(cfg)
    folder = write_random_model(folder, config, seed=seed, std=std, dtype=dtype)
    _, tensors = plain.load_folder(folder)
    g = torch.Generator().manual_seed(seed)
    for n, t in tensors.items():
        if n.endswith(".sink"):
            tensors[n] = (torch.randn(t.shape, generator=g) * 1.5).to(t.dtype)
        elif n.endswith(".correction"):
            tensors[n] = (torch.randn(t.shape, generator=g) * 0.15).to(t.dtype)
            if settled_routing:
                tensors[n] = (torch.randperm(t.numel(), generator=g).float() * 0.3).to(t.dtype)
        elif n.endswith(".A_log"):
            tensors[n] = (torch.randn(t.shape, generator=g) * 0.7 - 2.0).to(t.dtype)
        elif n.endswith(".dt_bias"):
            tensors[n] = (torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith(".conv"):
            tensors[n] = (torch.randn(t.shape, generator=g) * 0.5).to(t.dtype)
        elif n.endswith(".router"):
            tensors[n] = (t.float() * (0.25 if settled_routing else 2.0)).to(t.dtype)
        elif t.dim() == 1:
            tensors[n] = (1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
    save_file(tensors, Path(folder) / "model.safetensors")
    return Path(folder)


@functools.lru_cache(maxsize=None)
def folder_contents(folder: str):
    return plain.load_folder(folder)


_plain_cache: dict = {}


def plain_logits(folder, tokens, sixteen=False):
    """(logits computed in float64, what a position may be off by through rounding alone, as a fraction of the largest
    logit).  For float32 arithmetic: four times the distance of a float32 run.  With `sixteen`, for activations kept in
    bfloat16: in an otherwise float64 computation the inputs of every matrix product and attention's queries, keys and
    values are disturbed by random relative errors four times as large as a rounding to bfloat16 makes (up to 2^-7); the
    largest distance among three draws counts, or four times the distance of a run that rounds these to bfloat16
    exactly.  A position at which rounding decides which expert runs, or at which a delta head puts out next to nothing
    (its direction, which is all its norm keeps, is then noise), is ill-conditioned: rounding moves its logits out of
    proportion, and the comparison allows for it."""
    key = (str(folder), tuple(tokens), sixteen)
    if key not in _plain_cache:
        cfg, tensors = folder_contents(str(folder))
        ref = plain.forward(cfg, tensors, list(tokens), torch.float64)
        if sixteen:
            g = torch.Generator().manual_seed(len(tokens))
            shake = lambda x: x * (1.0 + 2.0 ** -7 * (2.0 * torch.rand(x.shape, generator=g, dtype=x.dtype) - 1.0))
            lows = [plain.forward(cfg, tensors, list(tokens), torch.float64, round_inputs=shake) for _ in range(3)]
            exact = plain.forward(cfg, tensors, list(tokens), torch.float64, round_inputs=lambda x: x.to(torch.bfloat16).to(x.dtype))
            moved = torch.stack([(ref - low).abs().amax(-1) for low in lows] + [4.0 * (ref - exact).abs().amax(-1)]).amax(0)
        else:
            moved = 4.0 * (ref - plain.forward(cfg, tensors, list(tokens), torch.float32).double()).abs().amax(-1)
        _plain_cache[key] = (ref, moved / float(ref.abs().max()))
    return _plain_cache[key]


def generate_greedy(cfg, tensors, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(plain.forward(cfg, tensors, toks)[-1])))
    return toks[len(prompt):]


def compare_with_plain(results: dict, folder, requests: dict, tol: float):
    """Every logits row against the plain implementation in float64, as a fraction of the largest logit of the
    sequence; names the first position beyond its allowance.  In float32 a position may be off by `tol` or by what
    `plain_logits` finds that rounding alone may do to it, whichever is more.  The same in the 16-bit comparison (a
    `tol` of a thousandth or more), where a norm behind every sublayer brings the rounding of a sublayer's output back
    to unit size layer after layer, so that a deep stack moves by several per cent of its logits' scale under
    rounding alone; there one position in twenty-five of a request (or two) may be off by up to four times its
    allowance: the estimate is four draws."""
    worst = 0.0
    sixteen = tol >= 1e-3
    for r, toks in requests.items():
        ref, rounding = plain_logits(folder, toks, sixteen=sixteen)
        scale = float(ref.abs().max())
        spare = max(2, len(toks) // 25) if sixteen else 0
        for p in range(len(toks)):
            if (r, p) not in results:
                continue
            err = float((results[(r, p)].double().cpu() - ref[p]).abs().max()) / scale
            allowed = max(tol, float(rounding[p]))
            if allowed < err <= 4.0 * allowed and spare > 0:
                spare -= 1
                continue
            worst = max(worst, err * tol / allowed)
            assert err <= allowed, (f"request {r!r}, position {p} (first wrong one): error {err:.3e} of the "
                                    f"logit scale exceeds {allowed:.1e} (worst before it: {worst:.3e})")
    note_error(worst, tol)
    return worst
