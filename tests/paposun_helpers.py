"""Small Paposun configurations for the tests (none has the sizes of a published model), model folders with
random weights, and the comparison with the plain implementation (`plain_paposun`)."""
from __future__ import annotations

import functools
from pathlib import Path

import torch

import plain_paposun as plain
from helpers import note_error
from spite_b200.config import PaposunConfig
from spite_b200.weights import save_file, write_random_model


def _rot(dims, base, scaling=None):
    d = {"dims": dims, "base": base}
    if scaling:
        d["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return d


def _attn(heads, kv, dim, vdim, scale, rot, chunk=None, kv_from=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if chunk is not None:
        d["mask"] = {"size": chunk}
    if kv_from is not None:
        d["kv_from"] = kv_from
    return d


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


# awkward sizes: value heads smaller and larger than key heads, a rotation of 6 and of all elements, with and
# without rescaled wavelengths, chunks of 20 and 40 on one cache, a layer that sees everything read through a chunk
# of 7, memories of one and three heads whose value columns fill no block of 32 or pass one, no feed-forward here and there
CONFIG_K = {
    "architecture": "Paposun", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_scale": 2.0,
    "layers": [
        _layer("attention", _attn(4, 2, 24, 16, 0.2, _rot(6, 50.0, (8.0, 1.0, 4.0, 16)), chunk=20), ff=96),
        _layer("attention", _attn(4, 2, 24, 16, 0.3, _rot(6, 50.0, (8.0, 1.0, 4.0, 16)), chunk=40, kv_from=0)),
        _layer("mlstm", _mlstm(3, 20, 12, 10.0), ff=40),
        _layer("attention", _attn(3, 3, 16, 32, 0.25, _rot(16, 10000.0))),
        _layer("attention", _attn(3, 3, 16, 32, 0.15, _rot(16, 10000.0), chunk=7, kv_from=3), ff=64),
        _layer("mlstm", _mlstm(1, 40, 70, 4.0)),
    ]}

# rows of 64 and 128 elements and a width of 128: the tcgen05 and TMA kernels; a chunk of one page; value heads of 96
# in rows of 128; a memory whose heads have more than 128 key rows; the first layer is an attention
CONFIG_L = {
    "architecture": "Paposun", "vocab": 520, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "logit_scale": 1.0,
    "layers": [
        _layer("attention", _attn(4, 2, 64, 64, 0.125, _rot(32, 1e6, (4.0, 1.0, 4.0, 64)), chunk=150), ff=192),
        _layer("mlstm", _mlstm(2, 64, 64, 15.0)),
        _layer("attention", _attn(8, 2, 64, 64, 0.1, _rot(32, 1e6, (4.0, 1.0, 4.0, 64)), chunk=150, kv_from=0), ff=128),
        _layer("attention", _attn(2, 1, 128, 96, 0.09, _rot(64, 500.0), chunk=64), ff=256),
        _layer("mlstm", _mlstm(1, 136, 32, 15.0), ff=128),
    ]}

# one head everywhere, a model of memories alone after one attention, a factor above one
CONFIG_M = {
    "architecture": "Paposun", "vocab": 97, "width": 40, "norm": {"eps": 1e-3}, "residual_mult": 1.25, "logit_scale": 0.5,
    "layers": [
        _layer("mlstm", _mlstm(4, 8, 8, 2.0), ff=24),
        _layer("attention", _attn(1, 1, 8, 8, 0.4, _rot(2, 10.0), chunk=3), ff=24),
        _layer("mlstm", _mlstm(2, 33, 5, 30.0)),
    ]}

CONFIGS = {"K": (CONFIG_K, 0.12, 5), "L": (CONFIG_L, 0.09, 6), "M": (CONFIG_M, 0.2, 7)}


def write_model(folder, name: str, dtype=torch.bfloat16) -> Path:
    """A model folder with random weights; norm gains are drawn around one so that a lost gain shows, and the gates'
    projections of the memories are large enough to move the gates over their range."""
    cfg, std, seed = CONFIGS[name]
    config = PaposunConfig.from_dict(cfg)
    folder = write_random_model(folder, config, seed=seed, std=std, dtype=dtype)
    _, tensors = plain.load_folder(folder)
    g = torch.Generator().manual_seed(seed)
    for n, t in tensors.items():
        if t.dim() == 1 and not n.endswith(".b"):
            tensors[n] = (1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith(("mix.i", "mix.f")):
            tensors[n] = (t.float() * 6.0).to(t.dtype)
        elif n.endswith(("mix.i.b", "mix.f.b")):
            tensors[n] = (torch.randn(t.shape, generator=g) * 1.5).to(t.dtype)
    save_file(tensors, Path(folder) / "model.safetensors")
    return Path(folder)


@functools.lru_cache(maxsize=None)
def folder_contents(folder: str):
    return plain.load_folder(folder)


_plain_cache: dict = {}


def plain_logits(folder, tokens, sixteen=False):
    """(logits computed in float64, what a position may be off by through rounding alone, as a fraction of the largest
    logit).  For float32 arithmetic: four times the distance of a float32 run.  With `sixteen`, for activations kept in
    bfloat16: in an otherwise float64 computation the inputs of every matrix product and attention's queries, keys,
    values and heads are disturbed by random relative errors four times as large as a rounding to bfloat16 makes
    (up to 2^-7); the largest distance among three draws counts, or four times the distance of a run that rounds these
    to bfloat16 exactly as an engine would (which reproduces the turns of sign that the engine's own rounding causes).  A position at which a head of a memory puts out next
    to nothing (its direction, which is all its norm keeps, then turns on the sign of q . k), or n . q nearly cancels,
    is ill-conditioned: there rounding moves the logits by far more than elsewhere, out of proportion to its size, and
    the comparison allows for it."""
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
    `plain_logits` finds that rounding alone may do to it, whichever is more.  In the 16-bit comparison (a `tol` of a
    thousandth or more) the positions that the disturbed runs move by more than twice `tol` are ill-conditioned and
    left to the float32 comparison (they must stay a minority); of the others one in twenty-five of a request (or two) may
    be off by up to four times their allowance: the estimate is four draws."""
    worst = 0.0
    sixteen = tol >= 1e-3
    judged = skipped = 0
    for r, toks in requests.items():
        ref, rounding = plain_logits(folder, toks, sixteen=sixteen)
        scale = float(ref.abs().max())
        spare = max(2, len(toks) // 25) if sixteen else 0
        for p in range(len(toks)):
            if (r, p) not in results:
                continue
            if sixteen and float(rounding[p]) > 2.0 * tol:
                skipped += 1
                continue
            judged += 1
            err = float((results[(r, p)].double().cpu() - ref[p]).abs().max()) / scale
            allowed = max(tol, float(rounding[p]))
            if allowed < err <= 4.0 * allowed and spare > 0:
                spare -= 1
                continue
            worst = max(worst, err * tol / allowed)
            assert err <= allowed, (f"request {r!r}, position {p} (first wrong one): error {err:.3e} of the "
                                    f"logit scale exceeds {allowed:.1e} (worst before it: {worst:.3e})")
    assert judged >= skipped, f"{skipped} ill-conditioned positions beside {judged} others: this model tests little"
    note_error(worst, tol)
    return worst
