"""Random Gapevik configurations on the GPU: width, vocabulary, layer order, head counts and sizes (no multiples of
16, value heads larger and smaller than key heads, more query heads per kv head than the tensor-core kernels take),
rotations of two elements up to the whole head, chunks and windows shorter than a page, longer than the prompts or
none, caps, convolutions of one to eight taps, latent ranks, delta heads of 4 to 300 key rows on one or several q/k
heads, experts with none to three identity experts and one to four choices or no feed-forward, layers that borrow
another layer's weights, residual and embedding factors are drawn per seed; then the engine runs whole prompts,
portions, decoding and a mixed schedule in float32 (bit-identical between the cuts) and in bfloat16 against the plain
implementation."""
import random

import pytest
import torch

import gapevik_helpers as S
import helpers as H
from gapevik_helpers import _attn, _delta, _latent, _layer, _moe

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def random_config(seed: int) -> dict:
    rng = random.Random(3000 + seed)
    width = rng.choice([40, 64, 72, 100, 128, 192, 256, 320])
    layers = []
    for i in range(rng.randint(2, 8)):
        owners = [j for j, L in enumerate(layers) if "weights_of" not in L]
        if owners and rng.random() < 0.25:
            j = rng.choice(owners)
            layers.append(dict(layers[j], weights_of=j))
            continue
        mlp = None
        if rng.random() < 0.75:
            experts, identity = rng.choice([1, 2, 3, 5, 8]), rng.choice([0, 0, 1, 2, 3])
            mlp = _moe(rng.choice([8, 24, 40, 64, 96]), experts, identity, rng.randint(1, min(4, experts + identity)))
        kind = rng.choice(["attention", "latent_attention", "delta"])
        size = rng.choice([None, 1, 5, 16, 33, 40, 64, 100, 128, 200, 1000])
        if kind == "attention":
            heads = rng.choice([1, 2, 3, 4, 6, 8, 12, 20])
            kv = rng.choice([k for k in range(1, heads + 1) if heads % k == 0])
            dim, vdim = rng.choice([8, 10, 16, 24, 32, 40, 48, 64, 80, 128]), rng.choice([8, 10, 16, 24, 32, 48, 64, 96, 128])
            dims = rng.choice([d for d in (2, 4, 6, 8, 10, 16, 24, 32, 64, 128, dim) if d <= dim])
            m = _attn(heads, kv, dim, vdim, round(rng.uniform(0.5, 1.5) / dim ** 0.5, 4), dims, rng.choice([10.0, 1e4, 5e5]),
                      chunk=size, softcap=rng.choice([None, 1.0, 5.0, 30.0, 50.0]), conv=rng.choice([None, 1, 2, 3, 4, 4, 8]))
        elif kind == "latent_attention":
            heads = rng.choice([1, 2, 3, 4, 8, 16, 20])
            dim, rot = rng.choice([4, 8, 12, 16, 32, 64]), rng.choice([2, 4, 6, 8, 16, 32, 64])
            kv_rank = rng.choice([5, 16, 18, 32, 48, 96, 112, 200])
            if rng.random() < 0.4:                            # rows of 64 or 128 elements: the tcgen05 and TMA kernels
                rot = rng.choice([16, 32])
                kv_rank = rng.choice([64, 128]) - rot
            m = _latent(heads, dim, rot, rng.choice([4, 8, 20, 32, 64]), rng.choice([3, 10, 40, 64, 80]), kv_rank,
                        round(rng.uniform(0.5, 1.5) / (dim + rot) ** 0.5, 4), rng.choice([10.0, 1e4, 2e4]), window=size)
        else:
            heads = rng.choice([1, 2, 3, 4, 6, 8])
            kv = rng.choice([k for k in range(1, heads + 1) if heads % k == 0])
            m = _delta(heads, kv, rng.choice([4, 8, 20, 32, 33, 48, 64, 100, 128, 136, 300]),
                       rng.choice([5, 8, 12, 32, 48, 64, 70, 96, 128]), rng.choice([1, 2, 3, 4, 4, 8]))
        layers.append(_layer(kind, m, mlp))
    return {"architecture": "Gapevik", "vocab": rng.choice([101, 256, 517, 1000]), "width": width,
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "residual_mult": rng.choice([0.2, 0.5, 1.0, 1.4]),
            "embedding": {"scale": rng.choice([1.0, 3.0, width ** 0.5])}, "layers": layers}


N_CONFIGS = 12


@pytest.fixture(scope="module", params=range(N_CONFIGS))
def model_folder(request, tmp_path_factory):
    seed = request.param
    cfg = random_config(seed)
    S.CONFIGS[f"random{seed}"] = (cfg, 0.07, seed)
    try:
        folder = S.write_model(tmp_path_factory.mktemp(f"gapevik_random_{seed}"), f"random{seed}")
    finally:
        del S.CONFIGS[f"random{seed}"]
    return folder, cfg, seed


def _run(model, steps, page):
    from spite_b200.engine import Engine
    eng = Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=page, max_requests=4)
    out = H.run_steps(eng, steps)
    eng.check()
    assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups
    return out


def test_float32_every_cut(model_folder):
    from spite_b200.engine import Model
    folder, cfg, seed = model_folder
    model = Model.from_folder(folder, dtype="float32", device=DEV)
    reqs = {r: H.random_tokens(cfg["vocab"], n, seed * 10 + i) for i, (r, n) in enumerate({"a": 230, "b": 33, "c": 1, "d": 58}.items())}
    n_prompt = {r: max(1, len(t) - 7) for r, t in reqs.items()}
    cuts = {"whole": _run(model, H.steps_whole(reqs), 64), "portions": _run(model, H.steps_portions(reqs, seed=seed), 16),
            "decoded": _run(model, H.steps_last_decoded(reqs, 40), 64),
            "mixed": _run(model, H.steps_mixed(reqs, n_prompt, seed=seed), 16)}
    for res in cuts.values():
        S.compare_with_plain(res, folder, reqs, 4e-5)
    H.assert_cuts_identical(cuts)


def test_bfloat16_every_cut(model_folder, tmp_path_factory):
    from spite_b200.engine import Model
    _, cfg, seed = model_folder
    S.CONFIGS[f"random{seed}"] = (cfg, 0.07, seed)
    try:                                                     # (see `write_model`: no choice of experts is left to rounding)
        folder = S.write_model(tmp_path_factory.mktemp(f"gapevik_random_{seed}_settled"), f"random{seed}", settled_routing=True)
    finally:
        del S.CONFIGS[f"random{seed}"]
    model = Model.from_folder(folder, dtype="bfloat16", device=DEV)
    reqs = {r: H.random_tokens(cfg["vocab"], n, seed * 10 + i) for i, (r, n) in enumerate({"a": 150, "b": 33, "c": 1}.items())}
    n_prompt = {r: max(1, len(t) - 7) for r, t in reqs.items()}
    # every position is held to a twentieth of the logit scale, the typical position to a fiftieth, or to a few times
    # what rounding to bfloat16 alone does there
    for steps, page in ((H.steps_whole(reqs), 64), (H.steps_portions(reqs, seed=seed), 16), (H.steps_last_decoded(reqs, 40), 64),
                        (H.steps_mixed(reqs, n_prompt, seed=seed), 64)):
        res = _run(model, steps, page)
        S.compare_with_plain(res, folder, reqs, 5e-2)
        ref, rounding = S.plain_logits(folder, reqs["a"], sixteen=True)
        errs = torch.tensor([float((res[("a", p)].double().cpu() - ref[p]).abs().max()) for p in range(len(reqs["a"]))]) / float(ref.abs().max())
        allowed = max(2e-2, float(rounding.median()))
        assert float(errs.median()) <= allowed, f"median error {float(errs.median()):.3e} exceeds {allowed:.1e}"
