"""Random Paposun configurations on the GPU: width, vocabulary, layer order, head counts and sizes (no multiples of
16, odd value sizes, value heads larger and smaller than key heads, more query heads per kv head than the tensor-core
kernels take), rotations of two elements up to the whole head with and without rescaled wavelengths, chunks shorter
than a page and longer than the prompts or none, layers that read another layer's keys and values through a chunk of
their own, memories of one to six heads with key sizes from 4 to 300, gate caps, feed-forwards or none, residual and
logit factors are drawn per seed; then the engine runs whole prompts, portions, decoding and a mixed schedule in
float32 (bit-identical between the cuts) and in bfloat16 against the plain implementation."""
import random

import pytest
import torch

import helpers as H
import paposun_helpers as S
from paposun_helpers import _attn, _layer, _mlstm, _rot

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def random_config(seed: int) -> dict:
    rng = random.Random(2000 + seed)
    width = rng.choice([40, 64, 72, 100, 128, 192, 256, 320])
    layers, owners = [], []                  # owners: (layer, mixer) of attention layers with keys and values of their own
    for i in range(rng.randint(2, 7)):
        ff = rng.choice([None, 32, 60, 96, 200, 384])
        if rng.random() < 0.4:
            layers.append(_layer("mlstm", _mlstm(rng.choice([1, 2, 3, 4, 6]), rng.choice([4, 8, 20, 32, 33, 48, 64, 100, 128, 136, 300]),
                                                 rng.choice([5, 8, 12, 32, 48, 64, 70, 96, 128]), rng.choice([2.0, 4.0, 15.0, 30.0])), ff))
            continue
        if owners and rng.random() < 0.4:
            j, o = rng.choice(owners)
            m = _attn(o["heads"], o["kv_heads"], o["dim"], o["vdim"], round(o["scale"] * rng.uniform(0.7, 1.3), 4), o["rot"],
                      chunk=rng.choice([None, 5, 16, 33, 64, 100, 128, 200, 1000, o.get("mask", {}).get("size")]), kv_from=j)
        else:
            heads = rng.choice([1, 2, 3, 4, 6, 8, 12, 20])
            kv = rng.choice([k for k in range(1, heads + 1) if heads % k == 0])
            dim, vdim = rng.choice([8, 10, 16, 24, 32, 40, 48, 64, 80, 128]), rng.choice([8, 9, 16, 24, 32, 48, 64, 96, 128])
            dims = rng.choice([d for d in (2, 4, 6, 8, 10, 16, 24, 32, 64, 128, dim) if d <= dim and d % 2 == 0])
            scaling = None if rng.random() < 0.4 else (rng.choice([2.0, 4.0, 8.0, 32.0]), rng.choice([0.5, 1.0, 2.0]),
                                                       rng.choice([4.0, 8.0]), rng.choice([8, 32, 64, 512]))
            # (score scales around 1 / sqrt(head size): with scores of tens, one bfloat16 rounding of a key moves a softmax by
            # several per cent in any implementation, and the bfloat16 comparison would measure that)
            m = _attn(heads, kv, dim, vdim, round(rng.uniform(0.5, 1.5) / dim ** 0.5, 4),
                      _rot(dims, rng.choice([10.0, 100.0, 10000.0, 1e6]), scaling),
                      chunk=rng.choice([None, 5, 16, 33, 64, 100, 128, 200, 1000]))
            owners.append((i, m))
        layers.append(_layer("attention", m, ff))
    return {"architecture": "Paposun", "vocab": rng.choice([101, 256, 517, 1000]), "width": width,
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "residual_mult": rng.choice([0.2, 0.5, 1.0, 1.4]),
            "logit_scale": rng.choice([0.125, 0.5, 1.0, 3.0]), "layers": layers}


N_CONFIGS = 14


@pytest.fixture(scope="module", params=range(N_CONFIGS))
def model_folder(request, tmp_path_factory):
    seed = request.param
    cfg = random_config(seed)
    S.CONFIGS[f"random{seed}"] = (cfg, 0.07, seed)
    try:
        folder = S.write_model(tmp_path_factory.mktemp(f"paposun_random_{seed}"), f"random{seed}")
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


def test_bfloat16_every_cut(model_folder):
    from spite_b200.engine import Model
    folder, cfg, seed = model_folder
    model = Model.from_folder(folder, dtype="bfloat16", device=DEV)
    reqs = {r: H.random_tokens(cfg["vocab"], n, seed * 10 + i) for i, (r, n) in enumerate({"a": 150, "b": 33, "c": 1}.items())}
    n_prompt = {r: max(1, len(t) - 7) for r, t in reqs.items()}
    # every position is held to a twentieth of the logit scale, the typical position to a hundredth, or to a few times
    # what rounding to bfloat16 alone does there
    for steps, page in ((H.steps_whole(reqs), 64), (H.steps_portions(reqs, seed=seed), 16), (H.steps_last_decoded(reqs, 40), 64),
                        (H.steps_mixed(reqs, n_prompt, seed=seed), 64)):
        res = _run(model, steps, page)
        S.compare_with_plain(res, folder, reqs, 5e-2)
        ref, rounding = S.plain_logits(folder, reqs["a"], sixteen=True)
        errs = torch.tensor([float((res[("a", p)].double().cpu() - ref[p]).abs().max()) for p in range(len(reqs["a"]))]) / float(ref.abs().max())
        allowed = max(1.2e-2, float(rounding.median()))
        assert float(errs.median()) <= allowed, f"median error {float(errs.median()):.3e} exceeds {allowed:.1e}"
