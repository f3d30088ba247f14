"""Paposun without a GPU: the configuration and its errors, tensor names, the plain implementation's mechanisms
against loops written out element by element, and the engine (cache, state slots, batches, trace replay) with the
plain torch kernel set in every cut."""
import json
import math

import pytest
import torch

import helpers as H
import paposun_helpers as S
import plain_paposun as plain
from reference_kernels import TorchReferenceKernels
from spite_b200.cache import Window
from spite_b200.config import ConfigError, PaposunConfig, load_config
from spite_b200.engine import Engine, Model


# ---------------------------------------------------------------------------- configuration
def test_configuration_round_trip_and_plan():
    for name, (cfg, _, _) in S.CONFIGS.items():
        c = PaposunConfig.from_dict(cfg)
        assert c.to_dict() == cfg, name
        plan = c.plan()
        assert [b.arrangement for b in plan.blocks] == ["sandwich_residual"] * len(cfg["layers"])
        assert plan.tie_word_embeddings and plan.logit_scale == cfg["logit_scale"]
    order = PaposunConfig.from_dict(S.CONFIG_K).plan().order
    assert [(c.layer, c.cache, c.write_cache) for c in order] == \
        [(0, 0, True), (1, 0, False), (2, 2, True), (3, 3, True), (4, 3, False), (5, 5, True)]


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(dim=12), "other sizes"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][2].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][2]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "mlp.kind"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["norm"].update(eps=0), "eps"),
])
def test_configuration_errors_name_the_key(change, word):
    cfg = json.loads(json.dumps(S.CONFIG_K))
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        PaposunConfig.from_dict(cfg)


def test_windows_of_layers_that_share_a_cache():
    assert Window("chunk", 20).union(Window("chunk", 40)) == Window("chunk", 40)
    assert Window("chunk", 20).union(Window("chunk", 30)) == Window("full")
    assert Window("chunk", 7).union(Window("full")) == Window("full")
    assert Window("sliding", 5).union(Window("sliding", 9)) == Window("sliding", 9)
    assert Window("chunk", 8).union(Window("chunk", 8)) == Window("chunk", 8)
    k = TorchReferenceKernels(torch.float32, "cpu")
    model = Model.from_config(PaposunConfig.from_dict(S.CONFIG_K), dtype="float32", device="cpu", kernels=k)
    specs = model.cache_specs()
    assert specs[0][0].window == Window("chunk", 40) and specs[3][0].window == Window("full")
    assert specs[2][0] is None and specs[2][1].shape == (3, k.mlstm_state_size(20, 12))
    assert specs[5][1].shape == (1, 40 * 70 + 3 * 44)


# ---------------------------------------------------------------------------- the plain implementation's mechanisms
def test_rotation_frequencies_by_wavelength():
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}}
    f = plain.rotation_frequencies(rot)
    plainf = [100.0 ** (-2 * i / 8) for i in range(4)]
    # wavelengths 6.3, 19.9, 62.8, 198.7 against the borders 10 and 40
    assert f[0] == plainf[0] and f[2] == plainf[2] / 4 and f[3] == plainf[3] / 4
    s = (40 / (2 * math.pi / plainf[1]) - 1.0) / 3.0
    assert abs(f[1] - ((1 - s) * plainf[1] / 4 + s * plainf[1])) < 1e-12
    assert plain.rotation_frequencies({"dims": 8, "base": 100.0}) == plainf


def test_rotation_pairs_the_two_halves_of_the_leading_elements():
    rot = {"dims": 4, "base": 10.0}
    x = torch.arange(12, dtype=torch.float64).reshape(2, 1, 6) + 1.0
    y = plain.rotate(x, rot, start=3)
    f = plain.rotation_frequencies(rot)
    for t in range(2):
        for i in range(2):
            a = (3 + t) * f[i]
            u, v = float(x[t, 0, i]), float(x[t, 0, i + 2])
            assert abs(float(y[t, 0, i]) - (u * math.cos(a) - v * math.sin(a))) < 1e-12
            assert abs(float(y[t, 0, i + 2]) - (v * math.cos(a) + u * math.sin(a))) < 1e-12
        assert torch.equal(y[t, 0, 4:], x[t, 0, 4:])


def test_chunk_mask_counts_from_position_zero():
    see = plain.chunk_mask(7, 3)
    assert see[2].tolist() == [True, True, True, False, False, False, False]
    assert see[3].tolist() == [False, False, False, True, False, False, False]
    assert see[6].tolist() == [False] * 6 + [True]


def test_memory_against_its_closed_form():
    """S_t = sum_s exp(i_s + sum_{s < r <= t} f_r - m_t) k_s v_s^T with m_t the running maximum that starts at 0."""
    torch.manual_seed(0)
    T, d, H, dim, vdim, cap = 9, 10, 2, 4, 3, 5.0
    w = {"q": torch.randn(H * dim, d), "k": torch.randn(H * dim, d), "v": torch.randn(H * vdim, d), "g": torch.randn(H * vdim, d),
         "o": torch.randn(d, H * vdim), "norm": torch.rand(H * vdim) + 0.5, "i": torch.randn(H, d) * 3, "i.b": torch.randn(H),
         "f": torch.randn(H, d) * 3, "f.b": torch.randn(H)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, d).double()
    mx = {"heads": H, "dim": dim, "vdim": vdim, "gate_cap": cap}
    got = plain.mlstm(h, w, mx, 1e-6)
    q = (h @ w["q"].T).reshape(T, H, dim) / math.sqrt(dim)
    k = (h @ w["k"].T).reshape(T, H, dim)
    v = (h @ w["v"].T).reshape(T, H, vdim)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    z = cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap)
    gf = -torch.log1p(torch.exp(-z))
    out = torch.zeros(T, H, vdim).double()
    for a in range(H):
        for t in range(T):
            F = [float(gf[s + 1:t + 1, a].sum()) for s in range(t + 1)]
            m = max([float(gf[:t + 1, a].sum())] + [float(gi[s, a]) + F[s] for s in range(t + 1)])      # the start value 0 decays too
            S = sum(math.exp(float(gi[s, a]) + F[s] - m) * torch.outer(k[s, a], v[s, a]) for s in range(t + 1))
            n = sum(math.exp(float(gi[s, a]) + F[s] - m) * k[s, a] for s in range(t + 1))
            den = max(abs(float(n @ q[t, a])), math.exp(-m)) + 1e-6
            o = (S.T @ q[t, a]) / den
            out[t, a] = o / torch.sqrt((o * o).mean() + 1e-6)
    ref = ((out.reshape(T, -1) * w["norm"]) * torch.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert float((got - ref).abs().max()) < 1e-9 * float(ref.abs().max())


# ---------------------------------------------------------------------------- the engine on the host
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: S.write_model(tmp_path_factory.mktemp(f"paposun_{n}"), n) for n in ("K", "M")}


def host_engine(folder, tokens, page_size=16, max_requests=4):
    k = TorchReferenceKernels(torch.float32, "cpu")
    model = Model.from_folder(folder, dtype="float32", device="cpu", kernels=k)
    return Engine(model, cache_tokens=tokens, page_size=page_size, max_requests=max_requests)


def requests_for(folder, lens, seed):
    vocab = json.loads((folder / "config.json").read_text())["vocab"]
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("name", ["K", "M"])
def test_folder_round_trip_and_whole_prompts(folders, name):
    folder = folders[name]
    assert load_config(folder).to_dict() == S.CONFIGS[name][0]
    reqs = requests_for(folder, (47, 1, 20), 10)
    eng = host_engine(folder, 64 * 3)
    S.compare_with_plain(H.run_steps(eng, H.steps_whole(reqs)), folder, reqs, 2e-5)
    assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups


def test_the_residual_stream_after_every_layer(folders):
    folder = folders["K"]
    toks = requests_for(folder, (45,), 20)["r0"]
    cfg, tensors = S.folder_contents(str(folder))
    taps = []
    plain.forward(cfg, tensors, toks, taps=taps)
    eng = host_engine(folder, 64)
    seen = []
    eng.model.layer_tap = lambda i, h: seen.append(h.clone())
    H.run_steps(eng, H.steps_whole({"a": toks}))
    assert len(seen) == len(taps)
    for i, h in enumerate(seen):
        assert float((h - taps[i]).abs().max()) <= 2e-5 * float(taps[i].abs().max()), f"layer {i}"


@pytest.mark.parametrize("name", ["K", "M"])
def test_portions_decoding_and_mixed_batches_on_the_host(folders, name):
    """Token by token after a prompt, portions down to two tokens, and up to four live requests in a pool that
    forces pages and state slots to be used again: the logits are those of the whole sequence."""
    folder = folders[name]
    reqs = requests_for(folder, (45, 9, 30, 3, 26, 17), 30)
    cuts = {"decoded": H.steps_last_decoded(reqs, 12), "portions": H.steps_portions(reqs, seed=2),
            "mixed": H.steps_mixed(reqs, {r: max(1, len(t) - 6) for r, t in reqs.items()}, seed=3)}
    for what, steps in cuts.items():
        eng = host_engine(folder, H.max_tokens_of(steps) if what == "mixed" else 64, page_size=16)
        S.compare_with_plain(H.run_steps(eng, steps), folder, reqs, 2e-5)
        assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups, what


def test_pages_behind_every_reader_s_chunk_go_back(folders):
    """Layers 0 and 1 share a cache through chunks of 20 and 40: its pages go back by the chunk of 40.  Layers 3 and 4
    share one of which layer 3 reads everything: nothing goes back before the request ends."""
    eng = host_engine(folders["K"], 256, page_size=8)
    toks = requests_for(folders["K"], (90,), 50)["r0"]
    H.run_steps(eng, [{"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [89]}], "end": []}])
    keys = eng.storage.group_keys
    by_window = {k.window: g for g, k in enumerate(keys)}
    shared = eng.cache.block_table("a", by_window[Window("chunk", 40)])
    assert [p >= 0 for p in shared] == [False] * 10 + [True] * 2          # positions 80..89 live in pages 10 and 11
    assert all(p >= 0 for p in eng.cache.block_table("a", by_window[Window("full")]))


def test_a_state_slot_that_is_used_again_starts_at_zero(folders):
    eng = host_engine(folders["M"], 128, max_requests=1)
    reqs = requests_for(folders["M"], (30, 25), 60)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"], "want": [29]}], "end": ["r0"]},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"][:10], "want": [9]}], "end": []},
             {"step": 2, "entries": [{"id": "r1", "tokens": reqs["r1"][10:], "want": [0, 14]}], "end": ["r1"]}]
    S.compare_with_plain(H.run_steps(eng, steps), folders["M"], reqs, 2e-5)


def test_trace_replay_on_the_host(folders, tmp_path):
    import io
    import numpy as np
    from spite_b200.engine.trace import replay
    folder = folders["K"]
    reqs = requests_for(folder, (50, 21, 5), 70)
    steps = H.steps_mixed(reqs, {r: len(t) - 4 for r, t in reqs.items()}, seed=9)
    eng = host_engine(folder, H.max_tokens_of(steps), page_size=64)
    log = io.StringIO()
    replay(eng, [json.dumps(s) for s in steps], tmp_path / "out", log=log)
    assert log.getvalue().split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    vocab = S.CONFIG_K["vocab"]
    pos, got = {}, {}
    for s in steps:
        n_rows = sum(len(e["want"]) for e in s["entries"])
        if not n_rows:
            continue
        rows = np.fromfile(tmp_path / "out" / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
        i = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = torch.from_numpy(rows[i].copy())
                i += 1
            pos[e["id"]] = base + len(e["tokens"])
    S.compare_with_plain(got, folder, reqs, 2e-5)
