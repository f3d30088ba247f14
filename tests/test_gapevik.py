"""Gapevik without a GPU: the configuration and its errors, tensor names, the plain implementation's mechanisms
against loops written out element by element, and the engine (cache, state slots, batches, trace replay) with the
plain torch kernel set in every cut."""
import json
import math

import pytest
import torch

import gapevik_helpers as S
import helpers as H
import plain_gapevik as plain
from reference_kernels import TorchReferenceKernels
from spite_b200.cache import Window
from spite_b200.config import ConfigError, GapevikConfig, load_config
from spite_b200.engine import Engine, Model


# ---------------------------------------------------------------------------- configuration
def test_configuration_round_trip_and_plan():
    for name, (cfg, _, _) in S.CONFIGS.items():
        c = GapevikConfig.from_dict(cfg)
        assert c.to_dict() == cfg, name
        plan = c.plan()
        own = [i for i, L in enumerate(cfg["layers"]) if "weights_of" not in L]
        assert [b.arrangement for b in plan.blocks] == ["postnorm_residual"] * len(own)
        assert plan.tie_word_embeddings and plan.embedding_scale == cfg["embedding"]["scale"]
    # a layer that borrows weights runs the lender's block on a cache of its own
    order = GapevikConfig.from_dict(S.CONFIG_A).plan().order
    assert [(c.layer, c.cache, c.write_cache) for c in order] == \
        [(0, 0, True), (1, 1, True), (2, 2, True), (0, 3, True), (3, 4, True), (2, 5, True), (4, 6, True)]


def test_tensor_names_and_borrowed_layers():
    c = GapevikConfig.from_dict(S.CONFIG_A)
    names = {n for b in c.weight_bindings() for n in b.sources}
    assert {"embed", "final.norm", "l0.mix.q.conv", "l0.mix.k.norm", "l0.mix.g", "l0.mlp.e2.down", "l0.mlp.correction",
            "l1.mix.dkv.norm", "l1.mix.sink", "l1.mix.uk", "l2.mix.A_log", "l2.mix.dt_bias", "l2.mix.b", "l2.mix.a",
            "l2.mix.norm", "l4.mlp.router", "l6.mix.uq"} <= names
    assert not any(n.startswith(("l3.", "l5.")) for n in names)          # layers 3 and 5 borrow their weights
    assert "l1.norm2" not in names and "l0.mlp.e3.gate" not in names      # no feed-forward there; three experts here
    by_target = {b.target: b for b in c.weight_bindings()}
    assert by_target["layers.0.ffn.router"].source_shape == (4, 72)      # three experts and one identity expert
    assert by_target["layers.3.mixer.q_proj"].source == "l4.mix.q"        # the fourth block is layer 4's


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][3].update(weights_of=3), "weights_of"),
    (lambda c: c["layers"][5].update(weights_of=3), "weights_of"),
    (lambda c: c["layers"][3].update(type="delta", mixer=c["layers"][2]["mixer"]), "that layer is"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda c: c["layers"][2].update(type="mlstm"), "not a mixer"),
    (lambda c: c["layers"][2]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][2]["mixer"].update(conv=9), "conv"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["norm"].update(eps=0), "eps"),
])
def test_configuration_errors_name_the_key(change, word):
    cfg = json.loads(json.dumps(S.CONFIG_A))
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        GapevikConfig.from_dict(cfg)


# ---------------------------------------------------------------------------- the plain implementation's mechanisms
def test_masks_count_from_position_zero():
    sees = plain.chunk_visible(12, 5)
    assert [int(sees[i].sum()) for i in range(12)] == [1, 2, 3, 4, 5, 1, 2, 3, 4, 5, 1, 2]
    assert bool(sees[7, 5]) and not bool(sees[7, 4]) and not bool(sees[5, 6])
    sees = plain.window_visible(10, 4)
    assert [int(sees[i].sum()) for i in range(10)] == [1, 2, 3, 4, 4, 4, 4, 4, 4, 4]
    assert bool(sees[8, 5]) and not bool(sees[8, 4]) and not bool(sees[3, 4])


def test_rotations_pair_neighbours_or_halves_of_the_leading_elements():
    x = torch.randn(5, 2, 10, dtype=torch.float64)
    pos = torch.arange(5) + 3
    a, b = plain.rotate_neighbours(x, 6, 50.0, pos), plain.rotate_halves(x, 6, 50.0, pos)
    assert torch.equal(a[..., 6:], x[..., 6:]) and torch.equal(b[..., 6:], x[..., 6:])
    for t in range(5):
        for i in range(3):
            ang = float(pos[t]) * 50.0 ** (-2.0 * i / 6)
            c, s = math.cos(ang), math.sin(ang)
            for (u, v), out in (((2 * i, 2 * i + 1), a), ((i, i + 3), b)):
                assert abs(float(out[t, 1, u]) - (float(x[t, 1, u]) * c - float(x[t, 1, v]) * s)) < 1e-12
                assert abs(float(out[t, 1, v]) - (float(x[t, 1, v]) * c + float(x[t, 1, u]) * s)) < 1e-12


def test_short_convolution_against_its_sum():
    u, w = torch.randn(9, 4, dtype=torch.float64), torch.randn(4, 3, dtype=torch.float64)
    y = plain.short_conv(u, w)
    for t in range(9):
        for c in range(4):
            ref = sum(float(w[c, j]) * float(u[t - 2 + j, c]) for j in range(3) if t - 2 + j >= 0)
            assert abs(float(y[t, c]) - ref) < 1e-12
    assert torch.allclose(y[0], w[:, 2] * u[0])                          # the last column is the current token's


def test_delta_rule_against_its_unrolled_form():
    """With beta = 1 and no decay, writing key k with value v and reading with q = k returns v exactly (the rule
    replaces what the memory held along k); with decay g, an earlier write along an orthogonal key comes back times g."""
    mx = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "conv": 1}
    eye = torch.eye(4, dtype=torch.float64)
    big = 1e3
    w = {"q": eye * big, "k": eye * big, "v": torch.zeros(3, 4, dtype=torch.float64), "q.conv": torch.ones(4, 1, dtype=torch.float64),
         "k.conv": torch.ones(4, 1, dtype=torch.float64), "v.conv": torch.ones(3, 1, dtype=torch.float64),
         "b": torch.zeros(1, 4, dtype=torch.float64), "a": torch.zeros(1, 4, dtype=torch.float64),
         "A_log": torch.tensor([math.log(0.5)], dtype=torch.float64), "dt_bias": torch.tensor([0.3], dtype=torch.float64),
         "g": torch.zeros(3, 4, dtype=torch.float64), "norm": torch.ones(3, dtype=torch.float64), "o": torch.eye(3, dtype=torch.float64)}
    w["v"][:, :3] = torch.eye(3, dtype=torch.float64) * 2.0
    w["b"][0, 3] = 50.0                                                   # beta = sigmoid(50 * h_3) = 1 where h_3 = 1
    w["g"][:, 3] = 10.0                                                   # the gate silu(10) is the same for every column
    h = torch.tensor([[1.0, 0, 0, 1.0], [0, 1.0, 0, 1.0], [1.0, 0, 0, 1.0]], dtype=torch.float64)
    out = plain.delta(h, w, mx, 1e-12)
    g = math.exp(-0.5 * math.log1p(math.exp(0.3)))
    v = plain.silu(h @ w["v"].T)
    # token 2 reads along key 0: the memory holds g^2 v_0 there, beta = 1 replaces it by v_2 = v_0: the read-out is v_0
    o2 = v[2] * 0.5                                                       # times dim^-1/2
    ref2 = o2 / torch.sqrt((o2 * o2).mean() + 1e-12) * plain.silu(torch.tensor(10.0, dtype=torch.float64))
    assert torch.allclose(out[2], ref2, atol=1e-6)
    assert g < 1.0


def test_router_chooses_by_corrected_share_and_weighs_by_the_share():
    ff = {"router": {"experts": 2, "identity": 1, "top": 2}}
    d = 4
    w = {"router": torch.zeros(3, d, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 0.0], dtype=torch.float64)}
    w["router"][0, 0], w["router"][1, 0], w["router"][2, 0] = 2.0, 1.0, 0.0
    for e in range(2):
        w[f"e{e}.gate"] = torch.randn(5, d, dtype=torch.float64)
        w[f"e{e}.up"] = torch.randn(5, d, dtype=torch.float64)
        w[f"e{e}.down"] = torch.randn(d, 5, dtype=torch.float64)
    h = torch.tensor([[1.0, 0.5, -0.3, 0.2]], dtype=torch.float64)
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=torch.float64), 0)

    def expert(e):
        return (plain.silu(h[0] @ w[f"e{e}.gate"].T) * (h[0] @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T
    assert torch.allclose(plain.moe(h, w, ff)[0], s[0] * expert(0) + s[1] * expert(1))
    # a correction lifts the identity expert over expert 1: it is chosen, and weighs in with its share alone
    w["correction"] = torch.tensor([0.0, 0.0, 0.3], dtype=torch.float64)
    assert torch.allclose(plain.moe(h, w, ff)[0], s[0] * expert(0) + s[2] * h[0])


# ---------------------------------------------------------------------------- the engine on the host
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: S.write_model(tmp_path_factory.mktemp(f"gapevik_{n}"), n) for n in ("A", "C")}


def host_engine(folder, tokens, page_size=16, max_requests=4):
    k = TorchReferenceKernels(torch.float32, "cpu")
    model = Model.from_folder(folder, dtype="float32", device="cpu", kernels=k)
    return Engine(model, cache_tokens=tokens, page_size=page_size, max_requests=max_requests)


def requests_for(folder, lens, seed):
    vocab = json.loads((folder / "config.json").read_text())["vocab"]
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("name", ["A", "C"])
def test_folder_round_trip_and_whole_prompts(folders, name):
    folder = folders[name]
    assert load_config(folder).to_dict() == S.CONFIGS[name][0]
    reqs = requests_for(folder, (47, 1, 20), 10)
    eng = host_engine(folder, 64 * 3)
    S.compare_with_plain(H.run_steps(eng, H.steps_whole(reqs)), folder, reqs, 2e-5)
    assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups


def test_the_residual_stream_after_every_layer(folders):
    folder = folders["A"]
    toks = requests_for(folder, (45,), 20)["r0"]
    cfg, tensors = S.folder_contents(str(folder))
    taps = []
    plain.forward(cfg, tensors, toks, taps=taps)
    eng = host_engine(folder, 64)
    seen = []
    eng.model.layer_tap = lambda i, h: seen.append(h.clone())
    H.run_steps(eng, H.steps_whole({"a": toks}))
    assert len(seen) == len(taps) == len(cfg["layers"])
    for i, h in enumerate(seen):
        assert float((h - taps[i]).abs().max()) <= 2e-5 * float(taps[i].abs().max()), f"layer {i}"


@pytest.mark.parametrize("name", ["A", "C"])
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


def test_caches_and_state_of_every_layer_run(folders):
    """Chunked attention and windowed latent attention get page groups of their own (the latent rows one plane); every
    layer run has its own cache, the borrowed ones too; convolutions and delta matrices live in state slots."""
    k = TorchReferenceKernels(torch.float32, "cpu")
    model = Model.from_config(GapevikConfig.from_dict(S.CONFIG_A), dtype="float32", device="cpu", kernels=k)
    specs = model.cache_specs()
    assert sorted(specs) == list(range(7))
    assert specs[0][0].window == Window("chunk", 20) and specs[3][0].window == Window("chunk", 20)
    assert specs[1][0].window == Window("sliding", 7) and specs[1][0].planes == 1 and specs[1][1] is None
    assert specs[0][1].shape == (2 * (4 + 2 * 2) * 24,)                   # two rows of the q, k and v columns
    assert specs[2][0] is None and specs[2][1].shape == (3 * 20 * 12 + 1 * (2 * 20 + 3 * 12),)


def test_pages_behind_a_window_go_back(folders):
    eng = host_engine(folders["A"], 256, page_size=8)
    toks = requests_for(folders["A"], (90,), 50)["r0"]
    H.run_steps(eng, [{"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [89]}], "end": []}])
    by_window = {k.window: g for g, k in enumerate(eng.storage.group_keys)}
    chunk = eng.cache.block_table("a", by_window[Window("chunk", 20)])
    assert [p >= 0 for p in chunk] == [False] * 10 + [True] * 2           # positions 80..89 live in pages 10 and 11
    slide = eng.cache.block_table("a", by_window[Window("sliding", 7)])
    assert [p >= 0 for p in slide] == [False] * 10 + [True] * 2           # position 90 will read 84..90


def test_a_state_slot_that_is_used_again_starts_at_zero(folders):
    eng = host_engine(folders["C"], 128, max_requests=1)
    reqs = requests_for(folders["C"], (30, 25), 60)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"], "want": [29]}], "end": ["r0"]},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"][:10], "want": [9]}], "end": []},
             {"step": 2, "entries": [{"id": "r1", "tokens": reqs["r1"][10:], "want": [0, 14]}], "end": ["r1"]}]
    S.compare_with_plain(H.run_steps(eng, steps), folders["C"], reqs, 2e-5)


def test_trace_replay_on_the_host(folders, tmp_path):
    import io
    import numpy as np
    from spite_b200.engine.trace import replay
    folder = folders["A"]
    reqs = requests_for(folder, (50, 21, 5), 70)
    steps = H.steps_mixed(reqs, {r: len(t) - 4 for r, t in reqs.items()}, seed=9)
    eng = host_engine(folder, H.max_tokens_of(steps), page_size=64)
    log = io.StringIO()
    replay(eng, [json.dumps(s) for s in steps], tmp_path / "out", log=log)
    assert log.getvalue().split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    vocab = S.CONFIG_A["vocab"]
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
