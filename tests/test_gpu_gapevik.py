"""Gapevik on the GPU.  First every new mechanism alone against loops written here from its equation (the short
convolution carried from step to step, the gated delta rule in prompts, portions and decoded tokens with a far token
and slots used again, capped scores on every attention kernel with windows, sinks and gates, the latent kernels with
halves paired, the per-head norm of a padded head, the router that chooses by corrected share with identity experts,
the heads' norm with a silu gate, the norm behind a sublayer that hands the stream on unnormed); then the engine in
float32 and bfloat16 against the plain implementation in every cut (whole, token by token, portions down to two
tokens, mixed batches in a pool whose pages and slots are used again, free pages poisoned), layer by layer, long
decoding, greedy generation through `LLM.generate`, `bin/trace_run` and the command line."""
import json
import math

import pytest
import torch

import gapevik_helpers as S
import helpers as H
import plain_gapevik as plain
from reference_kernels import TorchReferenceKernels
from spite_b200.cache import LayerCache, Window
from spite_b200.engine.batch import Segment, build_step_batch
from spite_b200.kernels.api import Routing
from spite_b200.parts import QkNorm, Rotation
from test_gpu_kernels import close, fill_cache, make_batch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# (a norm stands behind every sublayer: it brings whatever rounding a sublayer's output carries to unit size)
TOL = {"float32": 4e-5, "bfloat16": 2e-2}
KTOL = {torch.float32: 1e-5, torch.bfloat16: 1.2e-2}


def kernels(dtype):
    from spite_b200.kernels.cuda import CudaKernels
    return CudaKernels(dtype, DEV)


def step_batch(counts, slots, first=False):
    segs, off = [], 0
    for s, n in enumerate(counts):
        segs.append(Segment(s, slots[s], 0, n, off, first))
        off += n
    return build_step_batch(segs, [[0] * n for n in counts], [[] for _ in counts], [[[0]] * len(counts)], DEV), off


# ---------------------------------------------------------------------------- the short convolution
# (channels, taps, columns passed on, activation, output type, segments as token counts of three steps)
CONV_CASES = [
    (40, 4, 6, None, torch.bfloat16, [(19, 1, 7), (1, 1, 1), (40, 2, 1)]),
    (130, 3, 0, "silu", torch.float32, [(2, 1, 1), (1, 2, 33), (1, 1, 1)]),          # segments shorter than the taps reach back
    (7, 8, 3, "silu", torch.float32, [(3, 2, 2), (50, 1, 1)]),
    (256, 2, 8, None, torch.float32, [(17, 16, 15), (1, 1, 1)]),
    (33, 1, 5, "silu", torch.bfloat16, [(9, 1, 3)]),                                 # one tap: nothing is carried
]


@pytest.mark.parametrize("case", range(len(CONV_CASES)))
def test_short_convolution_carried_from_step_to_step(case):
    """Three steps over the same slots, dealt out of order, beside slots that hold leftovers: a token reads the rows of
    the steps before through the slot, the first tokens of a sequence read zeros, the columns behind the channels pass."""
    channels, taps, extra, act, out_dtype, segs = CONV_CASES[case]
    ks = kernels(torch.bfloat16 if out_dtype == torch.bfloat16 else torch.float32)
    n_slots = len(segs) + 2
    g = torch.Generator().manual_seed(500 + case)
    offset = 11
    state = torch.randn((n_slots, offset + (taps - 1) * channels + 5), generator=g).to(DEV)
    slots = torch.randperm(n_slots, generator=g)[:len(segs)].tolist()
    state[torch.tensor(slots)] = 0.0
    start = state.clone()
    w = torch.randn((channels, taps), generator=g)
    history = {s: torch.zeros((taps - 1, channels), dtype=torch.float64) for s in range(len(segs))}
    for step in range(3):
        counts = [sg[step] for sg in segs]
        batch, M = step_batch(counts, slots, step == 0)
        x = torch.randn((M, channels + extra + 3), generator=g)
        out = torch.full((M, channels + extra), 7.0, dtype=out_dtype, device=DEV)
        ks.short_conv(x.to(DEV), w.to(DEV), out, batch, state, channels=channels, activation=act, state_offset=offset)
        torch.cuda.synchronize()
        ref = torch.zeros((M, channels + extra), dtype=torch.float64)
        off = 0
        for s, n in enumerate(counts):
            rows = torch.cat([history[s], x[off:off + n, :channels].double()], 0)
            for i in range(n):
                y = sum(w[:, j].double() * rows[i + j] for j in range(taps))
                ref[off + i, :channels] = y * torch.sigmoid(y) if act == "silu" else y
            history[s] = rows[rows.shape[0] - (taps - 1):]
            off += n
        ref[:, channels:] = x[:, channels:channels + extra].double()
        close(out, ref, 1e-6 if out_dtype == torch.float32 else 8e-3, f"short convolution, step {step}")
    got = state.cpu()
    for s in range(len(segs)):
        assert torch.equal(got[slots[s], offset:offset + (taps - 1) * channels].view(taps - 1, channels).double(), history[s])
    keep = torch.ones_like(got, dtype=torch.bool)
    keep[torch.tensor(slots), offset:offset + (taps - 1) * channels] = False
    assert torch.equal(got[keep], start.cpu()[keep])          # nothing else in any slot was touched


def test_padding_rows_of_a_captured_step_come_out_as_the_first_row():
    """A captured decode step pads its rows with copies of its first row, slot included: the copies' rows are the
    first row's (their keys go to the same place of the cache), and the slot is renewed once."""
    ks = kernels(torch.float32)
    channels, taps = 70, 4
    g = torch.Generator().manual_seed(9)
    state = torch.randn((3, (taps - 1) * channels), generator=g).to(DEV)
    before = state.cpu().clone()
    w = torch.randn((channels, taps), generator=g)
    x = torch.randn((4, channels), generator=g)
    x[2] = x[0]; x[3] = x[0]
    batch, M = step_batch([1, 1, 1, 1], [2, 0, 2, 2])
    out = torch.empty((4, channels), dtype=torch.float32, device=DEV)
    ks.short_conv(x.to(DEV), w.to(DEV), out, batch, state, channels=channels)
    torch.cuda.synchronize()
    for s, slot in ((0, 2), (1, 0)):
        rows = torch.cat([before[slot].view(taps - 1, channels), x[s:s + 1]], 0).double()
        ref = sum(w[:, j].double() * rows[j] for j in range(taps))
        close(out[s], ref, 1e-6, "row")
        assert torch.equal(state[slot].cpu().view(taps - 1, channels), rows[1:].float())
    assert torch.equal(out[2], out[0]) and torch.equal(out[3], out[0])
    assert torch.equal(state[1].cpu(), before[1])


# ---------------------------------------------------------------------------- the gated delta rule
def delta_loops(q, k, v, zb, za, a_log, dt, q_scale, S):
    """One head, token by token, in float64: (outputs [T, vdim], S)."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=torch.float64)
    for t in range(T):
        kt = k[t] / math.sqrt(float(k[t] @ k[t]) + 1e-6)
        qt = q[t] / math.sqrt(float(q[t] @ q[t]) + 1e-6) * q_scale
        beta = 1.0 / (1.0 + math.exp(-float(zb[t])))
        z = float(za[t]) + dt
        g = math.exp(-math.exp(a_log) * (max(z, 0.0) + math.log1p(math.exp(-abs(z)))))
        S = g * S
        u = beta * (v[t] - S.T @ kt)
        S = S + torch.outer(kt, u)
        out[t] = S.T @ qt
    return out, S


# (heads, kv heads, dim, vdim, segments as token counts of three steps)
DELTA_CASES = [
    (3, 1, 20, 12, [(19, 1, 7), (1, 1, 1), (40, 2, 1)]),
    (1, 1, 40, 70, [(33, 1, 1), (5, 3, 2)]),
    (4, 2, 64, 64, [(70, 1, 1), (1, 1, 30)]),
    (2, 2, 136, 40, [(12, 1, 2)]),
    (2, 1, 33, 5, [(25, 1, 1), (2, 2, 2)]),
    (2, 2, 256, 40, [(9, 1, 1)]),
    (6, 3, 8, 8, [(30, 1, 1), (1, 1, 1)]),
    (1, 1, 300, 24, [(7, 1, 3)]),
    (2, 1, 72, 36, [(32, 33, 64), (97, 1, 31), (1, 65, 2)]),
    (1, 1, 512, 9, [(6, 1, 2)]),
]


@pytest.mark.parametrize("split", [False, True], ids=["eight columns a warp", "rows split further"])
@pytest.mark.parametrize("case", range(len(DELTA_CASES)))
def test_delta_rule_in_prompts_portions_and_decoded_tokens(case, split):
    """Three steps over the same slots: every segment goes on from the matrices the step before left, slots are dealt
    out of order, other slots hold leftovers that nothing touches.  Against float64 loops, in both forms of the kernel
    (a warp on eight value columns, as decode steps run it, and on fewer with the key rows split further)."""
    heads, kvh, dim, vdim, segs = DELTA_CASES[case]
    ks = kernels(torch.float32)
    n_slots = len(segs) + 2
    g = torch.Generator().manual_seed(300 + case)
    offset = 8
    state = torch.randn((n_slots, offset + heads * dim * vdim + 3), generator=g).to(DEV)
    slots = torch.randperm(n_slots, generator=g)[:len(segs)].tolist()
    state[torch.tensor(slots)] = 0.0
    start = state.cpu().clone()
    a_log = torch.randn(heads, generator=g) * 0.7 - 1.0
    dt = torch.randn(heads, generator=g)
    carried = {s: [torch.zeros(dim, vdim, dtype=torch.float64) for _ in range(heads)] for s in range(len(segs))}
    q_scale = dim ** -0.5
    cols = (3, 3 + kvh * dim, 3 + 2 * kvh * dim, 5 + 2 * kvh * dim + heads * vdim, 5 + 2 * kvh * dim + heads * vdim + heads)
    width = cols[4] + heads + 2
    for step in range(3):
        counts = [sg[step] for sg in segs]
        batch, M = step_batch(counts, slots, step == 0)
        x = torch.randn((M, width), generator=g)
        x[:, cols[3]:] *= 3.0
        out = torch.empty((M, heads * vdim), dtype=torch.float32, device=DEV)
        ks.delta_scan(x.to(DEV), out, batch, state, heads=heads, kv_heads=kvh, dim=dim, vdim=vdim, columns=cols,
                      a_log=a_log.to(DEV), dt_bias=dt.to(DEV), q_scale=q_scale, state_offset=offset, split_rows=split)
        torch.cuda.synchronize()
        ref = torch.zeros(M, heads, vdim, dtype=torch.float64)
        off, xd = 0, x.double()
        for s, n in enumerate(counts):
            rows = xd[off:off + n]
            for a in range(heads):
                gk = a // (heads // kvh)
                o, S1 = delta_loops(rows[:, cols[0] + gk * dim:cols[0] + (gk + 1) * dim], rows[:, cols[1] + gk * dim:cols[1] + (gk + 1) * dim],
                                    rows[:, cols[2] + a * vdim:cols[2] + (a + 1) * vdim], rows[:, cols[3] + a], rows[:, cols[4] + a],
                                    float(a_log[a]), float(dt[a]), q_scale, carried[s][a])
                carried[s][a] = S1
                ref[off:off + n, a] = o
            off += n
        close(out.view(M, heads, vdim), ref, 2e-5, f"delta rule, step {step}")
    got = state.cpu()
    for s in range(len(segs)):
        for a in range(heads):
            close(got[slots[s], offset + a * dim * vdim:offset + (a + 1) * dim * vdim].view(dim, vdim), carried[s][a], 2e-5, "S")
    keep = torch.ones_like(got, dtype=torch.bool)
    keep[torch.tensor(slots), offset:offset + heads * dim * vdim] = False
    assert torch.equal(got[keep], start[keep])


def test_delta_rule_keeps_a_token_from_hundreds_of_steps_back():
    """No decay to speak of, one token written with beta near one along a key of its own at position 2, every later
    key orthogonal to it: 700 tokens later a query along that key reads that token's value, in one prompt, decoded
    token by token, and in portions."""
    heads, dim, vdim, T = 2, 16, 8, 703
    ks = kernels(torch.float32)
    g = torch.Generator().manual_seed(4)
    cols = (0, dim, 2 * dim, 2 * dim + heads * vdim, 2 * dim + heads * vdim + heads)
    x = torch.zeros((T, cols[4] + heads))
    x[:, cols[1]:cols[1] + dim - 1] = torch.randn((T, dim - 1), generator=g)          # keys that leave the last direction alone
    x[:, cols[0]:cols[0] + dim] = torch.randn((T, dim), generator=g)
    x[:, cols[2]:cols[3]] = torch.randn((T, heads * vdim), generator=g)
    x[:, cols[3]:cols[3] + heads] = -2.0                                               # weak writes ...
    x[:, cols[4]:] = -30.0                                                             # ... and softplus(-30) = 0: no decay
    x[2, cols[1]:cols[1] + dim] = 0.0; x[2, cols[1] + dim - 1] = 5.0                   # the far token: its own key,
    x[2, cols[3]:cols[3] + heads] = 30.0                                               # written whole
    x[T - 1, cols[0]:cols[0] + dim] = 0.0; x[T - 1, cols[0] + dim - 1] = 3.0           # the last query looks along it
    a_log, dt = torch.zeros(heads), torch.zeros(heads)
    far = x[2, cols[2]:cols[3]].view(heads, vdim) * dim ** -0.5
    for cut, split in (([T], False), ([T], True), ([3] + [1] * (T - 3), False), ([2, 64, 5, 300, 31, 301], True)):
        state = torch.zeros((1, heads * dim * vdim), device=DEV)
        off = 0
        for n in cut:
            batch, _ = step_batch([n], [0], off == 0)
            out = torch.empty((n, heads * vdim), dtype=torch.float32, device=DEV)
            ks.delta_scan(x[off:off + n].contiguous().to(DEV), out, batch, state, heads=heads, kv_heads=1, dim=dim, vdim=vdim,
                          columns=cols, a_log=a_log.to(DEV), dt_bias=dt.to(DEV), q_scale=dim ** -0.5, split_rows=split)
            off += n
        close(out[-1].view(heads, vdim), far.double(), 1e-4, f"the far token's value, cut {cut[:3]}")


# ---------------------------------------------------------------------------- capped scores, kernel by kernel
def capped_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, window, cap, sinks, gates):
    """p_j = exp(cap tanh(s_j / cap)) / (exp(sink_h) + sum over the visible j'), times the gate; float64 loops."""
    out = torch.zeros(q.shape[:2] + (v_all[0].shape[-1],), dtype=torch.float64)
    group, off = nq // nkv, 0
    for s, (start, n) in enumerate(specs):
        for t in range(n):
            pos = start + t
            lo = window.lowest_visible(pos)
            for h in range(nq):
                sc = (k_all[s][lo:pos + 1, h // group].double() @ q[off + t, h].double()) * scale
                if cap is not None:
                    sc = cap * torch.tanh(sc / cap)
                m = float(sc.max()) if sinks is None else max(float(sc.max()), float(sinks[h]))
                e = torch.exp(sc - m)
                den = e.sum() + (0.0 if sinks is None else math.exp(float(sinks[h]) - m))
                o = (e / den) @ v_all[s][lo:pos + 1, h // group].double()
                out[off + t, h] = o * (1.0 if gates is None else float(gates[off + t, h]))
        off += n
    return out


# (kernel library that must serve the call, dtype, query heads, kv heads, row size, page size, window, cap, segments)
CAP_CASES = [
    ("attention", torch.float32, 5, 1, 24, 16, ("chunk", 50), 3.0, [(0, 1), (0, 60), (130, 1), (99, 3)]),
    ("attention", torch.bfloat16, 6, 3, 24, 16, ("sliding", 33), 5.0, [(0, 1), (0, 40), (130, 1), (61, 7)]),
    ("attention_mma", torch.bfloat16, 4, 2, 48, 16, ("chunk", 200), 4.0, [(0, 1), (199, 1), (200, 1), (398, 3), (1500, 1)]),
    ("attention_rows", torch.bfloat16, 6, 2, 32, 32, ("sliding", 40), 2.0, [(0, 45), (100, 30), (0, 12), (78, 4)]),
    ("attention_decode", torch.bfloat16, 8, 2, 64, 64, ("sliding", 100), 6.0, [(0, 1), (63, 1), (64, 1), (3000, 1), (517, 2)]),
    ("attention_decode", torch.bfloat16, 8, 4, 128, 64, ("chunk", 100), 4.0, [(99, 1), (100, 1), (299, 1), (250, 1)]),
    ("attention_tc", torch.bfloat16, 6, 2, 64, 64, ("chunk", 200), 5.0, [(0, 300), (150, 130), (0, 70)]),
    ("attention_tc", torch.bfloat16, 4, 1, 128, 64, ("sliding", 70), 3.0, [(0, 140), (900, 64)]),
]


@pytest.mark.parametrize("case", range(len(CAP_CASES)))
def test_capped_scores_in_every_attention_kernel(case):
    """Scores of both signs well beyond the cap, so that the cap shapes every softmax; sinks and gates beside it; one
    row whose query is aligned with the first key it may see (a window's or a chunk's edge): the key just outside
    would have taken the row over."""
    library, dtype, nq, nkv, hd, P, win, cap, specs = CAP_CASES[case]
    ks = kernels(dtype)
    window = Window(*win)
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 3
    batch, tables = make_batch(specs, P, n_pages, 160 + case, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(161 + case)
    k_all = [torch.randn((s + n, nkv, hd), generator=g).to(dtype) for s, n in specs]
    v_all = [torch.randn((s + n, nkv, hd), generator=g).to(dtype) for s, n in specs]
    q = torch.randn((M, nq, hd), generator=g) * 2.0
    last_pos = specs[-1][0] + specs[-1][1] - 1
    first_seen = window.lowest_visible(last_pos)
    q[M - 1, nq - 1] = k_all[-1][first_seen, nkv - 1].float() * (12.0 / math.sqrt(hd))
    if first_seen > 0:                                       # the key just outside is aligned even better
        k_all[-1][first_seen - 1, nkv - 1] = k_all[-1][first_seen, nkv - 1] * 1.5
    q = q.to(dtype)
    sinks = torch.randn(nq, generator=g) * 1.5
    gates = torch.rand((M, nq), generator=g)
    kv = torch.zeros((2, n_pages, nkv, P, hd), dtype=dtype)
    fill_cache(kv, tables, [(s + n, 0) for s, n in specs], k_all, v_all, P)
    out = torch.empty((M, nq * hd), dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks.paged_attention(q.reshape(M, nq * hd).to(DEV), out, batch, LayerCache(0, kv.to(DEV), None, P, False),
                       num_heads=nq, window=window, softmax_scale=scale, head_sinks=sinks.to(DEV), head_gates=gates.to(DEV),
                       score_softcap=cap)
    torch.cuda.synchronize()
    assert not ks.errors()
    assert ks.launches_by_library[library] > 0, dict(ks.launches_by_library)
    ref = capped_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, window, cap, sinks, gates)
    close(out.view(M, nq, hd), ref, KTOL[dtype], f"attention with capped scores ({library})")
    assert float((capped_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, window, None, sinks, gates) - ref).abs().max()) > 0.05
    if first_seen > 0:
        wider = Window("full", 0)
        assert float((capped_attention_reference(q, k_all, v_all, specs, nq, nkv, scale, wider, cap, sinks, gates) - ref).abs().max()) > 1e-2


# ---------------------------------------------------------------------------- the prepare kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,kd,hd,rd", [(4, 2, 24, 32, 6), (3, 3, 16, 32, 16), (2, 1, 10, 12, 4)])
def test_prepare_norms_a_padded_head_over_its_own_elements(dtype, nq, nkv, kd, hd, rd):
    """A head of kd elements in a row of hd (zeros behind it): the norm's mean is over kd, gains before the rotation of
    neighbouring pairs of the first rd elements, the padding stays zero."""
    ks, ref = kernels(dtype), TorchReferenceKernels(dtype, "cpu")
    P, specs = 16, [(0, 5), (37, 1), (20, 3)]
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 2
    batch, tables = make_batch(specs, P, n_pages, 31, DEV)
    batch_c, _ = make_batch(specs, P, n_pages, 31, "cpu")
    M = batch.n_tokens
    g = torch.Generator().manual_seed(32)
    qkv = torch.randn((M, nq + 2 * nkv, hd), generator=g)
    qkv[:, :nq + nkv, kd:] = 0.0
    qkv = torch.cat([qkv.reshape(M, -1), torch.randn((M, 8), generator=g)], 1).to(dtype)
    gain = lambda: torch.cat([1.0 + 0.3 * torch.randn(kd, generator=g), torch.zeros(hd - kd)])
    qg, kg = gain(), gain()
    freq = torch.tensor([50.0 ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float32)
    outs = []
    for k_set, dev, b in ((ks, DEV, batch), (ref, "cpu", batch_c)):
        kv = torch.zeros((2, n_pages, nkv, P, hd), dtype=dtype, device=dev)
        q_out = torch.empty((M, nq * hd), dtype=dtype, device=dev)
        gates = torch.empty((M, nq), dtype=torch.float32, device=dev)
        k_set.qk_prepare(qkv.to(dev), q_out, b, LayerCache(0, kv, None, P, True), num_heads=nq,
                         rotation=Rotation(freq.to(dev), "neighbours", rd), qk_norm=QkNorm(1e-5, True, qg.to(dev), kg.to(dev)),
                         temperature=None, gates_out=gates, norm_dim=kd)
        outs.append((q_out.float().cpu(), kv.float().cpu(), gates.cpu()))
    for a, b, what in zip(outs[0], outs[1], ("q", "cache", "gates")):
        close(a, b.double(), 2e-6 if dtype == torch.float32 else 8e-3, what)
    # the mean is over kd elements: written out for the elements behind the rotating ones
    one = outs[0][0].view(M, nq, hd)
    x = qkv[:, :nq * hd].float().view(M, nq, hd)
    want = x[..., rd:kd] / torch.sqrt(x[..., :kd].pow(2).sum(-1, keepdim=True) / kd + 1e-5) * qg[rd:kd]
    if kd > rd:
        close(one[..., rd:kd], want.double(), 2e-6 if dtype == torch.float32 else 8e-3, "norm over the head's own elements")
    assert float(one[..., kd:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,dn,dr,rq,rkv,row", [(3, 16, 8, 40, 40, 48), (5, 12, 6, 22, 30, 36), (8, 32, 32, 64, 96, 128)])
def test_latent_kernels_pair_the_halves(dtype, nq, dn, dr, rq, rkv, row):
    ks, ref = kernels(dtype), TorchReferenceKernels(dtype, "cpu")
    P, specs = 16, [(0, 5), (37, 1), (20, 3)]
    n_pages = sum(-(-(s + n) // P) for s, n in specs) + 2
    batch, _ = make_batch(specs, P, n_pages, 41, DEV)
    batch_c, _ = make_batch(specs, P, n_pages, 41, "cpu")
    M = batch.n_tokens
    g = torch.Generator().manual_seed(42)
    down = torch.randn((M, rq + rkv + dr + nq + 3), generator=g)
    q = torch.randn((M, nq * (dn + dr)), generator=g).to(dtype)
    freq = torch.tensor([100.0 ** (-2.0 * i / dr) for i in range(dr // 2)], dtype=torch.float32)
    qg, kg = 1.0 + 0.3 * torch.randn(rq, generator=g), 1.0 + 0.3 * torch.randn(rkv, generator=g)
    outs = []
    for k_set, dev, b in ((ks, DEV, batch), (ref, "cpu", batch_c)):
        rot = Rotation(freq.to(dev), "halves", dr)
        kv = torch.zeros((1, n_pages, 1, P, row), dtype=dtype, device=dev)
        cq = torch.empty((M, rq), dtype=dtype, device=dev)
        gates = torch.empty((M, nq), dtype=torch.float32, device=dev)
        k_set.latent_prepare(down.to(dev), cq, b, LayerCache(0, kv, None, P, True), q_rank=rq, kv_rank=rkv, rotation=rot,
                             q_gain=qg.to(dev), kv_gain=kg.to(dev), eps=1e-5, num_gates=nq, gates_out=gates)
        qa = torch.zeros((M, nq * row), dtype=dtype, device=dev)
        rows = torch.empty((nq * M,), dtype=torch.int32, device=dev)
        offs = torch.empty((nq + 1,), dtype=torch.int32, device=dev)
        qn = torch.empty((nq * M, dn), dtype=dtype, device=dev)
        k_set.latent_queries(q.to(dev), qa, b, num_heads=nq, head_dim=dn, kv_rank=rkv, rotation=rot, rows_out=rows,
                             offsets_out=offs, sorted_out=qn)
        outs.append((cq.float().cpu(), kv.float().cpu(), gates.cpu(), qa.float().cpu(), qn.float().cpu()))
    for a, b, what in zip(outs[0], outs[1], ("query latent", "cache rows", "gates", "query rows", "unrotated parts")):
        close(a, b.double(), 2e-6 if dtype == torch.float32 else 8e-3, what)
    # element i turns with element i + dr/2: written out for one token and head
    t, h, i = M - 1, nq - 1, dr // 2 - 1
    pos = specs[-1][0] + specs[-1][1] - 1
    ang = pos * float(freq[i])
    u, v = float(q.view(M, nq, dn + dr)[t, h, dn + i]), float(q.view(M, nq, dn + dr)[t, h, dn + i + dr // 2])
    got = outs[0][3].view(M, nq, row)[t, h]
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert abs(float(got[rkv + i]) - (u * math.cos(ang) - v * math.sin(ang))) < tol
    assert abs(float(got[rkv + i + dr // 2]) - (v * math.cos(ang) + u * math.sin(ang))) < tol


# ---------------------------------------------------------------------------- the router and the identity experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,d,E,I,top", [(1, 64, 4, 1, 2), (23, 96, 6, 2, 3), (300, 128, 8, 2, 2), (40, 100, 1, 1, 1), (70, 72, 3, 0, 3)])
def test_router_by_corrected_share_and_identity_experts(dtype, M, d, E, I, top):
    """The choice is by softmax share plus correction (corrections large enough to change it), the weight is the
    share alone; the tokens of the real experts come first in the sorted order; identity experts return the token."""
    ks = kernels(dtype)
    g = torch.Generator().manual_seed(M + d)
    x = torch.randn((M, d), generator=g).to(dtype)
    wr = torch.randn((E + I, d), generator=g) * 0.3
    bias = torch.randn(E + I, generator=g) * 0.2
    r = ks.moe_route(x.to(DEV), wr.to(DEV), top, want_logits=True, scoring="softmax_biased", choice_bias=bias.to(DEV))
    torch.cuda.synchronize()
    logits = x.double() @ wr.double().T
    close(r.logits, logits, 1e-5, "router logits")
    share = torch.softmax(r.logits.cpu().double(), -1)                      # (the kernel's own logits: no close call is judged twice)
    choice = share + bias.double()
    order = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    margin = torch.sort(choice, dim=-1, descending=True).values
    clear = (margin[:, :-1] - margin[:, 1:]).amin(-1) > 1e-5 if E + I > 1 else torch.ones(M, dtype=torch.bool)
    ids = r.expert_ids.cpu().long().T
    assert torch.equal(ids[clear], order[clear])
    assert int(clear.sum()) >= M * 0.9
    w = r.weights.cpu().double().T
    close(w, share.gather(1, ids), 1e-5, "weights are the shares")
    assert bool(((share + bias.double()).gather(1, ids)[:, :-1] >= (share + bias.double()).gather(1, ids)[:, 1:] - 1e-6).all())
    for s in range(top):
        offs, rows = r.offsets[s].cpu().tolist(), r.sorted_rows[s].cpu().tolist()
        assert offs[0] == 0 and offs[-1] == M and len(offs) == E + I + 1
        for e in range(E + I):
            mine = rows[offs[e]:offs[e + 1]]
            assert mine == sorted(mine) and all(int(ids[t, s]) == e for t in mine)
        close(r.sorted_weights[s], r.weights[s][r.sorted_rows[s].long()].double(), 0.0, "weights in the sorted order")
    # identity experts: out (+)= weight * x for the slots that drew one
    wi = (r.weights.cpu().double() * (r.expert_ids.cpu() >= E)).sum(0)
    ref = wi[:, None] * x.double()
    out = torch.full((M, d), 5.0, dtype=torch.float32, device=DEV)
    ks.moe_identity(x.to(DEV), r, E, out, accumulate=False)
    close(out, ref, 1e-6, "identity experts, stored")
    ks.moe_identity(x.to(DEV), r, E, out, accumulate=True)
    close(out, 2 * ref, 1e-6, "identity experts, added")
    if I and M > 20:
        assert float(wi.max()) > 0                                          # some token drew an identity expert


# ---------------------------------------------------------------------------- between heads and output projection, and behind a sublayer
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_heads_norm_with_a_silu_gate(dtype):
    ks = kernels(dtype)
    g = torch.Generator().manual_seed(3)
    M, heads, size = 9, 3, 20
    x = torch.randn((M, heads * size), generator=g)
    gates = torch.randn((M, heads * size + 7), generator=g) * 2
    gain = (1.0 + 0.3 * torch.randn(size, generator=g)).repeat(heads)
    out = torch.empty((M, heads * size), dtype=dtype, device=DEV)
    ks.head_norm_gate(x.to(DEV), out, heads=heads, size=size, gates=gates.to(DEV), gate_column=4, gain=gain.to(DEV), eps=1e-5,
                      gate_activation="silu")
    v = x.double().view(M, heads, size)
    v = (v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)).view(M, -1) * gain.double()
    z = gates[:, 4:4 + heads * size].double()
    close(out, v * z * torch.sigmoid(z), 1e-6 if dtype == torch.float32 else 8e-3, "heads' norm, gain, silu gate")


@pytest.mark.parametrize("d", [72, 320, 1000, 4100])
def test_norm_behind_a_sublayer_hands_the_stream_on_unnormed(d):
    ks = kernels(torch.bfloat16)
    g = torch.Generator().manual_seed(d)
    M = 7
    y, h, gain = torch.randn((M, d), generator=g), torch.randn((M, d), generator=g), 1.0 + 0.3 * torch.randn(d, generator=g)
    hd, nxt = h.to(DEV), torch.empty((M, d), dtype=torch.bfloat16, device=DEV)
    ks.rms_norm_residual(y.to(DEV), gain.to(DEV), 1e-5, 0.5, hd, next_out=nxt)
    ref = h.double() + 0.5 * y.double() / torch.sqrt(y.double().pow(2).mean(-1, keepdim=True) + 1e-5) * gain.double()
    close(hd, ref, 1e-6, "the stream")
    assert torch.equal(nxt, hd.to(torch.bfloat16))
    c = torch.empty((M, d), dtype=torch.bfloat16, device=DEV)
    ks.cast_rows(hd, c)
    assert torch.equal(c, nxt)


# ---------------------------------------------------------------------------- the engine
@pytest.fixture(scope="module", params=list(S.CONFIGS))
def folder(request, tmp_path_factory):
    return S.write_model(tmp_path_factory.mktemp(f"gapevik_{request.param}"), request.param), request.param


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request, folder, tmp_path_factory):
    from spite_b200.engine import Model
    path, name = folder
    dtype = request.param
    if dtype == "bfloat16":                                  # (see `write_model`: no choice of experts is left to rounding)
        path = S.write_model(tmp_path_factory.mktemp(f"gapevik_{name}_settled"), name, settled_routing=True)
    model = Model.from_folder(path, dtype=dtype, device=DEV)
    vocab = model.plan.vocab_size
    lengths = {"a": 210 if name == "B" else 97, "b": 40, "c": 37, "d": 66, "e": 1, "f": 21}
    requests = {r: H.random_tokens(vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    return path, model, requests, TOL[dtype], dtype


def _engine(model, steps, page_size):
    from spite_b200.engine import Engine
    return Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=page_size, max_requests=4)


def poison_free_pages(engine):
    """Whatever a free page held last is not finite: a kernel that reads a masked key of a reused page shows it."""
    for g, pool in enumerate(engine.cache.pools):
        if pool._free:
            engine.storage.kv[g][:, :, torch.tensor(pool._free, device=DEV)] = float("nan")


def test_every_cut_gives_the_logits_of_the_whole_sequence(setup):
    path, model, requests, tol, dtype = setup
    n_prompt = {r: max(1, len(t) - 9) for r, t in requests.items()}
    cuts = {"whole": (H.steps_whole(requests), 64), "whole, small pages": (H.steps_whole(requests), 16),
            "last 32 decoded": (H.steps_last_decoded(requests, 32), 64),
            "portions": (H.steps_portions(requests, seed=4), 64),
            "portions of 2 and 3": (H.steps_portions(requests, seed=5, sizes=(2, 3)), 16),
            "mixed": (H.steps_mixed(requests, n_prompt, seed=6), 64),
            "mixed, small pages": (H.steps_mixed(requests, n_prompt, seed=7, sizes=(2, 5, 17, 40)), 16)}
    results = {}
    for what, (steps, page) in cuts.items():
        eng = _engine(model, steps, page)
        results[what] = H.run_steps(eng, steps, before_step=poison_free_pages)
        S.compare_with_plain(results[what], path, requests, tol)
        eng.check()
        assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups, what
    if dtype == "float32":
        H.assert_cuts_identical(results)


def test_the_residual_stream_layer_by_layer(setup):
    path, model, requests, tol, dtype = setup
    cfg, tensors = S.folder_contents(str(path))
    toks = requests["c"]
    layers = []
    plain.forward(cfg, tensors, toks, torch.float64, taps=layers)
    seen = []
    model.layer_tap = lambda i, h: seen.append(h.double().cpu())
    try:
        steps = H.steps_whole({"c": toks})
        H.run_steps(_engine(model, steps, 64), steps)
    finally:
        model.layer_tap = None
    assert len(seen) == len(layers) == len(cfg["layers"])
    for i, h in enumerate(seen):
        err = float((h - layers[i]).abs().max()) / float(layers[i].abs().max())
        assert err <= (4e-5 if dtype == "float32" else 5e-2), f"layer {i}: {err:.3e}"


def test_long_decoding_after_a_short_prompt(setup):
    """Three prompt tokens, then 160 tokens one by one (decode steps replayed from CUDA graphs, pages taken one after
    the other, every chunk and window of the configuration crossed while decoding)."""
    path, model, requests, tol, dtype = setup
    reqs = {"long": H.random_tokens(model.plan.vocab_size, 163, 77)}
    steps = H.steps_last_decoded(reqs, 160)
    eng = _engine(model, steps, 16)
    S.compare_with_plain(H.run_steps(eng, steps), path, reqs, tol)
    assert eng.graph_replays > 100


def test_decode_steps_of_several_requests_from_graphs(setup):
    """Three requests decode side by side, one ends early: the captured steps' padding rows (copies of the first row,
    slot included) leave convolutions, matrices and caches as they were."""
    path, model, requests, tol, dtype = setup
    reqs = {r: requests[r][:n] for r, n in (("b", 40), ("c", 30), ("f", 21))}
    steps = [{"entries": [{"id": r, "tokens": t[:5], "want": list(range(5))} for r, t in reqs.items()], "end": []}]
    for i in range(5, 40):
        live = [(r, t) for r, t in reqs.items() if i < len(t)]
        steps.append({"entries": [{"id": r, "tokens": [t[i]], "want": [0]} for r, t in live],
                      "end": [r for r, t in live if i == len(t) - 1]})
    for i, s in enumerate(steps):
        s["step"] = i
    eng = _engine(model, steps, 16)
    S.compare_with_plain(H.run_steps(eng, steps), path, reqs, tol)
    assert eng.graph_replays > 20


def test_greedy_generation_through_the_entry_point(setup):
    """`LLM.generate` (scheduler, sampler, engine): the tokens are the plain implementation's argmax at every
    step where its best two logits are not within rounding of each other."""
    from spite_b200 import LLM
    path, model, requests, tol, dtype = setup
    cfg, tensors = S.folder_contents(str(path))
    prompts = [requests["b"][:30], requests["c"][:7], requests["f"][:2], requests["d"][:50]]
    llm = LLM(model, cache_tokens=4 * 128, page_size=16, max_requests=3, max_batch_tokens=24)
    outs = llm.generate(prompts, max_tokens=12, temperature=0.0)
    compared = 0
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        toks = list(prompt)
        for tok in out:
            row = plain.forward(cfg, tensors, toks)[-1]
            top2 = torch.topk(row, 2).values
            if float(top2[0] - top2[1]) > 2 * max(tol, 5e-2 if dtype == "bfloat16" else 0) * float(row.abs().max()):
                assert tok == int(torch.argmax(row)), f"after {len(toks)} tokens"
                compared += 1
            toks.append(tok)                                 # follow the engine's own sequence
    assert compared >= (12 if dtype == "float32" else 4)


def test_trace_replay_program(folder, tmp_path):
    """`bin/trace_run` as a program: a mixed schedule in, logits files out, equal to the plain implementation."""
    import subprocess, sys
    import numpy as np
    from pathlib import Path
    path, name = folder
    vocab = json.loads((path / "config.json").read_text())["vocab"]
    requests = {r: H.random_tokens(vocab, n, 90 + i) for i, (r, n) in enumerate({"a": 70, "b": 33, "c": 5}.items())}
    steps = H.steps_mixed(requests, {r: len(t) - 4 for r, t in requests.items()}, seed=9)
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(path), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", str(H.max_tokens_of(steps))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    pos, got = {}, {}
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
        i = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = torch.from_numpy(rows[i].copy())
                i += 1
            pos[e["id"]] = base + len(e["tokens"])
        assert i == rows.shape[0]
    S.compare_with_plain(got, path, requests, 4e-5)


def test_the_command_line_runs_a_gapevik_folder(tmp_path):
    """`spite random`, `spite run` (greedy, float32: the plain implementation's tokens) and `spite bench`."""
    import subprocess, sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    spite = lambda *a: subprocess.run([sys.executable, str(root / "bin" / "spite")] + [str(x) for x in a],
                                      capture_output=True, text=True, timeout=900)
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(S.CONFIG_A))
    model = tmp_path / "model"
    assert spite("random", "--config", cfg_file, "--out", model, "--seed", 3, "--std", 0.08).returncode == 0
    cfg, W = plain.load_folder(model)
    prompt = H.random_tokens(211, 17, 2)
    proc = spite("run", "-m", model, "-p", " ".join(map(str, prompt)), "--max-tokens", 6, "--temperature", 0,
                 "--dtype", "fp32", "--page-size", 16, "--num-pages", 8)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == S.generate_greedy(cfg, W, prompt, 6)
    proc = spite("bench", "-m", model, "--n-prompt", 40, "--n-tokens", 12, "--n-runs", 2, "--json", "--dtype", "bf16")
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads(proc.stdout)
    assert report["decode_tps"] > 0 and report["prefill_tps"] > 0
