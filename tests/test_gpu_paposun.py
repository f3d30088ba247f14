"""Paposun on the GPU.  First every new mechanism alone against loops written here from its equation (the matrix
memory's scan in prompts, portions and decoded tokens with far tokens, small queries and state slots used again; the
heads' norm with gain and gate; the norm that follows a sublayer, with the stream's sum and the next norm; biases,
the rotation of a head's leading elements and queries alone in the prepare kernel; gelu in every product kernel);
then the engine in float32 and bfloat16 against the plain implementation in every cut (whole, token by token,
portions down to two tokens, mixed batches in a pool whose pages and slots are used again, free pages poisoned),
layer by layer, long decoding, greedy generation through `LLM.generate`, `bin/trace_run` and the command line."""
import json
import math

import pytest
import torch

import helpers as H
import paposun_helpers as S
import plain_paposun as plain
from spite_b200.cache import LayerCache, Window
from spite_b200.parts import Rotation
from test_gpu_kernels import close, make_batch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# (a norm stands behind every sublayer: it brings whatever rounding a sublayer's output carries to unit size, so the
# float32 engine sits a little further from float64 than in designs that norm only in front)
TOL = {"float32": 4e-5, "bfloat16": 2e-2}


def kernels(dtype):
    from spite_b200.kernels.cuda import CudaKernels
    return CudaKernels(dtype, DEV)


# ---------------------------------------------------------------------------- the matrix memory's scan
def memory_loops(q, k, v, a, c, bi, bf, cap, q_scale, S, n, m):
    """One head, token by token, in float64: (outputs [T, vdim], S, n, m).  a, c are the gates' pre-activations."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=torch.float64)
    for t in range(T):
        i = cap * math.tanh((float(a[t]) + bi) / cap)
        z = cap * math.tanh((float(c[t]) + bf) / cap)
        f = -math.log1p(math.exp(-z))
        m_new = max(f + m, i)
        keep, take = math.exp(f + m - m_new), math.exp(i - m_new)
        S = keep * S + take * torch.outer(k[t], v[t])
        n = keep * n + take * k[t]
        m = m_new
        qt = q[t] * q_scale
        out[t] = (S.T @ qt) / (max(abs(float(n @ qt)), math.exp(-m)) + 1e-6)
    return out, S, n, m


# (heads, dim, vdim, cap, q size, gate size, segments as token counts of three steps)
SCAN_CASES = [
    (3, 20, 12, 10.0, 1.0, 2.0, [(19, 1, 7), (1, 1, 1), (40, 2, 1)]),
    (1, 40, 70, 4.0, 1.0, 4.0, [(33, 1, 1), (5, 3, 2)]),
    (2, 64, 64, 15.0, 1.0, 3.0, [(70, 1, 1), (1, 1, 30)]),
    (1, 136, 32, 15.0, 1.0, 3.0, [(12, 1, 2)]),
    (2, 33, 5, 30.0, 1.0, 20.0, [(25, 1, 1), (2, 2, 2)]),
    (2, 256, 40, 8.0, 1.0, 2.0, [(9, 1, 1)]),
    (4, 8, 8, 2.0, 0.01, 1.0, [(30, 1, 1), (1, 1, 1)]),         # tiny queries: the denominator is exp(-m), so the maximum's start at 0 shows
    (1, 300, 24, 6.0, 1.0, 2.0, [(7, 1, 3)]),
    (2, 72, 36, 12.0, 1.0, 3.0, [(32, 33, 64), (97, 1, 31), (1, 65, 2)]),     # portions that end on, before and behind the edges of groups of 32 tokens
    (1, 512, 33, 9.0, 1.0, 2.0, [(34, 3, 1)]),
]


@pytest.mark.parametrize("chunked", [False, True], ids=["token by token", "32 tokens at a time"])
@pytest.mark.parametrize("case", range(len(SCAN_CASES)))
def test_memory_scan_in_prompts_portions_and_decoded_tokens(case, chunked):
    """Three steps over the same slots: every segment goes on from the state the step before left, slots are dealt out
    of order, one slot holds another request's leftovers before it is cleared and taken.  Against float64 loops, with
    the kernel that walks token by token and with the one that takes 32 tokens at a time."""
    heads, dim, vdim, cap, q_size, gate_size, segs = SCAN_CASES[case]
    ks = kernels(torch.float32)
    n_slots = len(segs) + 2
    size = ks.mlstm_state_size(dim, vdim)
    g = torch.Generator().manual_seed(300 + case)
    state = torch.randn((n_slots, heads, size), generator=g).to(DEV)             # leftovers everywhere
    slots = torch.randperm(n_slots, generator=g)[:len(segs)].tolist()
    state[torch.tensor(slots)] = 0.0                                              # what the engine does when a request takes a slot
    untouched = [s for s in range(n_slots) if s not in slots]
    before = state[torch.tensor(untouched)].clone()
    bi = torch.randn(heads, generator=g)
    bf = torch.randn(heads, generator=g) + 1.0
    carried = {s: [(torch.zeros(dim, vdim, dtype=torch.float64), torch.zeros(dim, dtype=torch.float64), 0.0)
                   for _ in range(heads)] for s in range(len(segs))}
    q_scale = dim ** -0.5
    cols = (0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim + 3, 2 * heads * dim + heads * vdim + 3 + heads)
    width = cols[4] + heads + 5
    for step in range(3):
        counts = [sg[step] for sg in segs]
        from spite_b200.engine.batch import Segment, build_step_batch
        seg_list, off = [], 0
        for s, n in enumerate(counts):
            seg_list.append(Segment(s, slots[s], 0, n, off, step == 0))
            off += n
        batch = build_step_batch(seg_list, [[0] * n for n in counts], [[] for _ in counts], [[[0]] * len(counts)], DEV)
        M = off
        proj = torch.randn((M, width), generator=g)
        proj[:, :cols[1]] *= q_size
        proj[:, cols[3]:] *= gate_size
        if step == 0 and counts[0] > 8:
            proj[3, cols[3]:cols[3] + heads] = 40.0           # one token is taken in far more strongly than the rest: it stays in the memory
        out = torch.empty((M, heads * vdim), dtype=torch.float32, device=DEV)
        ks.mlstm_scan(proj.to(DEV), out, batch, state, heads=heads, dim=dim, vdim=vdim, gate_cap=cap, q_scale=q_scale,
                      columns=cols, i_bias=bi.to(DEV), f_bias=bf.to(DEV), chunked=chunked)
        torch.cuda.synchronize()
        assert not ks.errors()
        ref = torch.zeros(M, heads, vdim, dtype=torch.float64)
        off = 0
        pd = proj.double()
        for s, n in enumerate(counts):
            rows = pd[off:off + n]
            for a in range(heads):
                S0, n0, m0 = carried[s][a]
                o, S1, n1, m1 = memory_loops(rows[:, cols[0] + a * dim:cols[0] + (a + 1) * dim], rows[:, cols[1] + a * dim:cols[1] + (a + 1) * dim],
                                             rows[:, cols[2] + a * vdim:cols[2] + (a + 1) * vdim], rows[:, cols[3] + a], rows[:, cols[4] + a],
                                             float(bi[a]), float(bf[a]), cap, q_scale, S0, n0, m0)
                carried[s][a] = (S1, n1, m1)
                ref[off:off + n, a] = o
            off += n
        # 32 tokens at a time the same terms are summed in another order, more of them in one sum
        close(out.view(M, heads, vdim), ref, 5e-5 if chunked else 2e-5, f"memory scan, step {step}")
    for s in range(len(segs)):                                # the state itself, as the slot holds it
        for a in range(heads):
            S1, n1, m1 = carried[s][a]
            got = state[slots[s], a].cpu().double()
            close(got[:dim * vdim].view(dim, vdim), S1, 2e-5, "S")
            stride = -(-(dim + 1) // 4) * 4
            for b in range(-(-vdim // 32)):
                copy = got[dim * vdim + b * stride:]
                close(copy[:dim], n1, 2e-5, "n")
                assert abs(float(copy[dim]) - m1) <= 1e-5 * max(1.0, abs(m1))
    assert torch.equal(state[torch.tensor(untouched)], before)


def test_memory_keeps_a_token_from_hundreds_of_steps_back():
    """Forget gates near one (log f near 0) and one token taken in strongly at position 2: after 700 more tokens, a
    query aligned with that token's key still reads that token's value: in one prompt (token by token, and 32 tokens at
    a time), decoded one by one, and in portions of many sizes."""
    ks = kernels(torch.float32)
    heads, dim, vdim, cap, T = 2, 48, 40, 15.0, 703
    from spite_b200.engine.batch import Segment, build_step_batch
    g = torch.Generator().manual_seed(9)
    cols = (0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim, 2 * heads * dim + heads * vdim + heads)
    proj = torch.randn((T, cols[4] + heads), generator=g)
    proj[:, cols[3]:cols[4]] = -6.0                            # take in little ...
    proj[2, cols[3]:cols[4]] = 6.0                             # ... but this one
    proj[:, cols[4]:] = 14.0                                   # forget next to nothing
    proj[T - 1, :cols[1]] = proj[2, cols[1]:cols[2]] * 3.0     # the last query looks for the key of token 2
    zero = torch.zeros(heads, device=DEV)
    size = ks.mlstm_state_size(dim, vdim)
    outs = []
    for counts, chunked in (([T], False), ([3] + [1] * (T - 3), False), ([T], True), ([31, 33, 64, 1, 2, 200, 9, 300, 63], True)):
        assert sum(counts) == T
        state = torch.zeros((1, heads, size), device=DEV)
        got, at = [], 0
        for i, n in enumerate(counts):
            batch = build_step_batch([Segment(0, 0, at, n, 0, i == 0)], [[0] * n], [[]], [[[0]]], DEV)
            out = torch.empty((n, heads * vdim), dtype=torch.float32, device=DEV)
            ks.mlstm_scan(proj[at:at + n].contiguous().to(DEV), out, batch, state, heads=heads, dim=dim, vdim=vdim, gate_cap=cap,
                          q_scale=dim ** -0.5, columns=cols, i_bias=zero, f_bias=zero, chunked=chunked)
            got.append(out.cpu())
            at += n
        outs.append(torch.cat(got))
    for out in outs:
        last = out[T - 1].view(heads, vdim)
        for a in range(heads):
            v2 = proj[2, cols[2] + a * vdim:cols[2] + (a + 1) * vdim]
            cos = float(torch.nn.functional.cosine_similarity(last[a], v2, dim=0))
            assert cos > 0.95, cos
    close(outs[1], outs[0], 1e-5, "decoded against the prompt")
    # Seven hundred decays near one, each rounded to float32: the walk token by token itself stands a few 1e-4 from the
    # same loops in float64, and the other order of the sums may differ from it by as much.
    ref = torch.zeros(T, heads, vdim, dtype=torch.float64)
    pd = proj.double()
    for a in range(heads):
        ref[:, a] = memory_loops(pd[:, a * dim:(a + 1) * dim], pd[:, cols[1] + a * dim:cols[1] + (a + 1) * dim],
                                 pd[:, cols[2] + a * vdim:cols[2] + (a + 1) * vdim], pd[:, cols[3] + a], pd[:, cols[4] + a], 0.0, 0.0, cap,
                                 dim ** -0.5, torch.zeros(dim, vdim, dtype=torch.float64), torch.zeros(dim, dtype=torch.float64), 0.0)[0]
    for out in outs:
        close(out.view(T, heads, vdim), ref, 1e-3, "against loops in float64")


def test_malformed_scan_calls_launch_nothing():
    """Null pointers and sizes that make no sense return -1, key heads beyond the kernels' 512 rows -2, the chunked walk
    without working memory (or through the entry that has none) -1; the outputs keep their canary."""
    import ctypes as C
    from spite_b200.kernels import build
    from spite_b200.kernels.cuda import MlstmParams
    lib = build.load("recurrent")
    heads, dim, vdim, M = 2, 16, 24, 5
    proj = torch.zeros((M, 2 * heads * dim + heads * vdim + 2 * heads), device=DEV)
    out = torch.full((M, heads * vdim), 96.5, device=DEV)
    state = torch.full((1, heads, CudaSize.state(dim, vdim)), 96.5, device=DEV)
    cu = torch.tensor([0, M], dtype=torch.int32, device=DEV)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    zero = torch.zeros(heads, device=DEV)
    scratch = torch.zeros((2, heads, 1152), device=DEV)

    def params(**change):
        kw = dict(proj=proj.data_ptr(), stride=proj.shape[1], q_col=0, k_col=heads * dim, v_col=2 * heads * dim,
                  i_col=2 * heads * dim + heads * vdim, f_col=2 * heads * dim + heads * vdim + heads, i_bias=zero.data_ptr(),
                  f_bias=zero.data_ptr(), out=out.data_ptr(), state=state.data_ptr(), head_stride=state.shape[2],
                  cu_seqlens=cu.data_ptr(), slots=slots.data_ptr(), n_segments=1, heads=heads, dim=dim, vdim=vdim,
                  gate_cap=10.0, q_scale=0.25, chunked=0)
        kw.update(change)
        return MlstmParams(**kw)

    plain = lambda p: lib.spite_mlstm_scan(C.byref(p), None)
    chunk = lambda p, s=scratch, n=2: lib.spite_mlstm_scan_chunked(C.byref(p), C.c_void_p(None if s is None else s.data_ptr()), C.c_int(n), None)
    cases = [(plain(params(proj=None)), -1), (plain(params(out=None)), -1), (plain(params(state=None)), -1),
             (plain(params(heads=0)), -1), (plain(params(gate_cap=0.0)), -1), (plain(params(stride=3)), -1),
             (plain(params(head_stride=dim * vdim)), -1), (plain(params(dim=513, stride=10 ** 6, head_stride=10 ** 9)), -2),
             (plain(params(chunked=1)), -1), (chunk(params(chunked=1), None), -1), (chunk(params(chunked=1), scratch, 0), -1),
             (chunk(params(chunked=1, slots=None)), -1)]
    torch.cuda.synchronize()
    assert [got for got, _ in cases] == [want for _, want in cases]
    assert bool((out == 96.5).all()) and bool((state == 96.5).all())


class CudaSize:
    @staticmethod
    def state(dim, vdim):
        from spite_b200.kernels.api import KernelSet
        return KernelSet.mlstm_state_size(dim, vdim)


# ---------------------------------------------------------------------------- between the heads and the output projection
@pytest.mark.parametrize("dtype,in32", [(torch.float32, True), (torch.bfloat16, True), (torch.bfloat16, False), (torch.float32, False)])
@pytest.mark.parametrize("heads,size,norm,gain,gate", [(3, 12, True, True, True), (1, 70, True, True, True), (4, 64, False, False, True),
                                                        (5, 33, True, False, False), (2, 256, True, True, True), (8, 16, False, True, True)])
def test_head_norm_gate(dtype, in32, heads, size, norm, gain, gate):
    ks = kernels(dtype)
    M = 37
    g = torch.Generator().manual_seed(heads * 10 + size)
    xt = torch.float32 if in32 else dtype
    x = (torch.randn((M, heads * size), generator=g) * torch.rand((M, 1), generator=g) * 3).to(xt)
    x[1] *= 1e-4                                               # a head that puts out next to nothing: eps matters
    wide = torch.randn((M, 5 + heads * size + 3), generator=g).to(xt)
    gn = (1.0 + 0.3 * torch.randn(heads * size, generator=g)) if gain else None
    eps = 1e-5
    out = torch.empty((M, heads * size), dtype=dtype, device=DEV)
    ks.head_norm_gate(x.to(DEV), out, heads=heads, size=size, gates=wide.to(DEV) if gate else None, gate_column=5,
                      gain=gn.to(DEV) if gain else None, eps=eps if norm else None)
    ref = x.double().view(M, heads, size)
    if norm:
        ref = ref / torch.sqrt((ref * ref).mean(-1, keepdim=True) + eps)
    ref = ref.reshape(M, -1)
    if gain:
        ref = ref * gn.double()
    if gate:
        ref = ref * torch.sigmoid(wide[:, 5:5 + heads * size].double())
    close(out, ref, 1e-5 if dtype == torch.float32 else 6e-3, "heads' norm, gain and gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,M,follow", [(72, 5, True), (256, 33, True), (40, 1, False), (1000, 7, True), (4096, 3, False), (6, 2, True)])
def test_norm_behind_a_sublayer_joins_the_stream(dtype, d, M, follow):
    ks = kernels(dtype)
    g = torch.Generator().manual_seed(d + M)
    y = torch.randn((M, d), generator=g) * 5
    h = torch.randn((M, d), generator=g)
    w = 1.0 + 0.3 * torch.randn(d, generator=g)
    w2 = 1.0 + 0.3 * torch.randn(d, generator=g)
    eps, mult = 1e-3, 0.3
    hd = h.clone().to(DEV)
    nxt = torch.empty((M, d), dtype=dtype, device=DEV) if follow else None
    ks.rms_norm_residual(y.to(DEV), w.to(DEV), eps, mult, hd, next_gain=w2.to(DEV) if follow else None, next_out=nxt)
    yd = y.double()
    ref = h.double() + mult * yd / torch.sqrt((yd * yd).mean(-1, keepdim=True) + eps) * w.double()
    close(hd, ref, 2e-6, "stream")
    if follow:
        close(nxt, ref / torch.sqrt((ref * ref).mean(-1, keepdim=True) + eps) * w2.double(), 1e-5 if dtype == torch.float32 else 6e-3, "next norm")


def test_fill_rows():
    ks = kernels(torch.float32)
    g = torch.Generator().manual_seed(1)
    for M, d in ((3, 72), (17, 1000), (1, 5)):
        out = torch.randn((M, d), generator=g).to(DEV)
        vec = torch.randn(d, generator=g).to(DEV)
        keep = out.clone()
        ks.fill_rows(out, vec, accumulate=True)
        assert torch.equal(out, keep + vec)
        ks.fill_rows(out, vec)
        assert torch.equal(out, vec.expand(M, d))


# ---------------------------------------------------------------------------- the prepare kernel's additions
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,rot,q_only", [(4, 2, 24, 6, False), (4, 2, 24, 6, True), (3, 3, 32, 32, False), (8, 2, 64, 32, True),
                                                   (2, 1, 128, 64, False), (1, 1, 8, 2, False), (6, 3, 40, 10, True)])
def test_prepare_adds_biases_rotates_leading_elements_and_serves_queries_alone(dtype, nq, nkv, hd, rot, q_only):
    """Bias before the rotation; element i of a head pairs with element i + rot / 2 and the elements from `rot` on pass
    unchanged (rot / 2 odd included); with queries alone nothing is appended to the cache."""
    ks = kernels(dtype)
    P, n_pages = 16, 12
    specs = [(0, 19), (30, 1), (15, 3)]
    batch, tables = make_batch(specs, P, n_pages, 20, DEV)
    M = batch.n_tokens
    g = torch.Generator().manual_seed(nq * 100 + hd + rot)
    heads = nq if q_only else nq + 2 * nkv
    extra = 11 + (heads * hd + 11) % 2                          # columns of something else behind the heads; rows stay even
    qkv = torch.randn((M, heads * hd + extra), generator=g).to(dtype)
    bias = torch.randn(heads * hd, generator=g)
    inv_freq = torch.tensor([50.0 ** (-2 * i / rot) for i in range(rot // 2)], dtype=torch.float32)
    kv = torch.full((2, n_pages, nkv, P, hd), 7.0, dtype=dtype, device=DEV)
    q = torch.empty((M, nq * hd), dtype=dtype, device=DEV)
    ks.qk_prepare(qkv.to(DEV), q, batch, LayerCache(0, kv, None, P, not q_only), num_heads=nq,
                  rotation=Rotation(inv_freq.to(DEV), "halves", rot), qk_norm=None, temperature=None, bias=bias.to(DEV), q_only=q_only)
    torch.cuda.synchronize()
    x = (qkv[:, :heads * hd].double() + bias.double()).view(M, heads, hd)
    pos = torch.tensor([s + t for s, n in specs for t in range(n)], dtype=torch.float64)
    ang = pos[:, None] * inv_freq.double()[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    turned = x.clone()
    n_rot = nq if q_only else nq + nkv
    u, v = x[:, :n_rot, :rot // 2], x[:, :n_rot, rot // 2:rot]
    turned[:, :n_rot, :rot // 2] = u * cos - v * sin
    turned[:, :n_rot, rot // 2:rot] = v * cos + u * sin
    tol = 1e-5 if dtype == torch.float32 else 6e-3
    close(q.view(M, nq, hd), turned[:, :nq], tol, "q")
    if q_only:
        assert bool((kv == 7.0).all())
        return
    row = 0
    for s, (start, n) in enumerate(specs):
        for t in range(n):
            p = start + t
            page = tables[s][p // P]
            close(kv[0, page, :, p % P], turned[row, nq:nq + nkv], tol, "cached key")
            close(kv[1, page, :, p % P], turned[row, nq + nkv:], tol, "cached value")
            row += 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 96, 72), (8, 256, 128), (40, 200, 72), (64, 1024, 512), (300, 384, 256), (2048, 1024, 1024)])
def test_gelu_in_the_epilogue_of_every_product_kernel(dtype, M, N, K):
    ks = kernels(dtype)
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn((M, K), generator=g).to(dtype)
    w = (torch.randn((N, K), generator=g) * (3.0 / math.sqrt(K))).to(dtype)
    out = torch.empty((M, N), dtype=dtype, device=DEV)
    ks.linear(x.to(DEV), w.to(DEV), out, activation="gelu_tanh")
    z = x.double() @ w.double().T
    ref = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
    close(out, ref, 1e-5 if dtype == torch.float32 else 6e-3, f"gelu(x W^T), {M} rows")
    assert float((ref - z.clamp(min=0)).abs().max()) > 0.05         # not a relu


# ---------------------------------------------------------------------------- the engine
@pytest.fixture(scope="module", params=list(S.CONFIGS))
def folder(request, tmp_path_factory):
    return S.write_model(tmp_path_factory.mktemp(f"paposun_{request.param}"), request.param), request.param


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request, folder):
    from spite_b200.engine import Model
    path, name = folder
    dtype = request.param
    model = Model.from_folder(path, dtype=dtype, device=DEV)
    vocab = model.plan.vocab_size
    lengths = {"a": 330 if name == "L" else 97, "b": 40, "c": 37, "d": 66, "e": 1, "f": 21}
    requests = {r: H.random_tokens(vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    return path, model, requests, TOL[dtype], dtype


def _engine(model, steps, page_size):
    from spite_b200.engine import Engine
    return Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=page_size, max_requests=4)


def poison_what_is_free(engine):
    """Whatever a free page held last is not finite, and the state slots nobody holds are filled with large numbers:
    a kernel that reads a masked key of a reused page, or a slot that is taken without being cleared, shows."""
    for g, pool in enumerate(engine.cache.pools):
        if pool._free:
            engine.storage.kv[g][:, :, torch.tensor(pool._free, device=DEV)] = float("nan")
    for st in engine.storage.state.values():
        for s, held in enumerate(engine.cache.slots._held):
            if not held:
                st[s] = 1e4


def test_every_cut_gives_the_logits_of_the_whole_sequence(setup):
    path, model, requests, tol, dtype = setup
    n_prompt = {r: max(1, len(t) - 9) for r, t in requests.items()}
    cuts = {"whole": (H.steps_whole(requests), 64), "whole, small pages": (H.steps_whole(requests), 16),
            "last 32 decoded": (H.steps_last_decoded(requests, 32), 64),
            "portions": (H.steps_portions(requests, seed=4), 64),
            "portions of 2 and 3": (H.steps_portions(requests, seed=5, sizes=(2, 3)), 16),
            "mixed": (H.steps_mixed(requests, n_prompt, seed=6), 64),
            "mixed, small pages": (H.steps_mixed(requests, n_prompt, seed=7, sizes=(2, 5, 17, 40)), 16)}
    for what, (steps, page) in cuts.items():
        eng = _engine(model, steps, page)
        S.compare_with_plain(H.run_steps(eng, steps, before_step=poison_what_is_free), path, requests, tol)
        eng.check()
        assert eng.cache.free_pages() == [eng.n_pages] * eng.storage.n_groups, what


def test_the_residual_stream_layer_by_layer(setup):
    path, model, requests, tol, dtype = setup
    cfg, tensors = S.folder_contents(str(path))
    toks = requests["c"]
    layers, rounded = [], []
    plain.forward(cfg, tensors, toks, torch.float64, taps=layers)
    if dtype == "float32":
        plain.forward(cfg, tensors, toks, torch.float32, taps=rounded)
    else:
        g = torch.Generator().manual_seed(1)
        plain.forward(cfg, tensors, toks, torch.float64, taps=rounded,
                      round_inputs=lambda x: x * (1.0 + 2.0 ** -9 * (2.0 * torch.rand(x.shape, generator=g, dtype=x.dtype) - 1.0)))
    seen = []
    model.layer_tap = lambda i, h: seen.append(h.double().cpu())
    try:
        steps = H.steps_whole({"c": toks})
        H.run_steps(_engine(model, steps, 64), steps)
    finally:
        model.layer_tap = None
    assert len(seen) == len(layers)
    for i, h in enumerate(seen):
        scale = float(layers[i].abs().max())
        err = float((h - layers[i]).abs().max()) / scale
        allowed = max(1.5 * tol, 4.0 * float((rounded[i].double() - layers[i]).abs().max()) / scale)       # what rounding alone does, times four
        assert err <= allowed, f"layer {i}: {err:.3e} exceeds {allowed:.1e}"


def test_long_decoding_after_a_short_prompt(setup):
    """Three prompt tokens, then 300 tokens one by one (decode steps replayed from CUDA graphs, pages taken one after the
    other and given back behind every chunk, every chunk of the configuration crossed while decoding, the memories
    carried through 300 steps)."""
    path, model, requests, tol, dtype = setup
    toks = H.random_tokens(model.plan.vocab_size, 303, 77)
    reqs = {"long": toks}
    steps = H.steps_last_decoded(reqs, 300)
    eng = _engine(model, steps, 16)
    S.compare_with_plain(H.run_steps(eng, steps), path, reqs, tol)
    assert eng.graph_replays > 200


def test_greedy_generation_through_the_entry_point(setup):
    """`LLM.generate` (scheduler, sampler, engine): the tokens are the plain implementation's argmax at every step where
    its best two logits are not within rounding of each other."""
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
            row = plain.forward(cfg, tensors, toks, torch.float64)[-1]
            top2 = torch.topk(row, 2).values
            if float(top2[0] - top2[1]) > 2 * tol * float(row.abs().max()):
                assert tok == int(torch.argmax(row)), f"after {len(toks)} tokens"
                compared += 1
            toks.append(tok)                                 # follow the engine's own sequence
    assert compared >= 12


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
        n_rows = sum(len(e["want"]) for e in s["entries"])
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) if n_rows else None
        i = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = torch.from_numpy(rows[i].copy())
                i += 1
            pos[e["id"]] = base + len(e["tokens"])
        assert rows is None or i == rows.shape[0]
    S.compare_with_plain(got, path, requests, 2e-5)


def test_the_command_line_runs_a_paposun_folder(tmp_path):
    """`spite random`, `spite run` (greedy, float32: the plain implementation's tokens) and `spite bench`."""
    import subprocess, sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    spite = lambda *a: subprocess.run([sys.executable, str(root / "bin" / "spite")] + [str(x) for x in a],
                                      capture_output=True, text=True, timeout=900)
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(S.CONFIG_K))
    model = tmp_path / "model"
    assert spite("random", "--config", cfg_file, "--out", model, "--seed", 3, "--std", 0.1).returncode == 0
    cfg, W = plain.load_folder(model)
    prompt = H.random_tokens(S.CONFIG_K["vocab"], 17, 2)
    proc = spite("run", "-m", model, "-p", " ".join(map(str, prompt)), "--max-tokens", 6, "--temperature", 0,
                 "--dtype", "fp32", "--page-size", 16, "--num-pages", 8)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == S.generate_greedy(cfg, W, prompt, 6)
    proc = spite("bench", "-m", model, "--n-prompt", 40, "--n-tokens", 12, "--n-runs", 2, "--json", "--dtype", "bf16")
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads(proc.stdout)
    assert report["decode_tps"] > 0 and report["prefill_tps"] > 0
