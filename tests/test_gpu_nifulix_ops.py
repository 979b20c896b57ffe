"""The kernels behind Nifulix's mechanisms, each alone against the plain function of the same mechanism
(tests/plain/nifulix_plain.py, float64), at sizes of their own, with inputs made so that a fault shows: one
key whose score stands out placed just inside and just outside a window, among the kept first tokens and
right after them, far back among hundreds; shuffled pages; sequences that start in the middle of a page."""
import numpy as np
import pytest
import torch

from kvad_b200.ops import Ops
from tests.plain import nifulix_plain as pl

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KTOL = {"float32": 5e-6, "bfloat16": 1.2e-2}
PAGE = 64


def dev(a, dtype=None):
    t = torch.as_tensor(np.asarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to("cuda")


def rel(got, ref):
    got, ref = np.asarray(got.detach().double().cpu()), np.asarray(ref, dtype=np.float64)
    assert np.isfinite(got).all()
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def stored(a, dtype):
    """The values a tensor of the compute dtype holds, as float64."""
    return torch.as_tensor(np.asarray(a)).to(DT[dtype]).double().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [24, 100, 1000])
def test_rmsnorm_forms(dtype, width):
    rng, ops, eps = np.random.default_rng(width), Ops(DT[dtype]), 1e-3
    x = rng.standard_normal((11, width)) * 3
    w = rng.standard_normal(width) * 0.2
    xs, ws = stored(x, "float32"), stored(w, "float32")
    for offset in (False, True):
        out = torch.full((11, width), float("nan"), device="cuda", dtype=DT[dtype])
        ops.rmsnorm(dev(x, torch.float32), dev(w, torch.float32), eps, out, unit_offset=offset)
        assert rel(out, (pl.norm_offset if offset else pl.norm_plain)(xs, ws, eps)) < KTOL[dtype]
    # no weight, a list of rows, input of the compute dtype that is a view of some columns
    rows = torch.tensor([9, 0, 9, 4], dtype=torch.int32)
    out = torch.full((4, width), float("nan"), device="cuda", dtype=DT[dtype])
    ops.rmsnorm(dev(x, torch.float32), None, eps, out, rows=rows.cuda())
    assert rel(out, pl.rms_unit(xs[rows.numpy()], eps)) < KTOL[dtype]
    wide = dev(np.concatenate([x, x[:, :8]], 1), DT[dtype])
    out = torch.full((11, width), float("nan"), device="cuda", dtype=DT[dtype])
    ops.rmsnorm(wide[:, 8:8 + width] if width > 8 else wide[:, :width], dev(w, DT[dtype]), eps, out)
    src = stored(np.concatenate([x, x[:, :8]], 1), dtype)[:, 8:8 + width]
    assert rel(out, pl.norm_plain(src, stored(w, dtype), eps)) < KTOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_takes_up_a_scaled_sum(dtype):
    rng, ops, eps, mult = np.random.default_rng(3), Ops(DT[dtype]), 1e-5, 0.3
    x, d, w = rng.standard_normal((7, 40)), rng.standard_normal((7, 40)), rng.standard_normal(40) * 0.1
    xs, ds = stored(x, "float32"), stored(d, "float32")
    want = pl.norm_offset(xs + mult * ds, stored(w, "float32"), eps)
    xd, dd = dev(x, torch.float32), dev(d, torch.float32)
    rows = torch.tensor([6, 2], dtype=torch.int32).cuda()
    out = torch.full((2, 40), float("nan"), device="cuda", dtype=DT[dtype])
    ops.rmsnorm(xd, dev(w, torch.float32), eps, out, unit_offset=True, rows=rows, deferred=(dd, mult))
    assert rel(out, want[[6, 2]]) < KTOL[dtype]
    assert torch.equal(xd.cpu(), torch.as_tensor(x).float()) and torch.equal(dd.cpu(), torch.as_tensor(d).float())   # a row list writes nothing back
    out = torch.full((7, 40), float("nan"), device="cuda", dtype=DT[dtype])
    ops.rmsnorm(xd, dev(w, torch.float32), eps, out, unit_offset=True, deferred=(dd, mult))
    assert rel(out, want) < KTOL[dtype]
    assert rel(xd, xs + mult * ds) < 1e-6 and float(dd.abs().max()) == 0.0
    ops.scale_add(xd, dev(d, torch.float32), -mult)
    assert rel(xd, xs) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layout", ["half", "interleaved"])
def test_rotary_in_place_and_as_a_copy(dtype, layout):
    rng, ops = np.random.default_rng(4), Ops(DT[dtype])
    n, H, hd, dims, off, base = 9, 3, 20, 6, 10, 300.0
    x = rng.standard_normal((n, H * hd))
    pos = np.array([0, 1, 2, 63, 64, 65, 1000, 5000, 17])
    xs = stored(x, dtype).reshape(n, H, hd)
    want = xs.copy()
    want[..., off:off + dims] = pl.rotate(xs[..., off:off + dims], pos, base, dims, layout)
    inv = dev(base ** (-2.0 * np.arange(dims // 2) / dims), torch.float32)
    t = dev(x, DT[dtype])
    ops.rotary(t, t, dev(pos, torch.int32), inv, H, dims, interleaved=layout == "interleaved", head_stride_src=hd, offset_src=off)
    # (32-bit angles: position 5000 times a frequency near 1 carries ~3e-4 of absolute error into the sine)
    assert rel(t, want.reshape(n, -1)) < max(KTOL[dtype], 1e-3)
    src, dst = dev(x, DT[dtype]), torch.zeros((n, H * (dims + 2)), device="cuda", dtype=DT[dtype])
    ops.rotary(src, dst, dev(pos, torch.int32), inv, H, dims, interleaved=layout == "interleaved", head_stride_src=hd, offset_src=off,
               head_stride_dst=dims + 2, offset_dst=2)
    got = dst.double().cpu().numpy().reshape(n, H, dims + 2)
    assert np.abs(got[..., 2:] - want[..., off:off + dims]).max() < max(KTOL[dtype], 1e-3) * np.abs(want).max()
    assert np.abs(got[..., :2]).max() == 0 and torch.equal(src.cpu(), torch.as_tensor(x).to(DT[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_mul(dtype):
    rng, ops = np.random.default_rng(5), Ops(DT[dtype])
    both = rng.standard_normal((6, 2 * 37)) * 2
    t = dev(both, DT[dtype])
    bs = stored(both, dtype)
    for act, f in (("silu", pl.silu), ("sigmoid", pl.sigmoid)):
        out = torch.full((6, 37), float("nan"), device="cuda", dtype=DT[dtype])
        ops.gate_mul(t[:, :37], t[:, 37:], out, act)
        assert rel(out, f(bs[:, :37]) * bs[:, 37:]) < KTOL[dtype]


# ----------------------------------------------------------------------------- retention
def plain_retention(q, k, v, decay, rot, k_scale, eps, gate, S0=None, pos0=0):
    """[n, H, d] inputs; returns (out [n, H, dv], final state [H, dk, dv])."""
    n, H, dk = q.shape
    dv = v.shape[2]
    pos = np.arange(pos0, pos0 + n)
    if rot:
        q, k = pl.rotate(q, pos, rot[1], rot[0], rot[2]), pl.rotate(k, pos, rot[1], rot[0], rot[2])
    k = k * k_scale
    S = np.zeros((H, dk, dv)) if S0 is None else S0.copy()
    out = np.zeros((n, H, dv))
    for i in range(n):
        for h in range(H):
            S[h] = decay[h] * S[h] + np.outer(k[i, h], v[i, h])
            out[i, h] = S[h].T @ q[i, h]
    if eps is not None:
        out = pl.rms_unit(out, eps)
    if gate is not None:
        out = out * pl.silu(gate)
    return out, S


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv,rot", [(3, 16, 24, (8, 500.0, "half")), (2, 40, 12, (40, 1e4, "interleaved")),
                                         (1, 64, 64, None), (2, 128, 96, (64, 1e6, "half")), (5, 4, 4, (4, 10.0, "half")),
                                         (1, 256, 40, (128, 1e4, "half")), (2, 20, 7, (10, 30.0, "interleaved"))])
def test_retention_whole_in_portions_and_token_by_token(dtype, H, dk, dv, rot):
    rng, ops = np.random.default_rng(dk * dv), Ops(DT[dtype])
    lens = [37, 5, 70]                                     # three sequences in one launch
    decay = np.linspace(0.8, 0.99, H)
    eps, ks = 1e-5, dk ** -0.5
    data = [[rng.standard_normal((n, H * d)) for d in (dk, dk, dv, dv)] for n in lens]
    want, want_S = [], []
    for n, (q, k, v, g) in zip(lens, data):
        o, S = plain_retention(*(stored(a, dtype).reshape(n, H, -1) for a in (q, k, v)), decay, rot, ks, eps,
                               stored(g, dtype).reshape(n, H, dv))
        want.append(o.reshape(n, -1))
        want_S.append(S)
    inv = dev(rot[1] ** (-2.0 * np.arange(rot[0] // 2) / rot[0]), torch.float32) if rot else None
    kw = dict(inv_freq=inv, rot_dims=rot[0] if rot else 0, interleaved=bool(rot and rot[2] == "interleaved"), k_scale=ks, unit_norm_eps=eps)
    dec = dev(decay, torch.float32)
    slots = [4, 0, 2]

    def run(state, cuts):
        """`cuts`: per sequence, how its rows are cut into steps; step j runs the j-th portion of every sequence that has one."""
        got = [np.zeros((n, H * dv)) for n in lens]
        done = [0] * 3
        for j in range(max(len(c) for c in cuts)):
            live = [s for s in range(3) if j < len(cuts[s])]
            rows = [cuts[s][j] for s in live]
            cat = [np.concatenate([data[s][i][done[s]:done[s] + r] for s, r in zip(live, rows)]) for i in range(4)]
            q, k, v, g = (dev(a, DT[dtype]) for a in cat)
            starts = dev(np.concatenate([[0], np.cumsum(rows)]), torch.int32)
            lens_after = dev([done[s] + r for s, r in zip(live, rows)], torch.int32)
            out = torch.full((sum(rows), H * dv), float("nan"), device="cuda", dtype=DT[dtype])
            raw = torch.full((sum(rows), H * dv), float("nan"), device="cuda") if ops.retention_needs_raw(dk, dv) else None
            ops.retention(q, k, v, out, state, starts, lens_after, dev([slots[s] for s in live], torch.int32), len(live), dec, H, gate=g, raw=raw, **kw)
            o = out.double().cpu().numpy()
            at = 0
            for s, r in zip(live, rows):
                got[s][done[s]:done[s] + r] = o[at:at + r]
                at += r
                done[s] += r
        return got

    def check(cuts, tol_scale=1.0):
        state = torch.zeros((6, H, dk, dv), device="cuda")
        got = run(state, cuts)
        for s in range(3):
            assert rel(torch.as_tensor(got[s]), want[s]) < KTOL[dtype] * 4 * tol_scale, (cuts, s)
            assert rel(state[slots[s]], want_S[s]) < 2e-5, (cuts, s)
        assert float(state[[1, 3, 5]].abs().max()) == 0.0                      # other slots untouched
        return got

    whole = check([[n] for n in lens])
    pieces = check([[16, 16, 5], [2, 3], [1, 2, 17, 33, 17]])
    single = check([[20] + [1] * 17, [1] * 5, [64] + [1] * 6])
    if dtype == "float32":                                                      # the same walk however it is cut: the same bits
        for s in range(3):
            assert np.array_equal(whole[s], pieces[s]) and np.array_equal(whole[s], single[s])


def test_retention_far_token_survives_hundreds_of_steps():
    """One early token writes a large value; with decay 0.999 it must still be read 600 tokens later, and with
    decay 0.9 it must be gone: the state really is carried, and really decays per head."""
    ops, H, d, n = Ops(torch.float32), 2, 8, 640
    q, k, v = np.zeros((n, H, d)), np.zeros((n, H, d)), np.zeros((n, H, d))
    k[3, :, 0], v[3, :, 1], q[-1, :, 0] = 50.0, 1.0, 1.0
    rng = np.random.default_rng(1)
    k[4:, :, 2:] = rng.standard_normal((n - 4, H, d - 2)) * 0.1
    v[4:] = rng.standard_normal((n - 4, H, d)) * 0.1
    decay = np.array([0.999, 0.9])
    want, _ = plain_retention(q, k, v, decay, None, 1.0, None, None)
    out = torch.zeros((n, H * d), device="cuda")
    state = torch.zeros((1, H, d, d), device="cuda")
    args = [dev(a.reshape(n, -1), torch.float32) for a in (q, k, v)]
    ops.retention(*args, out, state, dev([0, n], torch.int32), dev([n], torch.int32), dev([0], torch.int32), 1, dev(decay, torch.float32), H)
    got = out.cpu().numpy().reshape(n, H, d)
    assert abs(got[-1, 0, 1] - 50 * 0.999 ** (n - 4)) < 1e-3 and got[-1, 0, 1] > 20
    assert abs(got[-1, 1, 1]) < 1e-20
    assert rel(out, want.reshape(n, -1)) < 1e-5


# ----------------------------------------------------------------------------- attention with shaped scores
def plain_scored(q, k, v, H, scale, cap, span, window, keep_first, gate=None):
    """q [n, H, dk], k [n, G, dk], v [n, G, dv] of ONE whole sequence."""
    n, G = q.shape[0], k.shape[1]
    ok = pl.visible(n, window, keep_first)
    dist = (np.arange(n)[:, None] - np.arange(n)[None, :]).astype(np.float64)
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        s = q[:, h] @ k[:, h // (H // G)].T * scale
        if cap:
            s = cap * np.tanh(s / cap)
        if span:
            s = s - 2.0 ** (-span * (h + 1) / H) * dist
        out[:, h] = pl.softmax_rows(np.where(ok, s, -np.inf)) @ v[:, h // (H // G)]
    return out if gate is None else out * pl.sigmoid(gate)


class Paged:
    """Keys and values of a few sequences in shuffled pages, as the cache lays them out."""

    def __init__(self, lens, G, dk, dv, dtype, seed, alias=False):
        rng = np.random.default_rng(seed)
        self.lens, self.G, self.dk, self.dv, self.dtype = lens, G, dk, dv, dtype
        n_pages = sum(-(-n // PAGE) for n in lens) + 3
        order = rng.permutation(n_pages)
        self.width = max(-(-n // PAGE) for n in lens) + 1
        self.table = np.full((len(lens), self.width), -1, np.int32)
        at = 0
        for s, n in enumerate(lens):
            for j in range(-(-n // PAGE)):
                self.table[s, j] = order[at]
                at += 1
        self.k_pages = torch.full((n_pages, G, PAGE, dk), float("nan"), device="cuda", dtype=DT[dtype])
        self.v_pages = None if alias else torch.full((n_pages, G, PAGE, dv), float("nan"), device="cuda", dtype=DT[dtype])
        self.table_dev = dev(self.table)

    def rows_meta(self, spans):
        """spans: per sequence (first row, rows): row -> sequence / position arrays for those rows."""
        seq = np.concatenate([[s] * r for s, (_, r) in enumerate(spans)])
        pos = np.concatenate([np.arange(a, a + r) for a, r in spans])
        return dev(seq, torch.int32), dev(pos, torch.int32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,window,keep,cap,span", [
    (4, 2, 16, 24, 20, 3, 5.0, 8.0), (3, 3, 32, 16, None, 0, None, 8.0), (6, 1, 20, 40, 70, 0, 30.0, 0.0),
    (8, 2, 64, 64, 64, 4, 30.0, 8.0), (2, 1, 6, 130, 129, 66, None, 2.0),
    (4, 2, 160, 160, 100, 3, 10.0, 8.0)])      # (long keys and values: prompts take blocks of eight warps)
def test_scored_attention_prompts_portions_and_single_rows(dtype, H, G, dk, dv, window, keep, cap, span):
    rng, ops, scale = np.random.default_rng(H * dk + dv), Ops(DT[dtype]), 0.3
    lens = [150, 9, 70]
    cache = Paged(lens, G, dk, dv, dtype, seed=dk)
    data = [[rng.standard_normal((n, w)) for w in (H * dk, G * dk, G * dv, H * dv)] for n in lens]
    want = [plain_scored(stored(q, dtype).reshape(n, H, dk), stored(k, dtype).reshape(n, G, dk), stored(v, dtype).reshape(n, G, dv), H, scale,
                         cap, span, window, keep, stored(g, dtype).reshape(n, H, dv)).reshape(n, -1) for n, (q, k, v, g) in zip(lens, data)]

    def step(spans, hp):
        """Runs rows [a, a + r) of every sequence as one step: store, then attend."""
        cat = [dev(np.concatenate([data[s][i][a:a + r] for s, (a, r) in enumerate(spans) if r]), DT[dtype]) for i in range(4)]
        live = [s for s, (_, r) in enumerate(spans) if r]
        seq = np.concatenate([[j] * spans[s][1] for j, s in enumerate(live)])
        pos = np.concatenate([np.arange(spans[s][0], sum(spans[s])) for s in live])
        table = dev(cache.table[live])
        ops.kv_store_blend(cat[1], cat[2], dev(seq, torch.int32), dev(pos, torch.int32), table, cache.k_pages, cache.v_pages)
        out = torch.full((len(seq), H * dv), float("nan"), device="cuda", dtype=DT[dtype])
        starts = dev(np.concatenate([[0], np.cumsum([spans[s][1] for s in live])]), torch.int32)
        ops.attention_scored(cat[0], out, starts, dev([sum(spans[s]) for s in live], torch.int32), len(live), max(r for _, r in spans), table,
                             cache.k_pages, cache.v_pages, H, scale, softcap=cap or 0.0, slope_span=span, window=window or 0, keep_first=keep,
                             gate=cat[3], heads_per_block=hp)
        o, at, res = out.double().cpu().numpy(), 0, {}
        for s in live:
            res[s] = o[at:at + spans[s][1]]
            at += spans[s][1]
        return res

    group = H // G
    got = step([(0, n) for n in lens], hp=max(d for d in (1, 2, 4) if group % d == 0))
    for s in range(3):
        assert rel(torch.as_tensor(got[s]), want[s]) < KTOL[dtype], ("whole", s)
    # the same through portions (2 rows, an odd count, across a page edge), then single rows with a whole group a block
    cache.k_pages.fill_(float("nan"))
    cuts = [[(0, 2), (2, 61), (63, 2), (65, 60)], [(0, 3), (3, 2), (5, 2), (7, 1)], [(0, 64), (64, 1), (65, 2), (67, 2)]]
    for j in range(4):
        got = step([c[j] for c in cuts], hp=1 if j % 2 else max(d for d in (1, 2, 4) if group % d == 0))
        for s in range(3):
            a, r = cuts[s][j]
            assert rel(torch.as_tensor(got[s]), want[s][a:a + r]) < KTOL[dtype] * max(1.0, np.abs(want[s]).max() / np.abs(want[s][a:a + r]).max()), ("portion", j, s)
    for p in range(125, 150):
        got = step([(p, 1), (0, 0), (0, 0)], hp=min(group, 32))
        assert rel(torch.as_tensor(got[0]), want[0][p:p + 1]) < KTOL[dtype] * max(1.0, np.abs(want[0]).max() / np.abs(want[0][p]).max()), ("single", p)


@pytest.mark.parametrize("mode", ["prompt", "single"])
def test_scored_attention_one_key_that_stands_out(mode):
    """All keys are alike but one, whose score is far above the rest and whose value is a marker; the query
    must read the marker exactly when the design says it sees that key: just inside the window but not just
    outside, among the kept first tokens but not right after them, and far back without a window."""
    ops, H, dk, dv, n = Ops(torch.float32), 2, 8, 4, 400
    window, keep = 96, 4

    def run(marked, window, keep, query=n - 1):
        cache = Paged([n], 1, dk, dv, "float32", seed=marked)
        q, k, v = np.zeros((n, H * dk)), np.zeros((n, dk)), np.zeros((n, dv))
        k[:, 1], q[:, 0], q[:, dk] = 0.1, 30.0, 30.0
        k[marked, 0], v[marked, 2] = 1.0, 1.0
        seq, pos = cache.rows_meta([(0, n)])
        ops.kv_store_blend(dev(k, torch.float32), dev(v, torch.float32), seq, pos, cache.table_dev, cache.k_pages, cache.v_pages)
        if mode == "prompt":
            out = torch.zeros((n, H * dv), device="cuda")
            ops.attention_scored(dev(q, torch.float32), out, dev([0, n], torch.int32), dev([n], torch.int32), 1, n, cache.table_dev, cache.k_pages,
                                 cache.v_pages, H, 1.0, window=window, keep_first=keep, heads_per_block=2)
            return float(out[query, 2])
        out = torch.zeros((1, H * dv), device="cuda")
        ops.attention_scored(dev(q[query:query + 1], torch.float32), out, dev([0, 1], torch.int32), dev([query + 1], torch.int32), 1, 1, cache.table_dev,
                             cache.k_pages, cache.v_pages, H, 1.0, window=window, keep_first=keep, heads_per_block=2)
        return float(out[0, 2])

    last = n - 1
    assert run(last - window + 1, window, keep) > 0.99          # the oldest position of the window
    assert run(last - window, window, keep) == 0.0              # one further back
    assert run(keep - 1, window, keep) > 0.99                   # the last kept first token
    assert run(keep, window, keep) == 0.0                       # the first that is not kept
    assert run(0, window, keep) > 0.99
    assert run(0, window, 0) == 0.0                             # nothing kept: the first token is gone too
    assert run(7, 0, 0) > 0.99                                  # no window: a key 390 back among hundreds
    assert run(64, window, 70, query=300) > 0.99 and run(70, window, 70, query=300) == 0.0     # kept tokens beyond the first page
    assert run(last, window, keep) > 0.99                       # itself


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_values_blended_where_they_are_stored(dtype):
    rng, ops = np.random.default_rng(8), Ops(DT[dtype])
    G, dk, dv, n = 2, 8, 12, 70
    cache = Paged([n], G, dk, dv, dtype, seed=1)
    k, v, other = (rng.standard_normal((n, G * d)) for d in (dk, dv, dv))
    seq, pos = cache.rows_meta([(0, n)])
    lam = 0.37
    ops.kv_store_blend(dev(k, DT[dtype]), dev(v, DT[dtype]), seq, pos, cache.table_dev, cache.k_pages, cache.v_pages,
                       v_other=dev(other, DT[dtype]), blend=dev([lam], DT[dtype]))
    lam_s = float(stored([lam], dtype)[0])
    want = (1 - lam_s) * stored(v, dtype) + lam_s * stored(other, dtype)
    for p in (0, 63, 64, 69):
        page = cache.table[0, p // PAGE]
        got_v = cache.v_pages[page, :, p % PAGE].reshape(-1)
        got_k = cache.k_pages[page, :, p % PAGE].reshape(-1)
        assert rel(got_v, want[p]) < KTOL[dtype]
        assert torch.equal(got_k.cpu(), torch.as_tensor(k[p]).to(DT[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(3, 8, 4, 12, 20, 100, 37), (4, 32, 32, 16, 256, 150, 70)])      # (the second: blocks of eight warps, 16-byte loads)
def test_latent_rows_normalised_turned_and_read_as_keys_and_values(dtype, sizes):
    """The latent cache: a row is [norm(c) | rotate(k_r)]; queries carried into the latent's space attend over it with
    the latent as the value.  Against the plain form that rebuilds every head's keys and values from the latent."""
    rng, ops = np.random.default_rng(9), Ops(DT[dtype])
    H, dn, dr, dv, rk, n, window = sizes
    eps, base, scale = 1e-5, 50.0, 0.3 * (8.0 / dn) ** 0.5
    raw = rng.standard_normal((n, rk + dr))
    w = 1 + 0.1 * rng.standard_normal(rk)
    uk, uv = rng.standard_normal((H * dn, rk)) * 0.3 * (20.0 / rk) ** 0.5, rng.standard_normal((H * dv, rk)) * 0.3 * (20.0 / rk) ** 0.5
    q = rng.standard_normal((n, H, dn + dr))
    cache = Paged([n], 1, rk + dr, rk, dtype, seed=2, alias=True)
    seq, pos = cache.rows_meta([(0, n)])
    inv = dev(base ** (-2.0 * np.arange(dr // 2) / dr), torch.float32)
    ops.latent_store(dev(raw, DT[dtype]), dev(w, torch.float32), eps, inv, seq, pos, cache.table_dev, cache.k_pages, rk, dr, interleaved=True)
    rs = stored(raw, dtype)
    c = pl.norm_plain(rs[:, :rk], stored(w, "float32"), eps)
    k_r = pl.rotate(rs[:, None, rk:], np.arange(n), base, dr, "interleaved")[:, 0]
    page = cache.table[0, 1]
    assert rel(cache.k_pages[page, 0, 5], np.concatenate([c[69], k_r[69]])) < KTOL[dtype]
    heads_a_block = 1 if H == 3 else 4
    # plain: per head keys and values from the latent
    qs = stored(q, dtype)
    q_r = pl.rotate(qs[..., dn:], np.arange(n), base, dr, "interleaved")
    ok = pl.visible(n, window)
    want = np.zeros((n, H, dv))
    for h in range(H):
        s = (qs[:, h, :dn] @ (c @ uk[h * dn:(h + 1) * dn].T).T + q_r[:, h] @ k_r.T) * scale
        want[:, h] = pl.softmax_rows(np.where(ok, s, -np.inf)) @ (c @ uv[h * dv:(h + 1) * dv].T)
    # the product path's form: the query carried into the latent's space (float64 here), one shared key, the latent as value
    ql = np.concatenate([np.einsum("nhd,hdr->nhr", qs[..., :dn], uk.reshape(H, dn, rk)), q_r], -1).reshape(n, -1)
    out = torch.full((n, H * rk), float("nan"), device="cuda", dtype=DT[dtype])
    ops.attention_scored(dev(ql, DT[dtype]), out, dev([0, n], torch.int32), dev([n], torch.int32), 1, n, cache.table_dev, cache.k_pages, None,
                         H, scale, value_dim=rk, window=window, heads_per_block=heads_a_block)
    got = np.einsum("nhr,hvr->nhv", out.double().cpu().numpy().reshape(n, H, rk), uv.reshape(H, dv, rk))
    assert rel(torch.as_tensor(got), want) < KTOL[dtype] * 3
