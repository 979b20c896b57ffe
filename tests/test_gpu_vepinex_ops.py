"""The kernels behind Vepinex's mechanisms, each alone against the plain function of the same mechanism
(tests/plain/vepinex_plain.py, float64), at sizes of their own (heads that share query/key heads, value columns
that do not fill a block, key sizes in every register class), over several sequences packed into one step with
shuffled slots, in portions down to one row, and with inputs made so that a fault shows: a first key that nothing
later overwrites and that the last query asks for, gates far beyond their cap, a first input gate that sets the
running maximum for hundreds of rows, router logits that tie."""
import numpy as np
import pytest
import torch

from kvad_b200.ops import Ops
from tests.plain import vepinex_plain as pl

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to("cuda")


def i32(a):
    return dev(np.asarray(a, dtype=np.int32))


def rel(got, ref):
    got, ref = np.asarray(got.detach().double().cpu()), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.isfinite(got).all()
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def stored(a, dtype):
    """The values a tensor of the given dtype holds, as float64."""
    return torch.as_tensor(np.asarray(a)).to(DT[dtype]).double().numpy()


def packed(lengths):
    starts = np.concatenate([[0], np.cumsum(lengths)])
    return starts, int(starts[-1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv", [(3, 20, 24), (1, 72, 16), (2, 8, 40), (2, 200, 5), (1, 320, 20)])
def test_matrix_memory_in_portions_with_gates_beyond_the_cap(dtype, H, dk, dv):
    rng, ops, cap = np.random.default_rng(dk), Ops(DT[dtype]), 6.0
    total_lens, slots = [150, 9, 1], [4, 0, 2]
    T = max(total_lens)
    q, k, v = (stored(rng.standard_normal((3, T, H * d)), dtype) for d in (dk, dk, dv))
    gates = stored(rng.standard_normal((3, T, 2 * H)) * 5.0, "float32")
    gates[0, 0, :H] = 40.0            # a first input gate at the cap: it sets the running maximum for all that follows
    gates[0, :, H:] += 8.0            # ... and this sequence forgets slowly, so its first key stays in reach
    scale = dk ** -0.5
    want = []
    for s, n in enumerate(total_lens):
        gi, gf = pl.gate_caps(gates[s, :n, :H], gates[s, :n, H:], cap)
        want.append(np.concatenate([pl.matrix_memory_cell(q[s, :n, a * dk:(a + 1) * dk] * scale, k[s, :n, a * dk:(a + 1) * dk],
                                                          v[s, :n, a * dv:(a + 1) * dv], gi[:, a], gf[:, a])[0] for a in range(H)], axis=1))
    state = torch.zeros((6, ops.recurrence_state_size("matrix_memory", H, dk, dv) + 3), device="cuda")
    done = [0, 0, 0]
    for portion in ([100, 9, 1], [1, 0, 0], [2, 0, 0], [47, 0, 0]):
        live = [s for s in range(3) if portion[s]]
        starts, n = packed([portion[s] for s in live])
        cut = lambda a: np.concatenate([a[s, done[s]:done[s] + portion[s]] for s in live])
        out = torch.full((n, H * dv), float("nan"), device="cuda")
        ops.gated_recurrence("matrix_memory", dev(cut(q), DT[dtype]), dev(cut(k), DT[dtype]), dev(cut(v), DT[dtype]), dev(cut(gates), torch.float32),
                             out, state, i32(starts), i32([slots[s] for s in live]), len(live), H, H, dk, dv, q_scale=scale, cap=cap)
        ref = np.concatenate([want[s][done[s]:done[s] + portion[s]] for s in live])
        # (the read-out is a quotient whose two sums can nearly cancel: rounding of 32-bit sums over 150 rows shows as 1e-4)
        assert rel(out, ref) < 5e-4, portion
        for s in live:
            done[s] += portion[s]
    assert float(state[[1, 3, 5]].abs().max()) == 0.0          # slots of no sequence are untouched


@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 16, 10), (2, 1, 136, 16), (3, 3, 6, 33), (6, 1, 40, 8), (2, 2, 500, 18)])
def test_delta_rule_keeps_a_first_key_that_nothing_overwrites(H, G, dk, dv):
    rng, ops = np.random.default_rng(dk + dv), Ops(torch.float32)
    lens, slots = [300, 4], [1, 5]
    T = max(lens)
    q = pl.unit_vectors(rng.standard_normal((2, T, G, dk)))
    k = rng.standard_normal((2, T, G, dk))
    k[0, 1:, :, 0] = 0.0
    k[0, 0] = 0.0
    k[0, 0, :, 0] = 1.0               # the first key is the first unit vector; no later key has a part along it
    k = pl.unit_vectors(k)
    q[0, -1] = k[0, 0]                # ... and the last query asks for exactly it
    v = rng.standard_normal((2, T, H, dv))
    a = rng.standard_normal((2, T, H, dk))
    a_log, dt_bias = rng.standard_normal(H) - 1.0, rng.standard_normal((H, dk)) - 1.0
    a[0, :, :, 0] = -60.0             # channel 0 of the first sequence does not decay: softplus(-60) is nothing
    beta = pl.sigmoid(rng.standard_normal((2, T, H)))
    f32 = lambda x: stored(x, "float32")
    q, k, v, a, a_log, dt_bias, beta = map(f32, (q, k, v, a, a_log, dt_bias, beta))
    g = [pl.channel_decay(a[s], a_log, dt_bias) for s in range(2)]
    want = [np.concatenate([pl.delta_cell(q[s, :n, h // (H // G)], k[s, :n, h // (H // G)], v[s, :n, h], beta[s, :n, h], g[s][:n, h])[0]
                            for h in range(H)], axis=1) for s, n in enumerate(lens)]
    assert np.allclose(want[0][-1].reshape(H, dv), beta[0, 0][:, None] * v[0, 0], atol=1e-9)      # what the first row wrote, 299 rows later
    state = torch.zeros((7, ops.recurrence_state_size("delta_rule", H, dk, dv)), device="cuda")
    done = [0, 0]
    for portion in ([130, 4], [1, 0], [169, 0]):
        live = [s for s in range(2) if portion[s]]
        starts, n = packed([portion[s] for s in live])
        cut = lambda x: dev(np.concatenate([x[s, done[s]:done[s] + portion[s]].reshape(portion[s], -1) for s in live]), torch.float32)
        out = torch.full((n, H * dv), float("nan"), device="cuda")
        ops.gated_recurrence("delta_rule", cut(q), cut(k), cut(v), cut(a), out, state, i32(starts), i32([slots[s] for s in live]), len(live),
                             H, G, dk, dv, beta=cut(beta), a_log=dev(a_log, torch.float32), dt_bias=dev(dt_bias.reshape(-1), torch.float32))
        assert rel(out, np.concatenate([want[s][done[s]:done[s] + portion[s]] for s in live])) < 2e-5, portion
        for s in live:
            done[s] += portion[s]
    # the decays worked out in a pass of their own (as for prompts): the same read-outs
    state2, ready = torch.zeros_like(state), dev(np.concatenate([a[0].reshape(T, -1), a[1, :4].reshape(4, -1)]), torch.float32)
    ops.decay_gate(ready, dev(a_log, torch.float32), dev(dt_bias.reshape(-1), torch.float32), H, dk)
    assert rel(ready, np.concatenate([g[0].reshape(T, -1), g[1][:4].reshape(4, -1)])) < 1e-6
    both = lambda x: dev(np.concatenate([x[0].reshape(T, -1), x[1, :4].reshape(4, -1)]), torch.float32)
    out = torch.full((T + 4, H * dv), float("nan"), device="cuda")
    ops.gated_recurrence("delta_rule", both(q), both(k), both(v), ready, out, state2, i32([0, T, T + 4]), i32(slots), 2, H, G, dk, dv, beta=both(beta),
                         a_log=dev(a_log, torch.float32), dt_bias=dev(dt_bias.reshape(-1), torch.float32), gates_ready=True)
    assert rel(out, np.concatenate([want[0], want[1]])) < 2e-5 and rel(state2, state.cpu().numpy()) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_short_convolution_over_portions_shorter_than_its_taps(dtype, taps):
    rng, ops = np.random.default_rng(taps), Ops(DT[dtype])
    G, dk, extra, n_sig = 3, 10, 7, 2
    C = 2 * G * dk + extra
    lens, slots = [40, 6], [2, 0]
    x = stored(rng.standard_normal((2, 40, C + n_sig + 3)), dtype)
    w = stored(rng.standard_normal((C, taps)) * 0.7, dtype)
    want = []
    for s, n in enumerate(lens):
        y = pl.silu(pl.short_conv(x[s, :n, :C], w))
        heads = pl.unit_vectors(y[:, :2 * G * dk].reshape(n, 2 * G, dk), 1e-6)
        heads[:, :G] *= 0.25
        want.append(np.concatenate([heads.reshape(n, -1), y[:, 2 * G * dk:], pl.sigmoid(x[s, :n, C:C + n_sig])], axis=1))
    off = 11
    state = torch.zeros((3, off + max(taps - 1, 1) * C), device="cuda")
    done = [0, 0]
    for portion in ([1, 6], [1, 0], [2, 0], [1, 0], [3, 0], [32, 0]):
        live = [s for s in range(2) if portion[s]]
        starts, n = packed([portion[s] for s in live])
        rows = dev(np.concatenate([x[s, done[s]:done[s] + portion[s]] for s in live]), DT[dtype])
        row_seq = np.concatenate([[j] * portion[s] for j, s in enumerate(live)])
        row_pos = np.concatenate([np.arange(done[s], done[s] + portion[s]) for s in live])
        y = torch.full((n, C + n_sig), float("nan"), device="cuda")
        sl = i32([slots[s] for s in live])
        ops.short_conv(rows, dev(w, DT[dtype]), y, state, off, i32(row_seq), i32(row_pos), i32(starts), sl, n_sigmoid=n_sig, unit_heads=2 * G,
                       unit_dim=dk, scaled_heads=G, head_scale=0.25, unit_eps=1e-6)
        ops.conv_state(rows, C, taps, state, off, i32(starts), sl, len(live))
        assert rel(y, np.concatenate([want[s][done[s]:done[s] + portion[s]] for s in live])) < 1e-5, portion
        for s in live:
            done[s] += portion[s]
    if taps > 1:                      # what is kept: the last taps - 1 inputs
        kept = state[slots[0], off:off + (taps - 1) * C].view(taps - 1, C)
        assert rel(kept, x[0, 40 - (taps - 1):40, :C]) == 0.0
    assert float(state[:, :off].abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("per_head", [True, False])
def test_head_norm_with_weight_and_gate(dtype, per_head):
    rng, ops, H, dv, eps = np.random.default_rng(5), Ops(DT[dtype]), 5, 18, 1e-3
    raw = stored(rng.standard_normal((9, H * dv)) * np.exp(rng.standard_normal((9, 1)) * 3), "float32")
    gate = stored(rng.standard_normal((9, H * dv)) * 2, dtype)
    w = stored(rng.standard_normal(H * dv if per_head else dv), dtype)
    want = pl.rms_unit(raw.reshape(9, H, dv), eps) * (w.reshape(H, dv) if per_head else w)[None] * pl.sigmoid(gate).reshape(9, H, dv)
    out = torch.full((9, H * dv), float("nan"), device="cuda", dtype=DT[dtype])
    ops.head_norm_gate(dev(raw, torch.float32), dev(gate, DT[dtype]), dev(w, DT[dtype]), out, H, eps, weight_per_head=per_head)
    assert rel(out, want.reshape(9, -1)) < (1e-5 if dtype == "float32" else 6e-3)


@pytest.mark.parametrize("E,top", [(5, 2), (7, 1), (4, 4), (130, 6)])
def test_router_choice_with_ties_and_weights_over_the_chosen_only(E, top):
    rng, ops = np.random.default_rng(E), Ops(torch.float32)
    z = stored(rng.standard_normal((33, E)) * 3, "float32")
    z[0] = 1.25                       # all level: the first `top` experts
    z[1, -1] = z[1, 0] = 50.0         # two level at the top: the lower index first
    chosen, weight = torch.full((33, top), -7, device="cuda", dtype=torch.int32), torch.full((33, top), float("nan"), device="cuda")
    padded = dev(np.concatenate([z, np.full((33, 3), 1e9)], 1), torch.float32)[:, :E]      # (a view: what lies beside the logits is not one)
    ops.moe_route(padded, top, chosen, weight)
    ref_c, ref_w = pl.choose(z, top)
    assert np.array_equal(chosen.cpu().numpy(), ref_c)
    assert rel(weight, ref_w) < 1e-6
    # the same inside the launch that groups the rows
    chosen.fill_(-7), weight.fill_(float("nan"))
    tiles = ops.moe_max_tiles(33, top, E, 32)
    lists = [torch.empty(n, device="cuda", dtype=torch.int32) for n in (tiles, tiles * 32, tiles * 32, 33 * top)]
    ops.moe_sort(chosen, E, 32, *lists, logits=padded, weight=weight)
    assert np.array_equal(chosen.cpu().numpy(), ref_c) and rel(weight, ref_w) < 1e-6
    assert sorted(lists[3].cpu().tolist()) == sorted(np.nonzero(lists[2].cpu().numpy() >= 0)[0].tolist())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,E,top,width,ff", [(70, 5, 2, 24, 20), (3, 6, 3, 40, 33), (200, 3, 1, 18, 70), (33, 40, 4, 64, 16), (300, 6, 2, 72, 200),
                                              (700, 3, 1, 136, 24), (3, 6, 3, 40, 32), (40, 2, 2, 264, 16), (1, 4, 2, 520, 24)])
def test_routed_experts_against_each_row_by_itself(dtype, n, E, top, width, ff):
    """Small steps run tiles of 32 positions on the CUDA cores; from 512 (row, choice) pairs on, bfloat16 with sizes in
    16-byte pieces runs tiles of 128 on the tensor cores from a gathered copy of the rows."""
    from kvad_b200.ops import tcgen05_wait_timeouts
    rng, ops, limit = np.random.default_rng(n), Ops(DT[dtype]), 0.8
    timeouts_before = tcgen05_wait_timeouts() if dtype == "bfloat16" else 0
    h = stored(rng.standard_normal((n, width)), dtype)
    w_in = stored(rng.standard_normal((E, 2 * ff, width)) / np.sqrt(width) * 2, dtype)
    w_out = stored(rng.standard_normal((E, width, ff)) / np.sqrt(ff), dtype)
    z = rng.standard_normal((n, E))
    z[:, E - 1] = -50.0               # an expert that nobody chooses
    chosen_ref, weight_ref = pl.choose(stored(z, "float32"), top)
    chosen, weight = i32(chosen_ref), dev(weight_ref, torch.float32)
    few = n * top <= ops.MOE_FEW_SLOTS          # (the weight-streaming form, where the sizes allow 16-byte pieces)
    tm = ops.moe_tile_rows(n, top, width % 8 == 0 and ff % 8 == 0)
    assert tm == (128 if dtype == "bfloat16" and n * top >= 512 and width % 8 == 0 and ff % 8 == 0 else 32)
    tiles = ops.moe_max_tiles(n, top, E, tm)
    tile_expert = torch.full((tiles,), -9, device="cuda", dtype=torch.int32)
    pos_row, pos_slot = (torch.full((tiles * tm,), -9, device="cuda", dtype=torch.int32) for _ in range(2))
    slot_pos = torch.full((n * top,), -9, device="cuda", dtype=torch.int32)
    ops.moe_sort(chosen, E, tm, tile_expert, pos_row, pos_slot, slot_pos)
    te, pr, ps, sp = tile_expert.cpu().numpy(), pos_row.cpu().numpy(), pos_slot.cpu().numpy(), slot_pos.cpu().numpy()
    assert sorted(ps[ps >= 0].tolist()) == list(range(n * top))                             # every slot once
    for p in np.nonzero(ps >= 0)[0]:
        assert te[p // tm] == chosen_ref.reshape(-1)[ps[p]] and pr[p] == ps[p] // top and sp[ps[p]] == p      # in a tile of its expert
    both = torch.full((tiles * tm, 2 * ff), float("nan"), device="cuda", dtype=DT[dtype])
    if tm == 128:
        rows = torch.full((tiles * tm, width), float("nan"), device="cuda", dtype=DT[dtype])
        ops.gather_rows(dev(h, DT[dtype]), pos_row, rows)
        ops.grouped_linear(rows, dev(w_in, DT[dtype]), both, tile_expert, pos_slot)
    else:
        ops.grouped_linear(dev(h, DT[dtype]), dev(w_in, DT[dtype]), both, tile_expert, pos_slot, in_rows=pos_row, few_rows=few)
    hid = torch.empty((tiles * tm, ff), device="cuda", dtype=DT[dtype])
    ops.clamped_glu(both[:, :ff], both[:, ff:], hid, limit)
    outs = torch.full((tiles * tm, width), float("nan"), device="cuda")
    ops.grouped_linear(hid, dev(w_out, DT[dtype]), outs, tile_expert, pos_slot, few_rows=few)
    residual = stored(rng.standard_normal((n, width)), "float32")
    res = dev(residual, torch.float32)
    ops.moe_combine(res, outs, slot_pos, weight)
    want = residual.copy()
    for r in range(n):
        for e, g in zip(chosen_ref[r], weight_ref[r]):
            y = pl.clamped_glu(h[r] @ w_in[e, :ff].T, h[r] @ w_in[e, ff:].T, limit)
            if dtype == "bfloat16":
                y = stored(y, dtype)
            want[r] += g * (y @ w_out[e].T)
    assert rel(res, want) < (1e-5 if dtype == "float32" else 1e-2)
    if tm == 128:
        assert tcgen05_wait_timeouts() == timeouts_before            # no bounded wait of the tensor-core product ran out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_gate_on_both_sides_of_its_limits(dtype):
    ops, limit = Ops(DT[dtype]), 1.5
    g = stored(np.linspace(-6, 6, 97)[None, :].repeat(3, 0), dtype)
    u = stored(np.linspace(4, -4, 97)[None, :].repeat(3, 0) * np.array([[1.0], [0.3], [-1.0]]), dtype)
    out = torch.empty((3, 97), device="cuda", dtype=DT[dtype])
    wide = dev(np.concatenate([g, u], 1), DT[dtype])
    ops.clamped_glu(wide[:, :97], wide[:, 97:], out, limit)
    assert rel(out, pl.clamped_glu(g, u, limit)) < (1e-6 if dtype == "float32" else 6e-3)
