"""Vepinex without a GPU: its configuration, plan, tensor list, cache needs and run order, sizes read from the
checkpoint's shapes, random-weights mode, and the plain implementation's pieces against each other."""
import json

import numpy as np
import pytest
import torch

from kvad_b200 import write_random_model
from kvad_b200.cache import KVNeed, StateNeed
from kvad_b200.config import ConfigError, JsonView, load_config, resolve
from kvad_b200.models.plan import LayerCall, Model
from kvad_b200.weights.safetensors_io import Checkpoint
from tests.plain import vepinex_plain as pl
from tests.vepinex_configs import CONFIGS, SEEDS


def build(folder):
    """The model as `Engine.from_pretrained` builds it, short of the device."""
    arch, cfg = load_config(folder)
    ckpt = Checkpoint.open_dir(folder)
    try:
        cfg = arch.with_checkpoint_shapes(cfg, lambda n: tuple(ckpt.entries[n].shape) if n in ckpt.entries else None)
    finally:
        ckpt.close()
    return cfg, Model(arch.plan(cfg))


def test_the_registry_finds_it_by_the_architecture_key():
    arch = resolve(JsonView(CONFIGS["A"]))
    assert arch.id == "vepinex"
    assert arch.read_config(JsonView(CONFIGS["A"])).width == 64


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_plan_asks_for_exactly_the_tensors_the_writer_writes(tmp_path, name):
    d = write_random_model(str(tmp_path), CONFIGS[name], SEEDS[name])
    cfg, model = build(d)
    stored = pl.read_tensors(str(tmp_path / "model.safetensors"))
    asked = {r.name: tuple(r.shape) for r in model.requests()}
    assert asked == {k: tuple(v.shape) for k, v in stored.items()}
    written = json.load(open(tmp_path / "config.json"))
    for got, want in zip(written["layers"], CONFIGS[name]["layers"]):     # the ranks are in the tensors' shapes only
        assert "decay_rank" not in got["mixer"] and "gate_rank" not in got["mixer"]
        assert got["mixer"] == {k: v for k, v in want["mixer"].items() if k not in ("decay_rank", "gate_rank")} and got["mlp"] == want["mlp"]
    for layer, want in zip(cfg.layers, CONFIGS[name]["layers"]):          # ... and come back from there
        if layer["type"] == "channel_delta":
            assert (layer["mixer"]["decay_rank"], layer["mixer"]["gate_rank"]) == (want["mixer"]["decay_rank"], want["mixer"]["gate_rank"])
    assert pl.forward(*pl.load(d), [1, 2, 3]).shape == (3, CONFIGS[name]["vocab"])


def test_cache_needs_and_run_order_follow_the_layers(tmp_path):
    d = write_random_model(str(tmp_path), CONFIGS["A"], SEEDS["A"])
    _, model = build(d)
    needs = model.cache_layout.needs
    assert needs[0] == KVNeed(1, 24 + 4, None, value_dim=0)                # the latent and the rotated part, no values
    assert needs[1] == StateNeed((4 * 8 * 16 + 2 * (2 * 2 * 16 + 4 * 8),), torch.float32)       # the matrices, and two kept inputs of q | k | v
    assert needs[2] == StateNeed((3 * (20 * 8 + 2 * (8 + 1)),), torch.float32)                  # the matrices; n and m per block of 16 columns
    assert len(needs) == 3                                                 # the last layer keeps nothing: it reads entry 0
    assert model.plan.order == (LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 2), LayerCall(3, 0, writes_cache=False))
    assert model.graph_safe and model.max_positions is None
    assert model.cache_layout.bytes_per_token(2) == 2 * 28


def test_libraries_are_those_of_the_models_parts():
    from kvad_b200.ops import libraries_for
    arch = resolve(JsonView(CONFIGS["A"]))
    fams = Model(arch.plan(arch.read_config(JsonView(CONFIGS["A"])))).kernel_families()
    libs = libraries_for(torch.bfloat16, fams)
    assert {"norm_rotary", "attention_scored", "gated_recurrence", "moe", "linear_tcgen05"} <= set(libs)
    assert not {"attention_prefill", "attention_decode", "attention_simt", "retention"} & set(libs)


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][0].update(type="convolution"), "type"),
    (lambda c: c["layers"][2]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "divide"),
    (lambda c: c["layers"][0]["mixer"].update(rot_dim=3), "rotat"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=2), "rotat"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "latent"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=16), "latent size"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "experts"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "mlp"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_a_configuration_that_cannot_be_run_is_refused(change, what):
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    change(cfg)
    arch = resolve(JsonView(cfg))
    with pytest.raises(ConfigError, match=what):
        arch.read_config(JsonView(cfg))


def test_fused_maps_keep_their_columns_apart():
    from kvad_b200.parts.linear import FusedLinear
    f = FusedLinear("x.", 8, [("a", 3), ("b", 5), ("c", 2, 8), ("d", 1, 4)], pad_to=16, bias_suffix=".b")
    assert [f.columns(i) for i in range(4)] == [slice(0, 3), slice(3, 8), slice(8, 10), slice(12, 13)] and f.out_features == 16
    mats = {f"x.{n}": torch.full((s, 8), float(i + 1)) for i, (n, s) in enumerate(zip("abcd", (3, 5, 2, 1)))}
    mats.update({f"x.{n}.b": torch.full((s,), 10.0 * (i + 1)) for i, (n, s) in enumerate(zip("abcd", (3, 5, 2, 1)))})
    f.load_own(lambda name, keep_f32=False: mats[name])
    assert f.weight[:, 0].tolist() == [1.0] * 3 + [2.0] * 5 + [3.0] * 2 + [0.0] * 2 + [4.0] + [0.0] * 3
    assert f.bias.tolist() == [10.0] * 3 + [20.0] * 5 + [30.0] * 2 + [0.0] * 2 + [40.0] + [0.0] * 3
    assert sorted(r.name for r in f.own_requests()) == sorted(mats)


def test_plain_mechanisms_agree_with_each_other():
    """The oracle's own pieces, checked against each other where the design says two things are the same."""
    rng = np.random.default_rng(0)
    # a rotation keeps lengths, position 0 turns nothing, and what lies past `dims` passes
    x = rng.standard_normal((5, 2, 8))
    y = pl.rotate_pairs(x, np.arange(5), 100.0, 6)
    assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1)) and np.array_equal(y[0], x[0]) and np.array_equal(y[..., 6:], x[..., 6:])
    # a convolution with one tap is a scaling; with more, the last column meets the row itself
    x, taps = rng.standard_normal((7, 3)), rng.standard_normal((3, 4))
    assert np.allclose(pl.short_conv(x, taps[:, 3:]), x * taps[:, 3])
    assert np.allclose(pl.short_conv(x, taps)[0], x[0] * taps[:, 3]) and np.allclose(pl.short_conv(x, taps)[1], x[1] * taps[:, 3] + x[0] * taps[:, 2])
    # the matrix memory in two portions is the matrix memory; with no forgetting and level gates it is a running mean of sorts
    T, dk, dv = 12, 5, 4
    q, k, v = rng.standard_normal((T, dk)), rng.standard_normal((T, dk)), rng.standard_normal((T, dv))
    gi, gf = pl.gate_caps(rng.standard_normal(T) * 9, rng.standard_normal(T) * 9, 4.0)
    assert np.all(np.abs(gi) <= 4.0) and np.all(gf < 0)
    whole, _ = pl.matrix_memory_cell(q, k, v, gi, gf)
    first, state = pl.matrix_memory_cell(q[:5], k[:5], v[:5], gi[:5], gf[:5])
    rest, _ = pl.matrix_memory_cell(q[5:], k[5:], v[5:], gi[5:], gf[5:], state)
    assert np.allclose(np.concatenate([first, rest]), whole)
    # the first row: the running maximum starts at 0, not at the first input gate
    o, (S, n, m) = pl.matrix_memory_cell(q[:1], k[:1], v[:1], np.array([-3.0]), np.array([-0.5]))
    assert m == -0.5 and np.allclose(S, np.exp(-3.0 + 0.5) * np.outer(k[0], v[0]))
    # the delta rule with beta = 1, no decay and orthonormal keys stores and returns each value exactly
    keys = np.eye(dk)[:4]
    vals = rng.standard_normal((4, dv))
    out, S = pl.delta_cell(keys, keys, vals, np.ones(4), np.ones((4, dk)))
    assert np.allclose(out, vals) and np.allclose(S[:4], vals)
    # ... and writing the same key twice replaces the value
    out, _ = pl.delta_cell(keys[[0, 0]], keys[[0, 0]], vals[:2], np.ones(2), np.ones((2, dk)))
    assert np.allclose(out[1], vals[1])
    # the router: the chosen weights sum to one; with all experts chosen it is the softmax of all logits
    z = rng.standard_normal((6, 5))
    c, w = pl.choose(z, 2)
    assert np.allclose(w.sum(-1), 1.0) and np.array_equal(c[:, 0], z.argmax(-1))
    c, w = pl.choose(z, 5)
    assert np.allclose(np.take_along_axis(pl.softmax_rows(z), c, -1), w)
    # the clamped gate: level above the limit on the gate side, clamped on both sides for the other
    assert pl.clamped_glu(np.array([9.0]), np.array([0.3]), 2.0) == pl.clamped_glu(np.array([2.0]), np.array([0.3]), 2.0)
    assert pl.clamped_glu(np.array([1.0]), np.array([-7.0]), 2.0) == pl.clamped_glu(np.array([1.0]), np.array([-2.0]), 2.0)
