"""Nifulix without a GPU: its configuration, plan, tensor list, cache needs and random-weights mode."""
import json

import numpy as np
import pytest

from kvad_b200 import write_random_model
from kvad_b200.cache import KVNeed, SlotBook, StateNeed
from kvad_b200.config import ConfigError, JsonView, load_config, resolve
from kvad_b200.models.plan import Model
from tests.nifulix_configs import CONFIGS, SEEDS
from tests.plain.nifulix_plain import PlainNifulix, read_tensors


def test_the_registry_finds_it_by_the_architecture_key():
    arch = resolve(JsonView(CONFIGS["P"]))
    assert arch.id == "nifulix"
    assert arch.read_config(JsonView(CONFIGS["P"])).width == 48


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_plan_asks_for_exactly_the_tensors_the_writer_writes(tmp_path, name):
    d = write_random_model(str(tmp_path), CONFIGS[name], SEEDS[name])
    arch, cfg = load_config(d)
    model = Model(arch.plan(cfg))
    stored = read_tensors(str(tmp_path / "model.safetensors"))
    asked = {r.name: tuple(r.shape) for r in model.requests()}
    assert asked == {k: tuple(v.shape) for k, v in stored.items()}
    assert json.load(open(tmp_path / "config.json"))["layers"] == CONFIGS[name]["layers"]
    # and the plain implementation runs on the folder
    assert PlainNifulix(d).forward([1, 2, 3]).shape == (3, CONFIGS[name]["vocab"])


def test_cache_needs_follow_the_mixers():
    arch, cfg = resolve(JsonView(CONFIGS["Q"])), None
    cfg = arch.read_config(JsonView(CONFIGS["Q"]))
    layout = Model(arch.plan(cfg)).cache_layout
    needs = layout.needs
    assert needs[0] == KVNeed(1, 32, None, value_dim=16, keep_first=0)
    assert needs[1] == KVNeed(1, 48, None, value_dim=0)                    # the latent and the rotated part, no values
    assert needs[2] == KVNeed(3, 16, 70, value_dim=32, keep_first=5)
    assert needs[3] == StateNeed((2, 24, 16))
    assert needs[5] == KVNeed(1, 34, 66, value_dim=0)
    assert layout.bytes_per_token(2) == 2 * ((32 + 16) + 48 + 2 * 3 * (16 + 32) + 34)


def test_libraries_are_those_of_the_models_parts():
    import torch

    from kvad_b200.ops import libraries_for
    arch = resolve(JsonView(CONFIGS["P"]))
    fams = Model(arch.plan(arch.read_config(JsonView(CONFIGS["P"])))).kernel_families()
    libs = libraries_for(torch.float32, fams)
    assert {"norm_rotary", "attention_scored", "retention"} <= set(libs)
    assert not {"attention_prefill", "attention_decode", "attention_simt", "linear_tcgen05"} & set(libs)
    assert "attention_decode" in libraries_for(torch.float32)               # a model of plain attention layers


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][0].update(type="convolution"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("decay"), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "divide"),
    (lambda c: c["layers"][2]["mixer"].update(rot_dim=3), "rot_dim"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=8), "one shape"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "mlp"),
])
def test_a_configuration_that_cannot_be_run_is_refused(change, what):
    cfg = json.loads(json.dumps(CONFIGS["P"]))
    change(cfg)
    arch = resolve(JsonView(cfg))
    with pytest.raises(ConfigError, match=what):
        arch.read_config(JsonView(cfg))


def test_kept_first_pages_are_never_dropped():
    book = SlotBook(2, [16], [70], page_size=64, keep_first=[5])
    s = book.acquire()
    book.grow(s, 400)
    book.trim_windows(s)
    table = book.pages[s][0]
    assert table[0] >= 0                                # holds positions 0..4, which every later query sees
    assert table[1:5] == [-1, -1, -1, -1]               # 64..319: behind the window of the query at 400 (331..400)
    assert all(p >= 0 for p in table[5:])
    free_before = book.pools[0].n_free
    book.release(s)
    assert book.pools[0].n_free == free_before + 3      # the kept page and the two of the window
    book.check_all_free()
    # without kept positions the first page goes too
    book = SlotBook(1, [16], [70], page_size=64)
    s = book.acquire()
    book.grow(s, 400)
    book.trim_windows(s)
    assert book.pages[s][0][:5] == [-1] * 5


def test_plain_mechanisms_agree_with_each_other():
    """The oracle's own pieces, checked against each other where the design says two things are the same."""
    from tests.plain import nifulix_plain as pl
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 2, 8))
    # a rotation keeps lengths, and position 0 turns nothing
    for layout in ("half", "interleaved"):
        y = pl.rotate(x, np.arange(5), 100.0, 6, layout)
        assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
        assert np.array_equal(y[0], x[0]) and np.array_equal(y[..., 6:], x[..., 6:])
    # a window of n keeps everything causal; kept first tokens stay visible
    assert np.array_equal(pl.visible(6, 6), np.tril(np.ones((6, 6), bool)))
    v = pl.visible(9, 3, 2)
    assert v[8].tolist() == [True, True, False, False, False, False, True, True, True]
