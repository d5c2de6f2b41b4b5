"""The Ravutar design on the CPU: configuration, tensor names and shapes, run order and cache entries, refused
configurations, loader errors and the random-weights folder."""
import copy
import json

import pytest
import torch

import ravutar_helpers as rh
from tinyinfer_b200 import models  # noqa: F401
from tinyinfer_b200.config import RavutarConfig, load_config, lookup_architecture, preset_config
from tinyinfer_b200.weights import write_random_model


def build(cfg):
    return lookup_architecture("Ravutar").model_factory(RavutarConfig.from_dict(cfg), torch.float32, "cpu")


@pytest.mark.parametrize("name", ["MIX", "WIDE", "ONE"])
def test_names_and_shapes_follow_the_configuration(name):
    cfg = getattr(rh, name)
    want = rh.tensor_shapes(cfg)
    got = build(cfg).expected_tensors()
    assert set(got) == set(want)
    assert {n: tuple(ts.shape) for n, ts in got.items()} == want


def test_a_size_that_only_the_checkpoint_gives(tmp_path):
    cfg = copy.deepcopy(rh.ONE)
    del cfg["layers"][0]["mixer"]["right"]["gate_rank"]
    shapes = {n: tuple(ts.shape) for n, ts in build(cfg).expected_tensors().items()}
    assert shapes["l0.mix.right.a1"] == (-1, 40) and shapes["l0.mix.right.a2"] == (40, -1)
    with pytest.raises(ValueError, match="only a checkpoint gives"):
        write_random_model(tmp_path / "r", RavutarConfig.from_dict(cfg), seed=1)


def test_run_order_and_cache_entries():
    model = build(rh.MIX)
    order = [(e.layer, e.cache, e.writes_cache) for e in model.spec.execution]
    assert order == [(0, 0, True), (1, 1, True), (2, 2, True), (1, 3, True), (2, 4, True), (3, 5, True)]
    needs = model.cache_needs()
    assert len(needs) == 6
    pages, state = needs[0]
    assert (pages.num_kv_heads, pages.head_dim, pages.planes) == (2, 20 + 12, 1)
    assert state.shape == (3 * (6 * 20 + 2 * 20 + 2 * 12) + 3 * 24 * 20,)          # convolution history, then the matrix state
    assert needs[1][0] is None and needs[1][1].shape == (6 * 12 * 20 + 2 * (6 * 12 + 2 * 3 * 20),)
    assert needs[2][1].shape == (2 * 12 * 36,) and needs[3] == needs[1] and needs[4] == needs[2]      # no convolution: no history
    assert [e.layer for e in build(rh.WIDE).spec.execution] == [0, 1, 0, 1, 0, 1]
    assert [e.layer for e in build(rh.ONE).spec.execution] == [0, 1]


def test_streams_and_constants_reach_the_specs():
    spec = build(rh.MIX).spec
    assert all(l.arrangement == "multi_stream" and l.streams == 3 and l.learned_mixing for l in spec.layers)
    first = spec.layers[0].mixer
    assert first.kind == "parallel" and first.scales == (0.9, 1.2) and first.prefixes == ("left.", "right.")
    attention, linear = first.branches
    assert attention.query_temperature == (0.4, 8) and attention.sink == 0.0 and attention.conv_taps == 4
    assert (linear.tau, linear.gate_rank, linear.norm_eps) == (6.0, 10, 1e-5)
    assert spec.layers[2].mixer.branches[0].query_temperature is None and spec.layers[2].feed_forward is None
    plain_residual = build(rh.WIDE).spec.layers[0]
    assert plain_residual.streams == 1 and not plain_residual.learned_mixing
    assert not any("hc" in n for n in build(rh.WIDE).expected_tensors())


@pytest.mark.parametrize("edit,message", [
    (lambda c: c["layers"][0].update(type="window"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "multiple of left.kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(groups=4), "multiple of groups"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=7), "multiple of norm_groups"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "lacks mixer.right"),
    (lambda c: c["layers"][0].update(mlp=dict(kind="moe")), "unknown feed-forward"),
    (lambda c: c.update(loop=dict(start=2, stop=9, times=2)), "loop"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.pop("norm"), "lacks required keys"),
])
def test_refused_configurations(edit, message):
    cfg = copy.deepcopy(rh.MIX)
    edit(cfg)
    with pytest.raises(ValueError, match=message):
        RavutarConfig.from_dict(cfg)


def test_folder_round_trip_and_loader_errors(tmp_path):
    from tinyinfer_b200.weights import WeightError, load_weights
    folder = rh.write_folder(tmp_path / "m", rh.ONE, seed=1)
    arch, cfg = load_config(folder)
    assert arch.name == "Ravutar" and cfg.to_dict() == RavutarConfig.from_dict(cfg.to_dict()).to_dict()
    model = arch.model_factory(cfg, torch.float32, "cpu")
    load_weights(model, folder)
    assert model.blocks[0].mixer.branches[1].w_a1.shape == (10, 40)

    def spoil(t):
        del t["l0.hc1.mix"]
        t["l1.mix.D"] = torch.zeros(5)
        t["extra"] = torch.zeros(1)
    bad = rh.write_folder(tmp_path / "bad", rh.ONE, seed=1, edit=spoil)
    with pytest.raises(WeightError) as err:
        load_weights(arch.model_factory(cfg, torch.float32, "cpu"), bad)
    assert err.value.missing == ["l0.hc1.mix"] and err.value.unexpected == ["extra"]
    assert [n for n, _, _ in err.value.wrong_shape] == ["l1.mix.D"]


def test_random_weights_folder_and_presets(tmp_path):
    cfg = preset_config("ravutar-tiny")
    folder = write_random_model(tmp_path / "r", cfg, seed=3)
    stored = json.loads((folder / "config.json").read_text())
    assert stored["architecture"] == "Ravutar" and stored["loop"] == dict(start=1, stop=3, times=2)
    arch, again = load_config(folder)
    assert again.run_order() == [0, 1, 2, 1, 2]
    model = arch.model_factory(again, torch.float32, "cpu")
    from tinyinfer_b200.weights import load_weights
    load_weights(model, folder)
    mix = model.blocks[0].coefficients["hc1.mix"]
    assert mix.shape == (2, 2) and abs(float(mix[0, 0]) - 1.0) < 0.6           # near the identity: the streams survive
    for name in ("ravutar-1b", "ravutar-2b"):
        assert preset_config(name).model_spec().layers
