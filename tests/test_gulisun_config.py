"""Configuration, run order, cache needs and weight loading of the Gulisun design, on the CPU."""
import json

import pytest
import torch

import gulisun_helpers as gh
import plain_gulisun as plain


def build(cfg):
    from tinyinfer_b200.config import architecture_of
    import tinyinfer_b200.models  # noqa: F401
    arch = architecture_of(cfg)
    typed = arch.config_class.from_dict(cfg)
    return typed, arch.model_factory(typed, torch.float32, "cpu")


def test_names_and_shapes_are_the_checkpoints():
    for cfg in (gh.MIX, gh.WIDE):
        _, model = build(cfg)
        assert {n: tuple(t.shape) for n, t in model.expected_tensors().items()} == gh.tensor_shapes(cfg)


def test_run_order_shares_cache_entries_and_groups_them():
    from tinyinfer_b200.cache import group_cache_needs
    typed, model = build(gh.MIX)
    order = model.spec.execution
    assert [(s.cache, s.writes_cache) for s in order] == [(0, True), (1, True), (2, True), (0, False), (3, True)]
    needs = model.cache_needs()
    assert needs[0][0].head_dim == 40 + 12 and needs[0][0].planes == 1 and needs[0][1] is None
    assert needs[1][0] is None and needs[1][1].shape == (3, 96)
    assert needs[3][1].shape == (5, 40)
    assert [entries for _need, entries in group_cache_needs(needs)] == [[0], [2]]
    assert typed.to_dict()["layers"] == gh.MIX["layers"] and typed.to_dict()["architecture"] == "Gulisun"


def test_bad_configurations_are_refused():
    from tinyinfer_b200.config import GulisunConfig
    cfg = json.loads(json.dumps(gh.MIX))
    cfg["layers"][3]["mixer"]["kv_from"] = 1                 # a recurrent layer has no rows to share
    with pytest.raises(ValueError):
        GulisunConfig.from_dict(cfg)
    cfg = json.loads(json.dumps(gh.MIX))
    cfg["layers"][3]["mixer"]["kv_rank"] = 48               # the reader's latent must be the writer's
    with pytest.raises(ValueError):
        GulisunConfig.from_dict(cfg)
    cfg = json.loads(json.dumps(gh.MIX))
    cfg["layers"][1]["type"] = "something"
    with pytest.raises(ValueError):
        GulisunConfig.from_dict(cfg)


def test_loader_reports_what_does_not_fit(tmp_path):
    from tinyinfer_b200.weights import WeightError, load_weights
    folder = gh.write_folder(tmp_path / "m", gh.MIX, seed=1)
    _, model = build(gh.MIX)
    load_weights(model, folder)                              # fits
    assert model.blocks[3].feed_forward is None and model.head is model.embedding

    def edit(t):
        del t["l0.mix.sink"]
        t["l3.mix.dkv"] = torch.zeros(52, 72)               # a reader has no down projection of its own
    folder = gh.write_folder(tmp_path / "bad", gh.MIX, seed=1, edit=edit)
    with pytest.raises(WeightError) as err:
        load_weights(model, folder)
    assert err.value.missing == ["l0.mix.sink"] and err.value.unexpected == ["l3.mix.dkv"]


def test_random_weights_mode_writes_a_folder_the_plain_statement_runs(tmp_path):
    from tinyinfer_b200.config import preset_config
    from tinyinfer_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "r", preset_config("gulisun-tiny"), seed=4)
    cfg, w = gh.read_folder(folder)
    logits = plain.forward(cfg, w, [5, 17, 3, 200])
    assert logits.shape == (4, 256) and torch.isfinite(logits).all()


def test_plain_statement_is_causal_and_its_recurrence_carries_state():
    cfg = gh.MIX
    w = {k: v.double() for k, v in gh.draw_tensors(cfg, 2).items()}
    tokens = [3, 14, 15, 92, 65, 35, 89, 79, 32, 38]
    full = plain.forward(cfg, w, tokens)
    assert torch.allclose(plain.forward(cfg, w, tokens[:6]), full[:6], atol=1e-9)
    assert not torch.allclose(plain.forward(cfg, w, tokens[1:])[-1], full[-1], atol=1e-3)
