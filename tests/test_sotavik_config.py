"""Configuration, tensor list and random weights of the Sotavik design (no GPU)."""
import json

import pytest
import torch

import tiny_sotavik as ts


def test_config_round_trip_and_spec():
    from supersonic_b200.config import ConfigError, config_from_dict, known_architectures
    assert "Sotavik" in known_architectures()
    for name, (d, _, _) in ts.CONFIGS.items():
        cfg = config_from_dict(d)
        assert config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
        spec = cfg.build_spec()
        assert len(spec.blocks) == len(d["layers"]) and spec.vocab_size == d["vocab"]
        for b, layer in zip(spec.blocks, d["layers"]):
            assert b.kind == "parallel" and b.feed_forward_norm is None
            assert (b.feed_forward is None) == (layer["mlp"] is None)
            assert b.mixer.kind == {"latent_attention": "latent_attention", "gla": "gated_linear_attention"}[layer["type"]]
            assert (b.position is not None) == (layer["type"] == "latent_attention")
        assert spec.head.params["scale"] == d["logit_scale"]
    bad = json.loads(json.dumps(ts.P))
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(ts.P))
    bad["layers"][0]["mixer"]["rot"]["dims"] = 7
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(ts.P))
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_decay_rank_comes_from_the_stored_shape(tmp_path):
    from supersonic_b200.config import ConfigError, config_from_dict, load_config
    from supersonic_b200.weights import WeightStore, write_model_folder
    cfg, _, _ = ts.build("P")
    folder = write_model_folder(cfg, 5, str(tmp_path / "m"), std=0.1)
    d = json.load(open(folder + "/config.json"))
    for layer in d["layers"]:
        layer["mixer"].pop("decay_rank", None)               # as a folder of this design is written
    json.dump(d, open(folder + "/config.json", "w"))
    bare = load_config(folder)
    with pytest.raises(ConfigError):
        bare.tensor_shapes()
    store = WeightStore.from_dir(folder)
    full = bare.with_shapes(store)
    assert full.layers[1]["mixer"]["decay_rank"] == 8
    store.check(full.tensor_shapes(), integer=full.integer_tensor)
    assert store.get("l0.mlp.table").dtype == torch.int32 and store.get("l0.norm1").shape == ()


def test_weight_check_wants_integer_tables_and_float_matrices():
    from supersonic_b200.weights import WeightError, WeightStore
    cfg, store, plain = ts.build("P")
    store.check(cfg.tensor_shapes(), integer=cfg.integer_tensor)
    wrong = dict(plain)
    wrong["l0.mlp.table"] = plain["l0.mlp.table"].float()
    with pytest.raises(WeightError):
        WeightStore.from_tensors(wrong).check(cfg.tensor_shapes(), integer=cfg.integer_tensor)
    for name, t in plain.items():
        if name.endswith(".table"):
            rows = t.sort(dim=1).values
            assert t.shape[1] == 1 or bool((rows[:, 1:] != rows[:, :-1]).all())      # a row's experts differ
            assert int(t.min()) >= 0


def test_preflight_counts_every_part():
    from supersonic_b200.engine import preflight
    cfg, store, _ = ts.build("Q")
    est = preflight.estimate(cfg.build_spec(), store, torch.bfloat16, 512, 256, None, 1024)
    assert est.weights > 0 and est.cache > 0 and est.workspace > 0
    from supersonic_b200.cache import KvNeed, StateNeed
    needs = preflight.cache_needs(cfg.build_spec())
    assert needs[0] == StateNeed(1 * 40 * 72) and needs[1] == KvNeed(1, 44, None, value_dim=0)


def test_preset_and_command_line_names():
    from supersonic_b200.config import preset_config, preset_names
    assert "sotavik-small" in preset_names()
    cfg = preset_config("sotavik-small")
    assert cfg.architectures == ["Sotavik"] and cfg.model_type == "sotavik"
    spec = cfg.build_spec()
    assert {b.mixer.kind for b in spec.blocks} == {"latent_attention", "gated_linear_attention"}
    assert cfg.parameter_count() > 100_000_000
