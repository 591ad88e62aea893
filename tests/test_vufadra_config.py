"""The Vufadra configuration without a GPU: reading and refusing config.json, the parts and the schedule it
builds, tensor shapes, what the cache is asked for, and the scaled rotation frequencies against the plain
statement."""
import copy
import json
import math

import pytest
import torch

import plain_vufadra as pv
import tiny_vufadra as tv
from supersonic_b200.config import ConfigError, config_from_dict, load_config


def test_reads_every_key_and_round_trips():
    cfg = config_from_dict(tv.A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (97, 64, 1e-5)
    assert cfg.bigram == {"buckets": 53, "mul_prev": 31, "mul_cur": 5}
    assert cfg.loop == {"start": 1, "stop": 3, "times": 3}
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.architectures == ["Vufadra"]


def test_schedule_walks_the_loop_with_a_cache_entry_per_run():
    spec = config_from_dict(tv.A).build_spec()
    assert [(s.layer, s.before) for s in spec.schedule] == \
        [(0, None), (1, (0, 0)), (2, None), (1, (0, 1)), (2, None), (1, (0, 2)), (2, None)]
    assert [s.cache for s in spec.schedule] == list(range(7))
    assert [a.kind for a in spec.adapters] == ["loop_input"] and spec.adapters[0].params["passes"] == 3
    # a loop over everything, walked twice; and no loop at all: no adapter, every layer once
    assert [(s.layer, s.before) for s in config_from_dict(tv.D).build_spec().schedule] == \
        [(0, (0, 0)), (1, None), (2, None), (0, (0, 1)), (1, None), (2, None)]
    plain = config_from_dict(tv.C).build_spec()
    assert [(s.layer, s.before) for s in plain.schedule] == [(0, None), (1, None), (2, None)] and not plain.adapters
    zero = copy.deepcopy(tv.A)
    zero["loop"]["times"] = 0
    unlooped = config_from_dict(zero)
    assert not unlooped.build_spec().adapters and unlooped.ignorable_tensor("loop.in")
    assert not config_from_dict(tv.A).ignorable_tensor("loop.in")


def test_parts_and_their_parameters():
    cfg = config_from_dict(tv.A)
    spec = cfg.build_spec()
    assert spec.embedding.kind == "pair_embedding" and spec.embedding.params["buckets"] == 53
    kinds = [b.mixer.kind for b in spec.blocks]
    assert kinds == ["mixer_pair", "real_gated_recurrence", "delta_rule"]
    b0 = spec.blocks[0]
    assert b0.kind == "parallel" and b0.mixer_norm.kind == "dynamic_tanh" and b0.feed_forward_norm.kind == "dynamic_tanh"
    assert b0.params == {"token_shift": {"size": 64}} and b0.weights == {"shift": "l0.shift"}
    left = b0.mixer.params["left"]["params"]
    assert (left["chunk"], left["num_heads"], left["num_kv_heads"], left["dim"], left["value_dim"]) == (20, 4, 2, 16, 24)
    assert b0.position.params["scaling"]["kind"] == "yarn" and b0.position.params["rotary_dim"] == 8
    assert spec.blocks[1].feed_forward is None and spec.blocks[1].feed_forward_norm is None
    assert spec.final_norm.kind == "dynamic_tanh"


def test_tensor_shapes_and_decay_rank_from_the_stored_tensor(tmp_path):
    from supersonic_b200.weights import WeightStore, write_model_folder
    cfg = config_from_dict(tv.C)
    shapes = cfg.tensor_shapes()
    assert shapes["bigram"] == [18, 50] and shapes["l1.mix.left.o"] == [50, 42] and shapes["l1.mix.right.u"] == [5, 6]
    assert shapes["l0.mix.ra"] == [5, 6, 6] and shapes["l0.mix.conv"] == [30, 5] and shapes["l2.mix.w1"] == [3, 50]
    assert "loop.in" not in shapes and "l2.norm2" not in shapes and shapes["final.norm.alpha"] == []
    folder = write_model_folder(cfg, 1, str(tmp_path / "m"))
    d = json.load(open(folder + "/config.json"))
    d["layers"][2]["mixer"].pop("decay_rank")
    d["layers"][1]["mixer"]["right"].pop("decay_rank")
    json.dump(d, open(folder + "/config.json", "w"))
    bare = load_config(folder)
    with pytest.raises(ConfigError):
        bare.tensor_shapes()
    full = bare.with_shapes(WeightStore.from_dir(folder))
    assert full.tensor_shapes() == shapes
    WeightStore.from_dir(folder).check(full.tensor_shapes())


@pytest.mark.parametrize("change,where", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv heads"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].__setitem__("blocks", 5), "blocks"),
    (lambda d: d["loop"].__setitem__("stop", 9), "loop"),
    (lambda d: d["embedding"]["bigram"].__setitem__("buckets", 0), "bucket"),
    (lambda d: d["layers"][2].__setitem__("mlp", {"kind": "moe", "ff": 8}), "mlp.kind"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_refuses_what_it_cannot_build(change, where):
    d = copy.deepcopy(tv.A)
    change(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert where in str(e.value)


def test_cache_needs_nest_and_flatten():
    from supersonic_b200.cache import KvNeed, StateNeed, flatten_needs
    from supersonic_b200.engine.preflight import cache_needs
    spec = config_from_dict(tv.A).build_spec()
    flat = flatten_needs(cache_needs(spec))
    assert flat["embedding"] == StateNeed(1, "int32")
    # stop 0 is the pair: attention pages (kept no longer than a chunk), the other half's matrices and last row
    assert flat[((0, "mixer"), "left")] == KvNeed(2, 16, 20, value_dim=24)
    assert flat[(((0, "mixer"), "right"), "state")] == StateNeed(2 * 12 * 12)
    assert flat[(((0, "mixer"), "right"), "last")] == StateNeed(64)
    assert flat[(0, "shift")] == StateNeed(64)
    # the looped layers have an entry per run
    for stop in (1, 3, 5):
        assert flat[((stop, "mixer"), "state")] == StateNeed(48) and flat[((stop, "mixer"), "tail")] == StateNeed(2 * 48)
    for stop in (2, 4, 6):
        assert flat[(stop, "mixer")] == StateNeed(3 * 20 * 20) and flat[(stop, "shift")] == StateNeed(64)


def test_state_rows_of_the_cache_on_the_host():
    """Nested needs become stores of their own; integer state stays integer; a slot comes back zeroed."""
    from supersonic_b200.cache import KvNeed, SequenceCache, StateNeed
    cache = SequenceCache({"e": StateNeed(1, "int32"), 0: {"mixer": {"left": KvNeed(1, 8, 16, value_dim=4), "right": StateNeed(6)},
                                                           "shift": StateNeed(3)}},
                          256, 128, torch.float32, "cpu")
    assert cache.state("e").dtype == torch.int32 and cache.state((0, "shift")).shape[1] == 3
    k, v, table, _ = cache.kv(((0, "mixer"), "left"))
    assert k.shape[-1] == 8 and v.shape[-1] == 4
    s = cache.acquire()
    cache.state(((0, "mixer"), "right"))[s] += 2.0
    cache.state("e")[s] += 5
    cache.release(s)
    assert cache.acquire() == s
    assert float(cache.state(((0, "mixer"), "right"))[s].abs().sum()) == 0 and int(cache.state("e")[s]) == 0


@pytest.mark.parametrize("rot", [{"base": 1000.0, "dims": 8, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}},
                                 {"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0}},
                                 {"base": 50.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}},
                                 {"base": 77.0, "dims": 24}])
def test_scaled_frequencies_and_table_gain_against_the_plain_statement(rot):
    from supersonic_b200.parts.rotary import scaled_inverse_frequencies, table_gain
    sc = rot.get("scaling")
    scaling = None if not sc else dict(sc, kind="yarn")
    inv = scaled_inverse_frequencies(rot["dims"], rot["base"], scaling)
    cos, sin = pv.rotary_angles(7, rot)
    gain = table_gain(scaling)
    ang = torch.arange(7, dtype=torch.float64)[:, None] * inv[None, :]
    assert torch.allclose(ang.cos() * gain, cos, atol=1e-12) and torch.allclose(ang.sin() * gain, sin, atol=1e-12)
    if sc:
        assert gain == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)
        plain = 1.0 / rot["base"] ** (2.0 * torch.arange(rot["dims"] // 2, dtype=torch.float64) / rot["dims"])
        assert float((inv / plain).min()) >= 1.0 / sc["factor"] - 1e-12 and float((inv / plain).max()) <= 1.0 + 1e-12


def test_random_weights_have_every_tensor_and_sane_constants():
    cfg, store, plain = tv.build("A")
    store.check(cfg.tensor_shapes())
    assert 0.0 <= float(plain["l0.shift"].float().min()) and float(plain["l0.shift"].float().max()) <= 1.0
    assert 0.4 < float(plain["l0.norm1.alpha"]) < 1.1
    assert abs(float(plain["l0.norm1"].float().mean()) - 1.0) < 0.2
