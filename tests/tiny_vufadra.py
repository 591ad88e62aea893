"""The tests' own small configurations of the Vufadra design, and weights for them.

They differ from one another in every size and in the order of the mixers: query heads over fewer, as many
and a single kv head; value rows narrower than, as wide as and wider than key rows; rotated coordinates fewer
than and equal to the head's; with and without frequency scaling; chunks shorter than, equal to and longer
than a cache page; convolutions of one to five taps; one and several gate blocks; decay ranks down to one;
layers without feed-forward; loops over some or all layers, walked once, twice or three times, and none.
Matrices are drawn wide so that weights and decays are far from uniform."""
import copy

import torch


def rglru(width, conv, blocks):
    return {"type": "rglru", "mixer": {"width": width, "conv": conv, "blocks": blocks}}


def delta(heads, dim, rank):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}


def pair(heads, kv_heads, dim, vdim, size, rot_dims, base, scaling, r_heads, r_dim, r_rank, scale=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size},
                               "rot": rot, "scale": scale if scale is not None else dim ** -0.5},
                      "right": {"heads": r_heads, "dim": r_dim, "decay_rank": r_rank}}}


def with_mlp(layer, ff):
    layer = copy.deepcopy(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return layer


def model(vocab, width, eps, bigram, loop, layers):
    d = {"architecture": "Vufadra", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "embedding": {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}, "layers": layers}
    if loop is not None:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


A = model(97, 64, 1e-5, (53, 31, 5), (1, 3, 3),
          [with_mlp(pair(4, 2, 16, 24, 20, 8, 1000.0, (8.0, 64, 16.0, 2.0), 2, 12, 6), 40),
           with_mlp(rglru(48, 3, 3), None),
           with_mlp(delta(3, 20, 5), 72)])

B = model(130, 48, 3e-6, (200, 7, 3), (0, 1, 1),
          [with_mlp(delta(1, 40, 4), 24),
           with_mlp(pair(3, 3, 24, 24, 64, 24, 77.0, None, 1, 16, 8, scale=0.21), 56),
           with_mlp(rglru(64, 1, 1), 32)])

# sizes that no fast kernel takes: odd widths, ranks and head sizes, one kv head, a rank of one, five taps
C = model(61, 50, 1e-4, (17, 1, 1), None,
          [with_mlp(rglru(30, 5, 5), 9),
           with_mlp(pair(6, 1, 10, 7, 7, 4, 50.0, (2.0, 16, 4.0, 1.0), 5, 6, 1), 11),
           with_mlp(delta(2, 33, 3), None)])

# round sizes, which every fast kernel takes
D = model(256, 128, 1e-6, (300, 13, 11), (0, 3, 2),
          [with_mlp(pair(8, 2, 64, 64, 128, 32, 10000.0, (4.0, 256, 32.0, 1.0), 2, 64, 16), 256),
           with_mlp(delta(2, 64, 16), 128),
           with_mlp(rglru(128, 4, 2), 128)])

CONFIGS = {"A": (A, 21, 0.15), "B": (B, 22, 0.2), "C": (C, 23, 0.25), "D": (D, 24, 0.1)}


def build(name_or_cfg, seed=0, std=0.15):
    """(typed configuration, weight store, the weights by name)."""
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.weights import random_store
    if isinstance(name_or_cfg, str):
        name_or_cfg, seed, std = CONFIGS[name_or_cfg]
    cfg = config_from_dict(name_or_cfg)
    store = random_store(cfg, seed, std=std)
    plain = {n: store.get(n) for n in store.names()}
    return cfg, store, plain


def changed(plain, **changes):
    """(weight store, weights by name) with some tensors replaced; ``__`` in a keyword stands for a dot."""
    from supersonic_b200.weights import WeightStore
    t = dict(plain)
    for k, v in changes.items():
        name = k.replace("__", ".")
        t[name] = v.to(t[name].dtype)
    return WeightStore.from_tensors(t), t
