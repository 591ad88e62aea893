"""The tests' own small configurations of the Sotavik design, and weights for them.

They differ from one another in every size: heads (1 to 4), plain and rotated query sizes,
rotated dimensions fewer than the rotated part, value sizes that differ from key sizes, head
widths that do not add up to the model's width, latent ranks, experts (top 1, 2 and 3, with and
without a shared expert, a layer without feed-forward), decay ranks, tau, logit scale, eps and
the order of the two mixers.  Matrices are drawn wide (std about 0.1 to 0.3) so that attention
and decays are far from uniform."""
import copy

import torch


def latent(heads, dim, rot_dim, vdim, rank, base=10000.0, dims=None, scale=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "rot": {"base": base, "dims": dims or rot_dim},
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}}


def gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}}


def moe(experts, top, ff, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": {"ff": shared} if shared else None}


def with_mlp(layer, mlp):
    layer = copy.deepcopy(layer)
    layer["mlp"] = mlp
    return layer


P = {"architecture": "Sotavik", "vocab": 97, "width": 64, "logit_scale": 0.7, "norm": {"eps": 1e-5},
     "layers": [with_mlp(latent(2, 16, 8, 24, 32), moe(5, 2, 40, 24)),
                with_mlp(gla(3, 20, 12, 4.0, 8), moe(3, 1, 16)),
                with_mlp(latent(1, 8, 16, 8, 16, base=500.0, dims=8), None)]}

Q = {"architecture": "Sotavik", "vocab": 130, "width": 48, "logit_scale": 1.0, "norm": {"eps": 3e-6},
     "layers": [with_mlp(gla(1, 40, 72, 9.0, 4), moe(4, 3, 24, 56)),
                with_mlp(latent(4, 24, 4, 16, 40, base=77.0, scale=0.21), moe(2, 2, 8)),
                with_mlp(gla(2, 8, 8, 1.0, 16), None),
                with_mlp(latent(3, 32, 32, 48, 64), moe(7, 2, 32, 32))]}

# sizes that no fast kernel takes (odd widths, ranks and head sizes, one expert of one, top = experts, a rotated
# part of two coordinates, a decay rank of one) beside ones that all of them take (multiples of 64)
R = {"architecture": "Sotavik", "vocab": 61, "width": 50, "logit_scale": 1.3, "norm": {"eps": 1e-4},
     "layers": [with_mlp(latent(3, 10, 6, 7, 21, base=300.0, dims=4), moe(3, 3, 9, 5)),
                with_mlp(gla(2, 7, 5, 2.5, 1), moe(1, 1, 11)),
                with_mlp(latent(5, 6, 2, 9, 12, base=50.0), moe(6, 1, 4, 13)),
                with_mlp(gla(1, 33, 3, 30.0, 3), None)]}

S = {"architecture": "Sotavik", "vocab": 256, "width": 128, "logit_scale": 0.5, "norm": {"eps": 1e-5},
     "layers": [with_mlp(latent(8, 64, 64, 64, 128), moe(8, 2, 128, 128)),
                with_mlp(latent(40, 16, 16, 16, 48, dims=8), moe(4, 4, 64)),
                with_mlp(gla(2, 128, 128, 8.0, 64), moe(16, 2, 64, 256))]}

CONFIGS = {"P": (P, 11, 0.15), "Q": (Q, 12, 0.2), "R": (R, 13, 0.25), "S": (S, 14, 0.1)}


def build(name_or_cfg, seed=0, std=0.15):
    """(typed configuration, weight store, float64 copies of the weights by name)."""
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.weights import random_store
    if isinstance(name_or_cfg, str):
        name_or_cfg, seed, std = CONFIGS[name_or_cfg]
    cfg = config_from_dict(name_or_cfg)
    store = random_store(cfg, seed, std=std)
    plain = {n: store.get(n) for n in store.names()}
    return cfg, store, plain


def replace(store_tensors, **changes):
    """A weight store with some tensors replaced (values are rounded to bfloat16 like stored weights)."""
    from supersonic_b200.weights import WeightStore
    t = dict(store_tensors)
    for k, v in changes.items():
        t[k.replace("__", ".")] = v.to(t[k.replace("__", ".")].dtype)
    return WeightStore.from_tensors(t), t
