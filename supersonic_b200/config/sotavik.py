"""Typed configuration of the ``Sotavik`` architecture.

Its config.json is nested.  Top level: ``vocab``, ``width``, ``logit_scale``, ``norm.eps`` and ``layers``, a list
with one entry per layer: ``type`` (``latent_attention`` or ``gla``), ``mixer`` (that mixer's sizes and
constants) and ``mlp`` (null, or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"},
"shared": {"ff"} or null}``).  ``build_spec`` turns that into parts: a ``parallel`` block per layer (a norm
with a single gain, read by mixer and feed-forward alike) with a depth average behind it, experts routed by
a token-id table, a head with scaled logits.  Tensor names are ``embed``, ``head``, ``final.norm`` and, per
layer i, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.dwa``.

One size is not in config.json: the inner width of a ``gla`` layer's decay projection, which is the first
dimension of ``l<i>.mix.a1`` (``with_shapes`` reads it from the stored tensor; a configuration made by hand
may give it as ``mixer.decay_rank``).  The design has no position limit; the cache bounds a sequence.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from .base import BlockSpec, ConfigError, ModelSpec, PartSpec, default_schedule

ARCHITECTURE = "Sotavik"
MIXERS = ("latent_attention", "gla")
NO_POSITION_LIMIT = 1 << 20


def _need(d: Dict[str, Any], keys, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"{where} is missing {missing}")


def _positive(d: Dict[str, Any], keys, where: str) -> None:
    for k in keys:
        if not (isinstance(d[k], int) and d[k] > 0):
            raise ConfigError(f"{where}.{k} must be a positive integer, got {d[k]!r}")


@dataclass(frozen=True)
class SotavikConfig:
    vocab: int
    width: int
    logit_scale: float
    norm_eps: float
    layers: List[Dict[str, Any]] = field(default_factory=list)
    eos_token_ids: List[int] = field(default_factory=list)
    model_type: str = "sotavik"

    # ---- reading -----------------------------------------------------
    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "SotavikConfig":
        _need(d, ("vocab", "width", "layers", "norm"), "config.json")
        _need(d["norm"], ("eps",), "norm")
        eos = d.get("eos_token_id")
        cfg = SotavikConfig(
            vocab=int(d["vocab"]), width=int(d["width"]), logit_scale=float(d.get("logit_scale", 1.0)),
            norm_eps=float(d["norm"]["eps"]), layers=copy.deepcopy(list(d["layers"])),
            eos_token_ids=[] if eos is None else [int(eos)] if isinstance(eos, int) else [int(e) for e in eos])
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not self.layers:
            raise ConfigError("layers must name at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            m = layer["mixer"]
            if layer["type"] == "latent_attention":
                _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"), where + ".mixer")
                _positive(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank"), where + ".mixer")
                _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                dims = m["rot"]["dims"]
                if not isinstance(dims, int) or dims <= 0 or dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must be even and at most rot_dim, got {dims!r}")
            elif layer["type"] == "gla":
                _need(m, ("heads", "dim", "vdim", "tau"), where + ".mixer")
                _positive(m, ("heads", "dim", "vdim"), where + ".mixer")
                if not float(m["tau"]) > 0:
                    raise ConfigError(f"{where}.mixer.tau must be positive")
            else:
                raise ConfigError(f"{where}.type {layer['type']!r} is not known (known: {list(MIXERS)})")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind", "moe") != "moe":
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not known (known: 'moe')")
            _need(mlp, ("expert", "router"), where + ".mlp")
            _need(mlp["expert"], ("ff",), where + ".mlp.expert")
            _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
            _positive(mlp["expert"], ("ff",), where + ".mlp.expert")
            _positive(mlp["router"], ("experts", "top"), where + ".mlp.router")
            for part in ("expert", "shared"):
                act = (mlp.get(part) or {}).get("act", "silu")
                if act != "silu":
                    raise ConfigError(f"{where}.mlp.{part}.act {act!r} is not supported (the design's experts gate with silu)")
            if mlp["router"]["top"] > mlp["router"]["experts"]:
                raise ConfigError(f"{where}.mlp.router.top exceeds the number of experts")
            if mlp.get("shared"):
                _need(mlp["shared"], ("ff",), where + ".mlp.shared")
                _positive(mlp["shared"], ("ff",), where + ".mlp.shared")
        for e in self.eos_token_ids:
            if not 0 <= e < self.vocab:
                raise ConfigError(f"eos_token_id {e} is outside the vocabulary")

    def with_shapes(self, store) -> "SotavikConfig":
        """The configuration with the sizes that only tensor shapes give: a gla layer's decay rank."""
        layers = copy.deepcopy(self.layers)
        for i, layer in enumerate(layers):
            name = f"l{i}.mix.a1"
            if layer["type"] == "gla" and "decay_rank" not in layer["mixer"] and name in store:
                shape = store.shape(name)
                if len(shape) == 2:
                    layer["mixer"]["decay_rank"] = int(shape[0])
        return SotavikConfig(self.vocab, self.width, self.logit_scale, self.norm_eps, layers,
                             list(self.eos_token_ids), self.model_type)

    # ---- writing -----------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": ARCHITECTURE, "layers": copy.deepcopy(self.layers),
                             "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
                             "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- what other parts of the framework ask ---------------------------------------
    @property
    def architectures(self) -> List[str]:
        return [ARCHITECTURE]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return NO_POSITION_LIMIT

    def _decay_rank(self, i: int) -> int:
        r = self.layers[i]["mixer"].get("decay_rank")
        if r is None:
            raise ConfigError(f"layers[{i}].mixer.decay_rank is not known: it is the first dimension of "
                              f"l{i}.mix.a1 (load the configuration together with its weights)")
        return int(r)

    # ---- the architecture as parts ----------------------------------
    def build_spec(self) -> ModelSpec:
        W, eps, n = self.width, self.norm_eps, len(self.layers)
        blocks = []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer["mixer"]
            position = None
            if layer["type"] == "latent_attention":
                mixer = PartSpec(
                    kind="latent_attention",
                    params={"hidden_size": W, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                            "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]),
                            "norm_eps": eps, "window": None},
                    weights={"q": f"{p}.mix.q", "dkv": f"{p}.mix.dkv", "dkv_norm": f"{p}.mix.dkv.norm",
                             "uk": f"{p}.mix.uk", "uv": f"{p}.mix.uv", "sink": f"{p}.mix.sink", "o": f"{p}.mix.o"})
                position = PartSpec(kind="rotary", params={
                    "head_dim": m["rot_dim"], "rotary_dim": m["rot"]["dims"], "theta": float(m["rot"]["base"]),
                    "max_positions": NO_POSITION_LIMIT, "scaling": None, "pairing": "interleaved"})
            else:
                mixer = PartSpec(
                    kind="gated_linear_attention",
                    params={"hidden_size": W, "num_heads": m["heads"], "dim": m["dim"], "value_dim": m["vdim"],
                            "tau": float(m["tau"]), "decay_rank": self._decay_rank(i), "norm_eps": eps},
                    weights={r: f"{p}.mix.{r}" for r in ("q", "k", "v", "g", "o", "norm", "a1", "a2")}
                    | {"a2_bias": f"{p}.mix.a2.b"})
            mlp = layer.get("mlp")
            ff = None
            if mlp is not None:
                E = mlp["router"]["experts"]
                names = {"table": f"{p}.mlp.table"}
                for e in range(E):
                    for r in ("gate", "up", "down"):
                        names[f"{r}.{e}"] = f"{p}.mlp.e{e}.{r}"
                shared = None
                if mlp.get("shared"):
                    shared = {"intermediate_size": mlp["shared"]["ff"]}
                    names.update({f"shared.{r}": f"{p}.mlp.shared.{r}" for r in ("gate", "up", "down")})
                ff = PartSpec(kind="experts",
                              params={"hidden_size": W, "n_experts": E, "top": mlp["router"]["top"],
                                      "expert_size": mlp["expert"]["ff"], "shared": shared,
                                      "router": {"kind": "table", "vocab_size": self.vocab}},
                              weights=names)
            blocks.append(BlockSpec(
                kind="parallel", mixer=mixer, feed_forward=ff,
                mixer_norm=PartSpec(kind="rmsnorm_scalar", params={"size": W, "eps": eps},
                                    weights={"weight": f"{p}.norm1"}),
                feed_forward_norm=None, position=position,
                params={"depth_average": {"index": i, "layers": n}},
                weights={"depth_weights": f"{p}.dwa"}))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, max_positions=NO_POSITION_LIMIT,
            embedding=PartSpec(kind="embedding", params={"vocab_size": self.vocab, "hidden_size": W},
                               weights={"weight": "embed"}),
            blocks=blocks, schedule=default_schedule(n),
            final_norm=PartSpec(kind="rmsnorm_scalar", params={"size": W, "eps": eps},
                                weights={"weight": "final.norm"}),
            head=PartSpec(kind="linear_head", params={"vocab_size": self.vocab, "hidden_size": W,
                                                      "scale": self.logit_scale},
                          weights={"weight": "head"}),
            stop_token_ids=list(self.eos_token_ids))
        spec.validate()
        return spec

    def tensor_shapes(self) -> Dict[str, List[int]]:
        W = self.width
        shapes: Dict[str, List[int]] = {"embed": [self.vocab, W], "final.norm": [], "head": [self.vocab, W]}
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer["mixer"]
            shapes[f"{p}.norm1"] = []
            H = m["heads"]
            if layer["type"] == "latent_attention":
                shapes[f"{p}.mix.q"] = [H * (m["dim"] + m["rot_dim"]), W]
                shapes[f"{p}.mix.dkv"] = [m["kv_rank"] + m["rot_dim"], W]
                shapes[f"{p}.mix.dkv.norm"] = [m["kv_rank"]]
                shapes[f"{p}.mix.uk"] = [H * m["dim"], m["kv_rank"]]
                shapes[f"{p}.mix.uv"] = [H * m["vdim"], m["kv_rank"]]
                shapes[f"{p}.mix.sink"] = [H]
                shapes[f"{p}.mix.o"] = [W, H * m["vdim"]]
            else:
                r = self._decay_rank(i)
                shapes[f"{p}.mix.q"] = [H * m["dim"], W]
                shapes[f"{p}.mix.k"] = [H * m["dim"], W]
                shapes[f"{p}.mix.v"] = [H * m["vdim"], W]
                shapes[f"{p}.mix.g"] = [H * m["vdim"], W]
                shapes[f"{p}.mix.o"] = [W, H * m["vdim"]]
                shapes[f"{p}.mix.norm"] = [m["vdim"]]
                shapes[f"{p}.mix.a1"] = [r, W]
                shapes[f"{p}.mix.a2"] = [H * m["dim"], r]
                shapes[f"{p}.mix.a2.b"] = [H * m["dim"]]
            mlp = layer.get("mlp")
            if mlp is not None:
                ff = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    shapes[f"{p}.mlp.e{e}.gate"] = [ff, W]
                    shapes[f"{p}.mlp.e{e}.up"] = [ff, W]
                    shapes[f"{p}.mlp.e{e}.down"] = [W, ff]
                shapes[f"{p}.mlp.table"] = [self.vocab, mlp["router"]["top"]]
                if mlp.get("shared"):
                    sf = mlp["shared"]["ff"]
                    shapes[f"{p}.mlp.shared.gate"] = [sf, W]
                    shapes[f"{p}.mlp.shared.up"] = [sf, W]
                    shapes[f"{p}.mlp.shared.down"] = [W, sf]
            shapes[f"{p}.dwa"] = [i + 2]
        return shapes

    def integer_tensor(self, name: str) -> bool:
        """Tensors that are integer tables, not parameters in floating point."""
        return name.endswith(".mlp.table")

    def is_norm_tensor(self, name: str) -> bool:
        return name.endswith(".norm") or name.endswith(".norm1")

    def special_random_tensor(self, name: str, seed: int, device, std: float) -> Optional[torch.Tensor]:
        """Random values for the tensors that are neither matrices nor norm weights: expert tables
        (rows of distinct experts), layer-mixing weights (about 1 / terms, so that the stream keeps its
        size), sinks and decay biases (of order one)."""
        from ..weights.random_fill import fnv1a64
        shape = self.tensor_shapes()[name]
        g = torch.Generator().manual_seed((seed * 0x9E3779B1 + fnv1a64(name)) % (1 << 62))
        if name.endswith(".mlp.table"):
            i = int(name.split(".")[0][1:])
            E = self.layers[i]["mlp"]["router"]["experts"]
            t = torch.rand(shape[0], E, generator=g).argsort(dim=1)[:, : shape[1]].to(torch.int32)
        elif name.endswith(".dwa"):
            t = ((1.0 + 0.5 * torch.randn(shape, generator=g)) / shape[0]).to(torch.bfloat16)
        elif name.endswith(".sink"):
            t = torch.randn(shape, generator=g).to(torch.bfloat16)
        elif name.endswith(".a2.b"):
            t = (1.0 + torch.randn(shape, generator=g)).to(torch.bfloat16)
        else:
            return None
        return t.contiguous().to(device)

    def parameter_count(self) -> int:
        total = 0
        for shape in self.tensor_shapes().values():
            n = 1
            for s in shape:
                n *= s
            total += n
        return total
