"""Typed configuration of the ``Vufadra`` architecture.

Its config.json is nested.  Top level: ``vocab``, ``width``, ``norm.eps``, ``embedding.bigram`` (``buckets``,
``mul_prev``, ``mul_cur``), ``loop`` (``start``, ``stop``, ``times``; absent or ``times`` 0: no loop) and ``layers``,
a list with one entry per layer: ``type`` (``rglru``, ``general_delta`` or ``parallel``), ``mixer`` (that mixer's
sizes and constants) and ``mlp`` (null, or ``{"kind": "dense", "ff"}``).  ``build_spec`` turns that into parts: a
pair embedding; per layer a ``parallel`` block with two ``dynamic_tanh`` norms and token shift around one of the
mixers ``real_gated_recurrence``, ``delta_rule`` or ``mixer_pair`` (``sigmoid_attention`` beside ``time_mixing``) and a
``swiglu`` feed-forward; a schedule that walks layers ``start .. stop - 1`` ``times`` times, every pass with cache
entries of its own and entered through the ``loop_input`` adapter; a ``dynamic_tanh`` norm and a linear head.

Tensor names: ``embed``, ``bigram``, ``loop.in``, ``loop.step``, ``final.norm`` (+ ``.alpha``, ``.b``), ``head`` and per
layer i ``l<i>.norm1``, ``l<i>.norm2`` (+ ``.alpha``, ``.b``), ``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.*``.

One size is not in config.json: the inner width of a decay's two-step projection, which is the first dimension
of its ``w1`` tensor (``with_shapes`` reads it from the stored tensor; a configuration made by hand may give it
as ``decay_rank`` in the mixer's entry).  The design has no position limit; the cache bounds a sequence.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from .base import BlockSpec, ConfigError, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Vufadra"
MIXERS = ("rglru", "general_delta", "parallel")
NO_POSITION_LIMIT = 1 << 20


def _need(d, keys, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"{where} is missing {missing}")


def _positive(d, keys, where: str) -> None:
    for k in keys:
        if not (isinstance(d[k], int) and not isinstance(d[k], bool) and d[k] > 0):
            raise ConfigError(f"{where}.{k} must be a positive integer, got {d[k]!r}")


@dataclass(frozen=True)
class VufadraConfig:
    vocab: int
    width: int
    norm_eps: float
    bigram: Dict[str, int]
    loop: Optional[Dict[str, int]]
    layers: List[Dict[str, Any]] = field(default_factory=list)
    eos_token_ids: List[int] = field(default_factory=list)
    model_type: str = "vufadra"

    # ---- reading -----------------------------------------------------
    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "VufadraConfig":
        _need(d, ("vocab", "width", "layers", "norm", "embedding"), "config.json")
        _need(d["norm"], ("eps",), "norm")
        _need(d["embedding"], ("bigram",), "embedding")
        _need(d["embedding"]["bigram"], ("buckets", "mul_prev", "mul_cur"), "embedding.bigram")
        loop = d.get("loop")
        if loop is not None:
            _need(loop, ("start", "stop", "times"), "loop")
            loop = {k: int(loop[k]) for k in ("start", "stop", "times")}
        eos = d.get("eos_token_id")
        cfg = VufadraConfig(
            vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
            bigram={k: int(d["embedding"]["bigram"][k]) for k in ("buckets", "mul_prev", "mul_cur")},
            loop=loop, layers=copy.deepcopy(list(d["layers"])),
            eos_token_ids=[] if eos is None else [int(eos)] if isinstance(eos, int) else [int(e) for e in eos])
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.bigram["buckets"] < 1 or self.bigram["mul_prev"] < 0 or self.bigram["mul_cur"] < 0:
            raise ConfigError("embedding.bigram: at least one bucket, multipliers not negative")
        if not self.layers:
            raise ConfigError("layers must name at least one layer")
        n = len(self.layers)
        if self.loop is not None and self.loop["times"] > 0:
            if not 0 <= self.loop["start"] < self.loop["stop"] <= n:
                raise ConfigError(f"loop: layers {self.loop['start']} .. {self.loop['stop']} - 1 of {n}")
        elif self.loop is not None and self.loop["times"] < 0:
            raise ConfigError("loop.times must not be negative")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            m = layer["mixer"]
            if layer["type"] == "rglru":
                _need(m, ("width", "conv", "blocks"), where + ".mixer")
                _positive(m, ("width", "conv", "blocks"), where + ".mixer")
                if m["width"] % m["blocks"]:
                    raise ConfigError(f"{where}.mixer: {m['width']} channels do not split into {m['blocks']} blocks")
            elif layer["type"] == "general_delta":
                _need(m, ("heads", "dim"), where + ".mixer")
                _positive(m, ("heads", "dim"), where + ".mixer")
            elif layer["type"] == "parallel":
                _need(m, ("left", "right"), where + ".mixer")
                left, right = m["left"], m["right"]
                _need(left, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"), where + ".mixer.left")
                _positive(left, ("heads", "kv_heads", "dim", "vdim"), where + ".mixer.left")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{where}.mixer.left: {left['heads']} heads over {left['kv_heads']} kv heads")
                _need(left["mask"], ("size",), where + ".mixer.left.mask")
                _positive(left["mask"], ("size",), where + ".mixer.left.mask")
                _need(left["rot"], ("base", "dims"), where + ".mixer.left.rot")
                dims = left["rot"]["dims"]
                if not isinstance(dims, int) or dims < 0 or dims % 2 or dims > left["dim"]:
                    raise ConfigError(f"{where}.mixer.left.rot.dims must be even and at most dim, got {dims!r}")
                if left["rot"].get("scaling"):
                    _need(left["rot"]["scaling"], ("factor", "original", "fast", "slow"), where + ".mixer.left.rot.scaling")
                _need(right, ("heads", "dim"), where + ".mixer.right")
                _positive(right, ("heads", "dim"), where + ".mixer.right")
            else:
                raise ConfigError(f"{where}.type {layer['type']!r} is not known (known: {list(MIXERS)})")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not known (known: 'dense')")
                _need(mlp, ("ff",), where + ".mlp")
                _positive(mlp, ("ff",), where + ".mlp")
        for e in self.eos_token_ids:
            if not 0 <= e < self.vocab:
                raise ConfigError(f"eos_token_id {e} is outside the vocabulary")

    def _rank_tensors(self, i: int):
        """(where in the layer's mixer entry the rank is kept, the tensor whose first dimension it is)."""
        kind = self.layers[i]["type"]
        if kind == "general_delta":
            return [((), f"l{i}.mix.w1")]
        if kind == "parallel":
            return [(("right",), f"l{i}.mix.right.w1")]
        return []

    def with_shapes(self, store) -> "VufadraConfig":
        """The configuration with the sizes that only tensor shapes give: the decays' inner widths."""
        layers = copy.deepcopy(self.layers)
        for i, layer in enumerate(layers):
            for path, name in self._rank_tensors(i):
                m = layer["mixer"]
                for key in path:
                    m = m[key]
                if "decay_rank" not in m and name in store and len(store.shape(name)) == 2:
                    m["decay_rank"] = int(store.shape(name)[0])
        return VufadraConfig(self.vocab, self.width, self.norm_eps, dict(self.bigram),
                             None if self.loop is None else dict(self.loop), layers, list(self.eos_token_ids),
                             self.model_type)

    # ---- writing -----------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": ARCHITECTURE, "embedding": {"bigram": dict(self.bigram)},
                             "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
                             "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            d["loop"] = dict(self.loop)
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

    def _rank(self, m: Dict[str, Any], name: str) -> int:
        r = m.get("decay_rank")
        if r is None:
            raise ConfigError(f"the decay's inner width is not known: it is the first dimension of {name} "
                              "(load the configuration together with its weights, or give decay_rank)")
        return int(r)

    def layer_order(self):
        """The stops of a forward pass: (layer, pass that the stop enters or None, number of the run of the layer)."""
        n = len(self.layers)
        times = self.loop["times"] if self.loop else 0
        if times <= 0:
            return [(i, None, 0) for i in range(n)]
        start, stop = self.loop["start"], self.loop["stop"]
        order = [(i, None, 0) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None, t) for i in range(start, stop)]
        return order + [(i, None, 0) for i in range(stop, n)]

    # ---- the architecture as parts ----------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec(kind="dynamic_tanh", params={"size": self.width},
                        weights={"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})

    def _mixer(self, i: int):
        W, eps = self.width, self.norm_eps
        layer, p = self.layers[i], f"l{i}.mix"
        m = layer["mixer"]
        if layer["type"] == "rglru":
            return PartSpec(
                kind="real_gated_recurrence",
                params={"hidden_size": W, "width": m["width"], "taps": m["conv"], "blocks": m["blocks"]},
                weights={"y": f"{p}.y", "y_bias": f"{p}.y.b", "x": f"{p}.x", "x_bias": f"{p}.x.b", "conv": f"{p}.conv",
                         "conv_bias": f"{p}.conv.b", "ra": f"{p}.ra", "ra_bias": f"{p}.ra.b", "ri": f"{p}.ri",
                         "ri_bias": f"{p}.ri.b", "lam": f"{p}.lam", "o": f"{p}.o"}), None
        if layer["type"] == "general_delta":
            return PartSpec(
                kind="delta_rule",
                params={"hidden_size": W, "num_heads": m["heads"], "dim": m["dim"],
                        "decay_rank": self._rank(m, f"{p}.w1"), "norm_eps": eps},
                weights={r: f"{p}.{r}" for r in ("r", "k", "v", "g", "a", "w1", "w2", "w0", "norm", "o")}
                | {"a_bias": f"{p}.a.b"}), None
        left, right = m["left"], m["right"]
        scaling = left["rot"].get("scaling")
        position = None
        if left["rot"]["dims"] > 0:
            position = PartSpec(kind="rotary", params={
                "head_dim": left["dim"], "rotary_dim": left["rot"]["dims"], "theta": float(left["rot"]["base"]),
                "max_positions": NO_POSITION_LIMIT, "pairing": "halves",
                "scaling": None if not scaling else {"kind": "yarn", "factor": float(scaling["factor"]),
                                                     "original": float(scaling["original"]),
                                                     "fast": float(scaling["fast"]), "slow": float(scaling["slow"])}})
        lp, rp = p + ".left", p + ".right"
        halves = {
            "left": {"kind": "sigmoid_attention", "position": True,
                     "params": {"hidden_size": W, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"],
                                "dim": left["dim"], "value_dim": left["vdim"], "scale": float(left["scale"]),
                                "chunk": int(left["mask"]["size"]), "window": None, "qk_norm": True, "norm_eps": eps},
                     "weights": {"q": f"{lp}.q", "k": f"{lp}.k", "v": f"{lp}.v", "o": f"{lp}.o", "q_norm": f"{lp}.q.norm",
                                 "k_norm": f"{lp}.k.norm", "bias": f"{lp}.pb"}},
            "right": {"kind": "time_mixing", "position": False,
                      "params": {"hidden_size": W, "num_heads": right["heads"], "dim": right["dim"],
                                 "decay_rank": self._rank(right, f"{rp}.w1"), "norm_eps": eps},
                      "weights": {r: f"{rp}.{r}" for r in ("r", "k", "v", "g", "w1", "w2", "w0", "norm", "o")}
                      | {"mu_" + s: f"{rp}.mu.{s}" for s in "rkvgw"} | {"bonus": f"{rp}.u"}}}
        return PartSpec(kind="mixer_pair", params={"hidden_size": W, "norm_eps": eps, "scale": 0.5, **halves},
                        weights={"left_out": f"{p}.left.out", "right_out": f"{p}.right.out"}), position

    def build_spec(self) -> ModelSpec:
        W = self.width
        blocks = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}"
            mixer, position = self._mixer(i)
            mlp = layer.get("mlp")
            ff = None if mlp is None else PartSpec(
                kind="swiglu", params={"hidden_size": W, "intermediate_size": mlp["ff"]},
                weights={r: f"{p}.mlp.{r}" for r in ("gate", "up", "down")})
            blocks.append(BlockSpec(
                kind="parallel", mixer=mixer, feed_forward=ff, mixer_norm=self._norm(f"{p}.norm1"),
                feed_forward_norm=None if ff is None else self._norm(f"{p}.norm2"), position=position,
                params={"token_shift": {"size": W}}, weights={"shift": f"{p}.shift"}))
        order = self.layer_order()
        looped = any(enters is not None for _, enters, _ in order)
        schedule = [ScheduleEntry(layer=i, cache=c, before=None if enters is None else (0, enters))
                    for c, (i, enters, _) in enumerate(order)]
        adapters = [PartSpec(kind="loop_input", params={"hidden_size": W, "passes": self.loop["times"]},
                             weights={"in": "loop.in", "step": "loop.step"})] if looped else []
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, max_positions=NO_POSITION_LIMIT,
            embedding=PartSpec(kind="pair_embedding",
                               params={"vocab_size": self.vocab, "hidden_size": W, **self.bigram},
                               weights={"weight": "embed", "pair": "bigram"}),
            blocks=blocks, schedule=schedule, final_norm=self._norm("final.norm"),
            head=PartSpec(kind="linear_head", params={"vocab_size": self.vocab, "hidden_size": W},
                          weights={"weight": "head"}),
            stop_token_ids=list(self.eos_token_ids), adapters=adapters)
        spec.validate()
        return spec

    def tensor_shapes(self) -> Dict[str, List[int]]:
        W = self.width
        shapes: Dict[str, List[int]] = {"embed": [self.vocab, W], "bigram": [self.bigram["buckets"] + 1, W],
                                        "head": [self.vocab, W]}

        def norm(name):
            shapes[name], shapes[name + ".b"], shapes[name + ".alpha"] = [W], [W], []
        norm("final.norm")
        if self.loop is not None and self.loop["times"] > 0:
            shapes["loop.in"], shapes["loop.step"] = [W, 2 * W], [self.loop["times"], W]
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer["mixer"]
            norm(f"{p}.norm1")
            shapes[f"{p}.shift"] = [W]
            q = p + ".mix"
            if layer["type"] == "rglru":
                C, nb = m["width"], m["blocks"]
                for r in ("y", "x"):
                    shapes[f"{q}.{r}"], shapes[f"{q}.{r}.b"] = [C, W], [C]
                shapes[f"{q}.conv"], shapes[f"{q}.conv.b"] = [C, m["conv"]], [C]
                for r in ("ra", "ri"):
                    shapes[f"{q}.{r}"], shapes[f"{q}.{r}.b"] = [nb, C // nb, C // nb], [nb, C // nb]
                shapes[f"{q}.lam"], shapes[f"{q}.o"] = [C], [W, C]
            elif layer["type"] == "general_delta":
                HD, r = m["heads"] * m["dim"], self._rank(m, f"{q}.w1")
                for role in ("r", "k", "v", "g", "a"):
                    shapes[f"{q}.{role}"] = [HD, W]
                shapes[f"{q}.a.b"], shapes[f"{q}.w1"], shapes[f"{q}.w2"], shapes[f"{q}.w0"] = [HD], [r, W], [HD, r], [HD]
                shapes[f"{q}.norm"], shapes[f"{q}.o"] = [HD], [W, HD]
            else:
                left, right = m["left"], m["right"]
                lq, rq = q + ".left", q + ".right"
                shapes[f"{lq}.q"] = [left["heads"] * left["dim"], W]
                shapes[f"{lq}.k"] = [left["kv_heads"] * left["dim"], W]
                shapes[f"{lq}.v"] = [left["kv_heads"] * left["vdim"], W]
                shapes[f"{lq}.q.norm"], shapes[f"{lq}.k.norm"] = [left["dim"]], [left["dim"]]
                shapes[f"{lq}.pb"], shapes[f"{lq}.o"] = [left["heads"]], [W, left["heads"] * left["vdim"]]
                HD, r = right["heads"] * right["dim"], self._rank(right, f"{rq}.w1")
                for s in "rkvgw":
                    shapes[f"{rq}.mu.{s}"] = [W]
                for role in ("r", "k", "v", "g"):
                    shapes[f"{rq}.{role}"] = [HD, W]
                shapes[f"{rq}.w1"], shapes[f"{rq}.w2"], shapes[f"{rq}.w0"] = [r, W], [HD, r], [HD]
                shapes[f"{rq}.u"], shapes[f"{rq}.norm"], shapes[f"{rq}.o"] = [right["heads"], right["dim"]], [HD], [W, HD]
                shapes[f"{lq}.out"], shapes[f"{rq}.out"] = [W], [W]
            mlp = layer.get("mlp")
            if mlp is not None:
                norm(f"{p}.norm2")
                shapes[f"{p}.mlp.gate"], shapes[f"{p}.mlp.up"] = [mlp["ff"], W], [mlp["ff"], W]
                shapes[f"{p}.mlp.down"] = [W, mlp["ff"]]
        return shapes

    def ignorable_tensor(self, name: str) -> bool:
        """Stored tensors that this configuration never reads: the loop's, where no layer is walked more than zero times."""
        return name in ("loop.in", "loop.step") and not (self.loop is not None and self.loop["times"] > 0)

    def is_norm_tensor(self, name: str) -> bool:
        last = name.rsplit(".", 1)[-1]
        return last in ("norm", "norm1", "norm2", "out") or name.endswith((".q.norm", ".k.norm"))

    def special_random_tensor(self, name: str, seed: int, device, std: float) -> Optional[torch.Tensor]:
        """Random values for the tensors that are neither matrices nor norm weights: biases and decay offsets of
        order one, a norm's alpha near one, mixing shares between 0 and 1, decay rates that keep a state for tens
        of tokens, small bonuses and convolution taps."""
        from ..weights.random_fill import fnv1a64
        shape = self.tensor_shapes()[name]
        g = torch.Generator().manual_seed((seed * 0x9E3779B1 + fnv1a64(name)) % (1 << 62))
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            t = 0.5 + 0.5 * torch.rand(shape, generator=g)
        elif last == "shift" or ".mu." in name:
            t = torch.rand(shape, generator=g)
        elif last in ("b", "pb", "w0"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "lam":
            t = torch.randn(shape, generator=g) - 2.0
        elif last == "u" or last == "step":
            t = 0.3 * torch.randn(shape, generator=g)
        elif last == "conv":
            t = torch.randn(shape, generator=g) / max(shape[1], 1) ** 0.5
        elif last in ("ra", "ri"):
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        else:
            return None
        return t.to(torch.bfloat16).contiguous().to(device)

    def parameter_count(self) -> int:
        total = 0
        for shape in self.tensor_shapes().values():
            n = 1
            for s in shape:
                n *= s
            total += n
        return total
