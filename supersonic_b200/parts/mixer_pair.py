"""Two mixers side by side: both read the same input, and their results are joined as

    result = scale * (rms(left) * w_left + rms(right) * w_right)

with the root mean square taken over the model width (eps inside the root) and a weight vector each.
Either half is any registered mixer; each keeps what it needs in the cache under the pair's id
(``(cache_id, "left")`` and ``(cache_id, "right")``), and each gets the position encoding only if it asks for it.
"""
from __future__ import annotations

import torch

from .registry import MIXERS, BuildContext, lookup, register_mixer


@register_mixer("mixer_pair")
class MixerPair:
    """params: ``hidden_size``, ``norm_eps``, ``scale`` (default 1/2), ``left`` and ``right``: each
    ``{"kind", "params", "weights", "position": bool}``; weights: ``left_out``, ``right_out`` [hidden]."""

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.eps = int(params["hidden_size"]), float(params["norm_eps"])
        self.scale = float(params.get("scale", 0.5))
        self.halves = []
        for side in ("left", "right"):
            sub = params[side]
            self.halves.append((side, lookup(MIXERS, sub["kind"], "mixer")(sub["params"], sub["weights"], build),
                                bool(sub.get("position", False))))
        self.out_w = [build.weights.stored(weights[s + "_out"]).float().contiguous() for s in ("left", "right")]
        for s, t in zip(("left_out", "right_out"), self.out_w):
            if tuple(t.shape) != (self.hidden,):
                raise ValueError(f"{weights[s]} has shape {tuple(t.shape)}, expected ({self.hidden},)")

    def cache_need(self):
        return {side: mixer.cache_need() for side, mixer, _ in self.halves}

    @staticmethod
    def cache_need_from(params):
        needs = {}
        for side in ("left", "right"):
            hook = getattr(lookup(MIXERS, params[side]["kind"], "mixer"), "cache_need_from", None)
            needs[side] = hook(params[side]["params"]) if hook is not None else None
        return needs

    @staticmethod
    def activation_elements(params) -> int:
        total = 4 * int(params["hidden_size"])
        for side in ("left", "right"):
            hook = getattr(lookup(MIXERS, params[side]["kind"], "mixer"), "activation_elements", None)
            total += int(hook(params[side]["params"])) if hook is not None else 4 * int(params["hidden_size"])
        return total

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        x = x.tensor() if hasattr(x, "tensor") else x
        outs = []
        for side, mixer, wants_position in self.halves:
            # a half adds into what it is given: a zeroed stream of its own
            out = torch.zeros_like(residual)
            mixer.forward(ctx, x, out, (cache_id, side), writes_cache, position if wants_position else None)
            outs.append(out)
        ctx.kernels.rms_pair_add(residual, outs[0], self.out_w[0], outs[1], self.out_w[1], self.eps, self.scale)
