"""Block arrangements.  ``pre_norm``: h += mixer(norm(h)); h += feed_forward(norm(h)),
the residual stream kept and summed in float32 (crates/runner/src/prefill_engine.rs:1116-1222).
``parallel``: h += mixer(n) + feed_forward(n) with the one n = norm(h), optionally followed by a
learned weighted sum over the results of all layers so far."""
from __future__ import annotations

import torch

from ..csrc.kernel_sets import NormedInput
from .registry import register_block


@register_block("pre_norm")
class PreNormBlock:
    """Interface of a block: ``forward(ctx, residual, cache_id, writes_cache)`` updates the
    float32 residual stream ``[T, hidden]`` in place."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, position):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.position = position

    @staticmethod
    def _give(x, part):
        """Parts that set ``takes_lazy_input`` get the norm unapplied (a NormedInput) so that
        their kernels may fold it in; all others get the normed activations."""
        return x if getattr(part, "takes_lazy_input", False) else x.tensor()

    def forward(self, ctx, residual, cache_id, writes_cache):
        x = NormedInput(ctx, residual, self.mixer_norm)
        ctx.stage = "mixer"           # names the running part for stage timings; nothing depends on it
        self.mixer.forward(ctx, self._give(x, self.mixer), residual, cache_id, writes_cache, self.position)
        if self.feed_forward is None:
            return
        x2 = NormedInput(ctx, residual, self.feed_forward_norm)
        ctx.stage = "feed_forward"
        self.feed_forward.forward(ctx, self._give(x2, self.feed_forward), residual)


@register_block("parallel")
class ParallelBlock:
    """x <- x + mixer(n) + feed_forward(n), n = norm(x): one norm, read by both sublayers (the
    feed-forward may be absent).

    ``params["depth_average"] = {"index": i, "layers": L}`` adds a weighted sum over depth.  Call R_0 what the
    embedding gives and R_(n+1) = s_n + mixer(norm(s_n)) + feed_forward(norm(s_n)) the raw result of layer n,
    where s_n is the stream that enters it; then s_(i+1) = sum_{j = 0 .. i+1} a_i[j] R_j with layer i's own
    i + 2 numbers a_i (``depth_weights``).  The R_j of a step are planes of one float32 stack ``ctx.streams``
    [L + 2, T, width]: plane i + 1 holds s_i, the sublayers add into it in place (which makes it R_(i+1)), and
    the weighted sum is written into plane i + 2, which the block returns as the stream from then on.
    """

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, position, params=None,
                 weights=None, build=None):
        if feed_forward_norm is not None:
            raise ValueError("a parallel block has one norm")
        self.mixer, self.feed_forward, self.mixer_norm, self.position = mixer, feed_forward, mixer_norm, position
        self.depth = (params or {}).get("depth_average")
        if self.depth is not None:
            self.index, self.layers = int(self.depth["index"]), int(self.depth["layers"])
            w = build.weights.stored(weights["depth_weights"]).float().contiguous()
            if tuple(w.shape) != (self.index + 2,):
                raise ValueError(f"{weights['depth_weights']} has shape {tuple(w.shape)}, expected ({self.index + 2},)")
            self.depth_weights = w
            self.one = torch.ones(1, dtype=torch.float32, device=build.device)

    _give = staticmethod(PreNormBlock._give)

    def forward(self, ctx, residual, cache_id, writes_cache):
        if self.depth is not None:
            if self.index == 0:
                T, width = residual.shape
                ctx.streams = torch.empty((self.layers + 2, T, width), dtype=torch.float32, device=residual.device)
                ctx.kernels.stream_mix(residual.unsqueeze(0), self.one, 1, ctx.streams[0])
                ctx.kernels.stream_mix(residual.unsqueeze(0), self.one, 1, ctx.streams[1])
            elif ctx.streams is None:
                raise RuntimeError("a depth-averaging layer ran before the first one of its step")
            residual = ctx.streams[self.index + 1]
        x = NormedInput(ctx, residual, self.mixer_norm)
        ctx.stage = "mixer"
        self.mixer.forward(ctx, self._give(x, self.mixer), residual, cache_id, writes_cache, self.position)
        if self.feed_forward is not None:
            ctx.stage = "feed_forward"
            self.feed_forward.forward(ctx, self._give(x, self.feed_forward), residual)
        if self.depth is None:
            return None
        out = ctx.streams[self.index + 2]
        ctx.kernels.stream_mix(ctx.streams, self.depth_weights, self.index + 2, out)
        return out
