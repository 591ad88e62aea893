"""Stream adapters: parts that act on the residual stream between two stops of the schedule.

A stop names one with ``ScheduleEntry.before = (adapter, pass)``; the model calls
``adapter(ctx, x, pass_no)`` before the stop's block and goes on with the tensor it returns.

``loop_input``: the entry of a pass over a run of layers that is walked several times with the same
weights: x <- W_in [x ; x0] + step[pass], where x0 is what the embedding gave (``ctx.embedded``) and
``step`` has a row per pass.
"""
from __future__ import annotations

import torch

from .registry import BuildContext, register_stream_adapter


@register_stream_adapter("loop_input")
class LoopInput:
    """params: ``hidden_size``, ``passes``; weights: ``in`` [hidden, 2 x hidden] (the stream's columns first),
    ``step`` [passes, hidden]."""

    needs_embedding = True

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.passes = int(params["hidden_size"]), int(params["passes"])
        self.w_in = build.weights.as_dtype(weights["in"], build.dtype)
        self.step = build.weights.stored(weights["step"]).float().contiguous()
        if tuple(self.w_in.shape) != (self.hidden, 2 * self.hidden) or tuple(self.step.shape) != (self.passes, self.hidden):
            raise ValueError(f"{weights['in']} / {weights['step']} have shapes {tuple(self.w_in.shape)} / "
                             f"{tuple(self.step.shape)}, expected {(self.hidden, 2 * self.hidden)} / "
                             f"{(self.passes, self.hidden)}")
        self.dtype = build.dtype

    @staticmethod
    def activation_elements(params) -> int:
        return 4 * int(params["hidden_size"])

    def __call__(self, ctx, x, pass_no: int):
        if not 0 <= pass_no < self.passes:
            raise ValueError(f"pass {pass_no} of {self.passes}")
        if ctx.embedded is None:
            raise RuntimeError("loop_input needs the embedding's output of the step")
        T = x.shape[0]
        both = torch.empty((T, 2 * self.hidden), dtype=self.dtype, device=x.device)
        out = torch.empty((T, self.hidden), dtype=torch.float32, device=x.device)
        ctx.kernels.concat_cast(x, ctx.embedded, both, self.step[pass_no], out)
        ctx.kernels.linear(both, self.w_in, out, accumulate=True)
        return out
