"""Attention with sigmoid weights inside chunks: grouped-query attention whose weights are not normalised.

For a token at position p with normed input h, query head g of H and its kv head g // (H / G):

    q_g = rot_p(rms(Wq_g h) * wq),   k = rot_p(rms(Wk h) * wk),   v = Wv h          (wq, wk [dim], one for all heads)
    a_gj = sigmoid((q_g . k_j) * scale + bias_g)       for the visible keys j
    out_g = sum_j a_gj v_j,      result = Wo [out_1 ... out_H]

Key j is visible to position p if j <= p and both lie in the same chunk of ``chunk`` positions, chunks counted
from the sequence's position 0 (so what a query sees does not depend on how a prompt was cut into steps); a
``window`` bounds it further.  Keys have ``dim`` coordinates, values ``value_dim``; the position encoding turns
the first coordinates of q and k.  Scores and weights are float32.
"""
from __future__ import annotations

import torch

from ..cache import PAGE_SHIFT, KvNeed
from .registry import BuildContext, register_mixer


@register_mixer("sigmoid_attention")
class SigmoidAttention:
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``dim``, ``value_dim``, ``scale``, ``chunk`` (None:
    no chunks), ``window`` (None), ``qk_norm`` (default True), ``norm_eps``; weights: ``q``, ``k``, ``v``, ``o`` and
    optionally ``q_norm``, ``k_norm`` [dim], ``bias`` [heads]."""

    def __init__(self, params, weights, build: BuildContext):
        self.hidden = int(params["hidden_size"])
        self.n_q, self.n_kv = int(params["num_heads"]), int(params["num_kv_heads"])
        self.dim, self.vdim = int(params["dim"]), int(params["value_dim"])
        self.scale, self.eps = float(params["scale"]), float(params.get("norm_eps", 1e-6))
        self.chunk, self.window = params.get("chunk"), params.get("window")
        if self.n_q % self.n_kv:
            raise ValueError(f"{self.n_q} query heads do not split over {self.n_kv} kv heads")
        if self.chunk is not None and int(self.chunk) < 1:
            raise ValueError("sigmoid_attention: a chunk holds at least one position")
        w, dt = build.weights, build.dtype
        q, k, v = (w.as_dtype(weights[r], dt) for r in ("q", "k", "v"))
        self.w_o = w.as_dtype(weights["o"], dt)
        want = {"q": (self.n_q * self.dim, self.hidden), "k": (self.n_kv * self.dim, self.hidden),
                "v": (self.n_kv * self.vdim, self.hidden), "o": (self.hidden, self.n_q * self.vdim)}
        for r, t in (("q", q), ("k", k), ("v", v), ("o", self.w_o)):
            if tuple(t.shape) != want[r]:
                raise ValueError(f"{weights[r]} has shape {tuple(t.shape)}, expected {want[r]}")
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.n_q * self.dim]
        self.q_norm = self.k_norm = self.bias = None
        if params.get("qk_norm", True):
            self.q_norm = w.stored(weights["q_norm"]).float().contiguous()
            self.k_norm = w.stored(weights["k_norm"]).float().contiguous()
            if tuple(self.q_norm.shape) != (self.dim,) or tuple(self.k_norm.shape) != (self.dim,):
                raise ValueError(f"{weights['q_norm']} / {weights['k_norm']}: expected ({self.dim},)")
        if weights.get("bias"):
            self.bias = w.stored(weights["bias"]).float().contiguous()
            if tuple(self.bias.shape) != (self.n_q,):
                raise ValueError(f"{weights['bias']} has shape {tuple(self.bias.shape)}, expected ({self.n_q},)")
        self.dtype = dt

    @staticmethod
    def _reach(params):
        """How far back a query can look: what the cache must keep.  A chunk never reaches further back than
        its own length, so pages behind it can be given back like those behind a window."""
        reach = [int(x) for x in (params.get("chunk"), params.get("window")) if x]
        return min(reach) if reach else None

    def cache_need(self):
        return KvNeed(self.n_kv, self.dim, self._reach({"chunk": self.chunk, "window": self.window}), value_dim=self.vdim)

    @staticmethod
    def cache_need_from(params):
        return KvNeed(int(params["num_kv_heads"]), int(params["dim"]), SigmoidAttention._reach(params),
                      value_dim=int(params["value_dim"]))

    @staticmethod
    def activation_elements(params) -> int:
        H, G = int(params["num_heads"]), int(params["num_kv_heads"])
        return (H + G) * int(params["dim"]) + (H + G) * int(params["value_dim"])

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        T, dev, k = ctx.batch.n_tokens, residual.device, ctx.kernels
        kv = ctx.cache.kv(cache_id)
        width = self.n_q * self.dim + (self.n_kv * (self.dim + self.vdim) if writes_cache else 0)
        qkv = torch.empty((T, width), dtype=self.dtype, device=dev)
        k.linear(x, self.w_qkv if writes_cache else self.w_q, qkv)
        k.qk_norm_rope_append(qkv, self.q_norm, self.k_norm, self.eps, position, kv, ctx.batch, self.n_q, self.n_kv,
                              self.dim, self.vdim, PAGE_SHIFT, writes_cache)
        k_cache, v_cache, table, _ = kv
        heads = torch.empty((T, self.n_q * self.vdim), dtype=self.dtype, device=dev)
        k.sigmoid_attention(qkv, k_cache, v_cache, ctx.batch, table, self.bias, heads, self.n_q, self.n_kv, self.dim,
                            self.vdim, PAGE_SHIFT, self.chunk, self.window, self.scale)
        k.linear(heads, self.w_o, residual, accumulate=True)
