"""The latent-attention mixer: softmax attention whose keys and values are carried by one
low-rank row per token.

With h the normed input: q = Wq h, head by head [dim plain | rot_dim rotated]; Wdkv h gives
kv_rank + rot_dim numbers: the first kv_rank, RMS-normed with a weight, are the latent c, the
last rot_dim, rotated by the token's position, are a key part k_r that all heads share.  Head
g's key is [Wuk_g c | k_r] and its value Wuv_g c; the score of query t on key j is
(q_plain . Wuk_g c_j + q_rot . k_r,j) * scale, causal, and the softmax may carry a sink: one
more term exp(sink_g) in the denominator that has no key and no value.

Only [c | k_r] is cached (one row per token, whatever the number of heads), and the keys and
values are never formed: q_plain is carried into the latent space once per query,
q' = Wuk_g^T q_plain, so that the score is q' . c_j + q_rot . k_r,j; the weighted sum of the
c_j is taken in the latent space and Wuv_g is applied to that sum.  Per cached token a head
then costs kv_rank + rot_dim multiply-adds for the score and kv_rank for the value, with no
per-token matrix product.
"""
from __future__ import annotations

import torch

from ..cache import PAGE_SHIFT, KvNeed
from .registry import BuildContext, register_mixer


@register_mixer("latent_attention")
class LatentAttention:
    """params: ``hidden_size``, ``num_heads``, ``dim``, ``rot_dim``, ``value_dim``, ``kv_rank``, ``scale``,
    ``norm_eps``, ``window`` (None = all earlier keys); weights: ``q``, ``dkv``, ``dkv_norm``, ``uk``, ``uv``,
    ``o`` and optionally ``sink``.  The position encoding it is given rotates the ``rot_dim`` parts."""

    takes_lazy_input = True

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.H = int(params["hidden_size"]), int(params["num_heads"])
        self.dim, self.rot, self.vdim = int(params["dim"]), int(params["rot_dim"]), int(params["value_dim"])
        self.rank = int(params["kv_rank"])
        self.scale, self.eps = float(params["scale"]), float(params["norm_eps"])
        self.window = params.get("window")
        w, dt = build.weights, build.dtype
        H, d, r, dv, rank = self.H, self.dim, self.rot, self.vdim, self.rank
        want = {"q": (H * (d + r), self.hidden), "dkv": (rank + r, self.hidden), "dkv_norm": (rank,),
                "uk": (H * d, rank), "uv": (H * dv, rank), "o": (self.hidden, H * dv)}
        got = {role: w.as_dtype(weights[role], dt) for role in ("q", "dkv", "uk", "uv", "o")}
        norm_w = w.stored(weights["dkv_norm"])
        got["dkv_norm"] = norm_w.float() if dt == torch.float32 else norm_w
        for role, shape in want.items():
            if tuple(got[role].shape) != shape:
                raise ValueError(f"{weights[role]} has shape {tuple(got[role].shape)}, expected {shape}")
        self.w_in = torch.cat([got["q"], got["dkv"]], dim=0).contiguous()      # one product for q and the low-rank row
        self.w_q = self.w_in[: H * (d + r)]
        self.norm_w = got["dkv_norm"]
        # Wuk_g^T [rank, dim] per head carries a plain query into the latent space; Wuv_g [vdim, rank] carries
        # the summed latent out of it
        self.w_absorb = got["uk"].view(H, d, rank).transpose(1, 2).contiguous()
        self.w_uv = got["uv"].view(H, dv, rank).contiguous()
        self.w_o = got["o"]
        self.sinks = None
        if weights.get("sink"):
            self.sinks = w.stored(weights["sink"]).float().contiguous()
            if tuple(self.sinks.shape) != (H,):
                raise ValueError(f"{weights['sink']} has shape {tuple(self.sinks.shape)}, expected ({H},)")
        self.dtype = dt

    def cache_need(self):
        return KvNeed(1, self.rank + self.rot, self.window, value_dim=0)

    @staticmethod
    def cache_need_from(params):
        return KvNeed(1, int(params["kv_rank"]) + int(params["rot_dim"]), params.get("window"), value_dim=0)

    @staticmethod
    def activation_elements(params) -> int:
        """Elements per token while the part runs: the projected row, the latent-space queries, the summed
        latents and the heads' outputs."""
        H, rank, r = int(params["num_heads"]), int(params["kv_rank"]), int(params["rot_dim"])
        return H * (int(params["dim"]) + r) + rank + r + H * (2 * rank + r) + H * int(params["value_dim"])

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        if position is None or not hasattr(position, "rotary_tables"):
            raise ValueError("latent attention needs a rotary position encoding for its rotated parts")
        H, d, r, dv, rank = self.H, self.dim, self.rot, self.vdim, self.rank
        T, dev = ctx.batch.n_tokens, residual.device
        cache, _, table, _ = ctx.cache.kv(cache_id)
        q_cols = H * (d + r)
        proj = torch.empty((T, q_cols + (rank + r if writes_cache else 0)), dtype=self.dtype, device=dev)
        ctx.kernels.linear(x, self.w_in if writes_cache else self.w_q, proj)
        position.check_range(ctx.batch)
        q_abs = torch.empty((T, H * (rank + r)), dtype=self.dtype, device=dev)
        ctx.kernels.latent_prepare(proj, q_cols, q_abs, self.norm_w, self.eps, position, ctx.batch, table, cache,
                                   H, d, r, rank, PAGE_SHIFT, writes_cache)
        ctx.kernels.head_linear(proj[:, :q_cols].view(T, H, d + r)[:, :, :d], self.w_absorb,
                                q_abs.view(T, H, rank + r)[:, :, :rank])
        latent = torch.empty((T, H * rank), dtype=self.dtype, device=dev)
        ctx.kernels.latent_attention(q_abs, cache, ctx.batch, table, latent, H, rank, r, PAGE_SHIFT, self.window,
                                     self.scale, self.sinks)
        heads = torch.empty((T, H * dv), dtype=self.dtype, device=dev)
        ctx.kernels.head_linear(latent.view(T, H, rank), self.w_uv, heads.view(T, H, dv))
        ctx.kernels.linear(heads, self.w_o, residual, accumulate=True)
