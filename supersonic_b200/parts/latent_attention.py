"""The latent-attention mixer: causal softmax attention that caches one low-rank row per token.

In equations, for a token at position p with normed input h, per head g of H:

    u_g = Wq_g h                       split as u_g = [a_g (dim) | b_g (rot_dim)]
    y   = Wdkv h                       split as y   = [y_lat (kv_rank) | y_rot (rot_dim)]
    c   = rms(y_lat) * w_norm          the latent row of the token
    r   = rot_p(y_rot),  b'_g = rot_p(b_g)      rotation by the position encoding the mixer is given
    K_g(j) = [Wuk_g c_j | r_j],   V_g(j) = Wuv_g c_j          for every earlier or equal position j
    s_gj = ([a_g | b'_g] . K_g(j)) * scale
    out_g = sum_j exp(s_gj) V_g(j) / (sum_j exp(s_gj) + exp(sink_g))       (without a sink: the plain softmax)
    result = Wo [out_1 ... out_H]

The cache holds [c_j | r_j] per token, whatever H is.  K and V are never formed: since
a_g . (Wuk_g c_j) = (Wuk_g^T a_g) . c_j, the query is moved into the latent space once
(a'_g = Wuk_g^T a_g), the score is a'_g . c_j + b'_g . r_j, the probabilities weight the c_j
themselves, and Wuv_g is applied to that one sum per query.  A cached token then costs a head
2 kv_rank + rot_dim multiply-adds and no matrix product.
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
