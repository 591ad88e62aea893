"""Gated linear attention: a mixer whose memory is a matrix per head instead of a list of keys.

In equations, for token t with normed input h, per head g (key width dim, value width vdim):

    q = (Wq_g h) / sqrt(dim),   k = Wk_g h,   v = Wv_g h
    z = Wa2 (Wa1 h) + b                          a low-rank projection, one number per head and key channel
    a = sigmoid(z) ** (1 / tau)                  decay in (0, 1) per key channel
    S_t = diag(a) S_(t-1) + k v^T                S_0 = 0, shape [dim, vdim]
    o = S_t^T q
    y_g = rms(o) * w_norm * silu(Wg_g h)         w_norm [vdim] is the same vector for every head
    result = Wo [y_1 ... y_H]

S is the sequence's state: it lives in the cache's fixed-size float32 rows and is carried from
step to step.  z, the decays, the state and o are float32 whatever the activation type; the
matrix products run in the activation type.
"""
from __future__ import annotations

import torch

from ..cache import StateNeed
from .registry import BuildContext, register_mixer


@register_mixer("gated_linear_attention")
class GatedLinearAttention:
    """params: ``hidden_size``, ``num_heads``, ``dim``, ``value_dim``, ``tau``, ``decay_rank``, ``norm_eps``;
    weights: ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``, ``a1``, ``a2``, ``a2_bias``."""

    takes_lazy_input = True

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.H = int(params["hidden_size"]), int(params["num_heads"])
        self.dim, self.vdim, self.rank = int(params["dim"]), int(params["value_dim"]), int(params["decay_rank"])
        self.tau, self.eps = float(params["tau"]), float(params["norm_eps"])
        from ..csrc.ops import SCAN_MAX_DIM
        if self.dim > SCAN_MAX_DIM:
            raise ValueError(f"gated linear attention: {self.dim} key channels a head; the recurrence kernel holds up "
                             f"to {SCAN_MAX_DIM}")
        w, dt = build.weights, build.dtype
        H, d, dv, r = self.H, self.dim, self.vdim, self.rank
        want = {"q": (H * d, self.hidden), "k": (H * d, self.hidden), "v": (H * dv, self.hidden),
                "g": (H * dv, self.hidden), "a1": (r, self.hidden), "a2": (H * d, r), "o": (self.hidden, H * dv)}
        got = {role: w.as_dtype(weights[role], dt) for role in want}
        for role, shape in want.items():
            if tuple(got[role].shape) != shape:
                raise ValueError(f"{weights[role]} has shape {tuple(got[role].shape)}, expected {shape}")
        # one product for everything that reads h: [q | k | v | g | a1]
        self.w_in = torch.cat([got[r_] for r_ in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.q_off, self.k_off, self.v_off = 0, H * d, 2 * H * d
        self.g_off, self.a_off = 2 * H * d + H * dv, 2 * H * d + 2 * H * dv
        self.w_a2, self.w_o = got["a2"], got["o"]
        self.z_bias = w.stored(weights["a2_bias"]).float().contiguous()
        norm_w = w.stored(weights["norm"])
        self.norm_w = norm_w.float() if dt == torch.float32 else norm_w
        if tuple(self.z_bias.shape) != (H * d,) or tuple(self.norm_w.shape) != (dv,):
            raise ValueError(f"{weights['a2_bias']} / {weights['norm']}: expected ({H * d},) and ({dv},)")
        self.dtype = dt

    def cache_need(self):
        return StateNeed(self.H * self.dim * self.vdim)

    @staticmethod
    def cache_need_from(params):
        return StateNeed(int(params["num_heads"]) * int(params["dim"]) * int(params["value_dim"]))

    @staticmethod
    def activation_elements(params) -> int:
        """Elements per token while the part runs: the projected row, z and o (float32: counted twice),
        and the gated output."""
        H, d, dv = int(params["num_heads"]), int(params["dim"]), int(params["value_dim"])
        return 2 * H * d + 2 * H * dv + int(params["decay_rank"]) + 2 * H * d + 3 * H * dv

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        if not writes_cache:
            raise ValueError("a recurrent mixer cannot read another layer's state without advancing it")
        H, d, dv = self.H, self.dim, self.vdim
        T, dev = ctx.batch.n_tokens, residual.device
        proj = torch.empty((T, self.w_in.shape[0]), dtype=self.dtype, device=dev)
        ctx.kernels.linear(x, self.w_in, proj)
        z = torch.empty((T, H * d), dtype=torch.float32, device=dev)
        ctx.kernels.linear(proj[:, self.a_off:], self.w_a2, z)
        o = torch.empty((T, H * dv), dtype=torch.float32, device=dev)
        ctx.kernels.gated_linear_scan(proj, self.q_off, self.k_off, self.v_off, z, self.z_bias, self.tau,
                                      d ** -0.5, ctx.cache.state(cache_id), ctx.batch, o, H, d, dv)
        y = torch.empty((T, H * dv), dtype=self.dtype, device=dev)
        ctx.kernels.head_norm_gate(o, self.norm_w, self.eps, proj[:, self.g_off:], y, H, dv)
        ctx.kernels.linear(y, self.w_o, residual, accumulate=True)
