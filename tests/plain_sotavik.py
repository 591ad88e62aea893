"""A plain, slow statement of the Sotavik design, one function per mechanism, for the tests.

Everything is float64 torch on the CPU, token by token where the design is recurrent, with no
cache, no batching and no code shared with the engine.  ``cfg`` is the configuration as a
dictionary (the keys of config.json), ``w`` maps tensor names to tensors.

Notation: x is the stream entering a layer, h its normed copy, X_j the raw results of the
layers (X_0 the embedding), T the number of tokens.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """One gain for all coordinates."""
    return rms(x, eps) * g.to(F)


def silu(z):
    return z * torch.sigmoid(z)


def rotate_interleaved(v, pos, base, dims):
    """Pairs (2i, 2i+1) of the first ``dims`` coordinates of ``v`` [T, ..., d] turned by pos * base^(-2i/dims)."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=F)
    ang = pos.to(F)[:, None] * base ** (-2.0 * i / dims)          # [T, dims/2]
    while ang.dim() < v.dim():
        ang = ang.unsqueeze(1)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * torch.cos(ang) - b * torch.sin(ang)
    out[..., 1:dims:2] = b * torch.cos(ang) + a * torch.sin(ang)
    return out


def latent_attention(h, w, p, m, eps, pos=None, window=None, use_sink=True):
    """h [T, width]; ``p`` the tensor prefix ('l0.mix'), ``m`` the mixer's sizes.  ``window``: a query
    sees the last ``window`` keys only (its own included)."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if pos is None else pos
    q = (h @ w[p + ".q"].to(F).T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    low = h @ w[p + ".dkv"].to(F).T
    c = rms(low[:, :rank], eps) * w[p + ".dkv.norm"].to(F)
    k_rot = low[:, rank:]
    rot = m["rot"]
    q_rot = rotate_interleaved(q_rot, pos, float(rot["base"]), int(rot["dims"]))
    k_rot = rotate_interleaved(k_rot, pos, float(rot["base"]), int(rot["dims"]))
    k_plain = (c @ w[p + ".uk"].to(F).T).view(T, H, d)
    v = (c @ w[p + ".uv"].to(F).T).view(T, H, dv)
    sink = w[p + ".sink"].to(F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        for hd in range(H):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (k_plain[lo: t + 1, hd] @ q_plain[t, hd] + k_rot[lo: t + 1] @ q_rot[t, hd]) * m["scale"]
            sk = float(sink[hd]) if use_sink else -math.inf
            top = max(float(s.max()), sk)
            e = torch.exp(s - top)
            out[t, hd] = (e[:, None] * v[lo: t + 1, hd]).sum(0) / (e.sum() + math.exp(sk - top))
    return out.reshape(T, H * dv) @ w[p + ".o"].to(F).T


def gated_linear_attention(h, w, p, m, eps, state=None):
    """Returns (output [T, width], final state [H, d, dv])."""
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w[p + ".q"].to(F).T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + ".k"].to(F).T).view(T, H, d)
    v = (h @ w[p + ".v"].to(F).T).view(T, H, dv)
    z = (h @ w[p + ".a1"].to(F).T) @ w[p + ".a2"].to(F).T + w[p + ".a2.b"].to(F)
    decay = torch.sigmoid(z).pow(1.0 / tau).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * w[p + ".norm"].to(F)
    gate = silu(h @ w[p + ".g"].to(F).T)
    return (o.reshape(T, H * dv) * gate) @ w[p + ".o"].to(F).T, S


def gated_unit(h, w, p):
    return (silu(h @ w[p + ".gate"].to(F).T) * (h @ w[p + ".up"].to(F).T)) @ w[p + ".down"].to(F).T


def table_experts(h, tokens, w, p, mlp):
    """Every token's experts come from a table indexed by its id, equal weights."""
    top = int(mlp["router"]["top"])
    table = w[p + ".table"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist()[:top]:
            out[t] += gated_unit(h[t:t + 1], w, f"{p}.e{int(e)}")[0] / top
    if mlp.get("shared"):
        out = out + gated_unit(h, w, p + ".shared")
    return out


def forward(cfg, w, tokens, keep_layers=False):
    """Logits [T, vocab] of one sequence from its first token on (and the stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"].to(F)[tokens]
    results, layers = [x], []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = scalar_norm(x, w[p + ".norm1"], eps)
        if layer["type"] == "latent_attention":
            mixed = latent_attention(h, w, p + ".mix", layer["mixer"], eps)
        elif layer["type"] == "gla":
            mixed, _ = gated_linear_attention(h, w, p + ".mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        ff = table_experts(h, tokens, w, p + ".mlp", layer["mlp"]) if layer.get("mlp") else 0.0
        results.append(x + (mixed + ff))
        mix = w[p + ".dwa"].to(F)
        x = sum(mix[j] * results[j] for j in range(i + 2))
        layers.append(x)
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].to(F).T * float(cfg["logit_scale"])
    return (logits, torch.stack(layers)) if keep_layers else logits
