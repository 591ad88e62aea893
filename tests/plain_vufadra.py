"""A plain, slow statement of the Vufadra design in float64 on the CPU: one function per mechanism, one
sequence at a time, every recurrence a Python loop over its tokens.  It shares no code with the library:
the tests compare the library's kernels, cache and step function against it.

``weights`` maps tensor names to tensors, ``config`` is the dictionary of a config.json.  Every function
takes a whole sequence ``[T, ...]`` and starts from empty state; ``forward`` returns the logits of every
position and the stream after every layer run.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def _w(weights, name):
    return weights[name].to(F)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + z.clamp(min=0)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dynamic_tanh(x, weights, name):
    return torch.tanh(_w(weights, name + ".alpha") * x) * _w(weights, name) + _w(weights, name + ".b")


def shifted(h, mu):
    """h_t + (h_(t-1) - h_t) * mu with h_(-1) = 0."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]])
    return h + (before - h) * mu


def embedding(tokens, weights, config):
    big = config["embedding"]["bigram"]
    n, a, b = int(big["buckets"]), int(big["mul_prev"]), int(big["mul_cur"])
    rows = [n if t == 0 else (int(tokens[t - 1]) * a + int(tokens[t]) * b) % n for t in range(len(tokens))]
    return _w(weights, "embed")[torch.as_tensor(tokens)] + _w(weights, "bigram")[torch.as_tensor(rows)]


# ---- mixers ---------------------------------------------------------------------------------------
def real_gated_recurrence(h, weights, p, m):
    """The ``rglru`` mixer."""
    T = h.shape[0]
    C, taps, nb = int(m["width"]), int(m["conv"]), int(m["blocks"])
    y = gelu_tanh(h @ _w(weights, p + ".y").T + _w(weights, p + ".y.b"))
    xb = h @ _w(weights, p + ".x").T + _w(weights, p + ".x.b")
    conv, conv_b = _w(weights, p + ".conv"), _w(weights, p + ".conv.b")
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), xb])
    u = conv_b.expand(T, C).clone()
    for j in range(taps):                       # the last column multiplies the current token
        u = u + padded[j:j + T] * conv[:, j]
    ub = u.view(T, nb, C // nb)
    r = sigmoid(torch.einsum("boi,tbi->tbo", _w(weights, p + ".ra"), ub) + _w(weights, p + ".ra.b")).reshape(T, C)
    i = sigmoid(torch.einsum("boi,tbi->tbo", _w(weights, p + ".ri"), ub) + _w(weights, p + ".ri.b")).reshape(T, C)
    a = torch.exp(-8.0 * r * softplus(_w(weights, p + ".lam")))
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(C, dtype=F)
    out = torch.empty(T, C, dtype=F)
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return (out * y) @ _w(weights, p + ".o").T


def _head_norm(o, eps):
    return o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)


def generalized_delta(h, weights, p, m, eps):
    """The ``general_delta`` mixer."""
    T, H, d = h.shape[0], int(m["heads"]), int(m["dim"])
    r = (h @ _w(weights, p + ".r").T).view(T, H, d)
    k = (h @ _w(weights, p + ".k").T).view(T, H, d)
    v = (h @ _w(weights, p + ".v").T).view(T, H, d)
    z = torch.tanh(h @ _w(weights, p + ".w1").T) @ _w(weights, p + ".w2").T + _w(weights, p + ".w0")
    w = torch.exp(-math.exp(-0.5) * sigmoid(z)).view(T, H, d)
    a = sigmoid(h @ _w(weights, p + ".a").T + _w(weights, p + ".a.b")).view(T, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=F)            # [head, key channel, value channel]
    o = torch.empty(T, H, d, dtype=F)
    for t in range(T):
        seen = torch.einsum("hk,hkv->hv", u[t], S)
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * seen[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, r[t])
    o = _head_norm(o, eps).reshape(T, H * d) * _w(weights, p + ".norm")
    o = o * sigmoid(h @ _w(weights, p + ".g").T)
    return o @ _w(weights, p + ".o").T


def rotary_angles(T, rot):
    """cos and sin [T, dims/2] with the YaRN change of the frequencies."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    gain = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def at(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(at(float(sc["fast"]))), 0)
        hi = min(math.ceil(at(float(sc["slow"]))), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        gain = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(T, dtype=F)[:, None] * torch.tensor(f, dtype=F)[None, :]
    return torch.cos(ang) * gain, torch.sin(ang) * gain


def rotate(x, cos, sin):
    """x [T, heads, dim]: the first 2 * cos.shape[1] coordinates turn, i with i + half."""
    half = cos.shape[1]
    a, b, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def chunked_sigmoid_attention(h, weights, p, m, eps):
    """The left half of the ``parallel`` mixer."""
    T, H, G, d, dv = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ _w(weights, p + ".q").T).view(T, H, d)
    k = (h @ _w(weights, p + ".k").T).view(T, G, d)
    v = (h @ _w(weights, p + ".v").T).view(T, G, dv)
    q = unit_rms(q, eps) * _w(weights, p + ".q.norm")
    k = unit_rms(k, eps) * _w(weights, p + ".k.norm")
    cos, sin = rotary_angles(T, m["rot"])
    q, k = rotate(q, cos, sin), rotate(k, cos, sin)
    size = int(m["mask"]["size"])
    pos = torch.arange(T)
    visible = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    pb = _w(weights, p + ".pb")
    out = torch.empty(T, H, dv, dtype=F)
    for g in range(H):
        kv = g // (H // G)
        score = (q[:, g] @ k[:, kv].T) * float(m["scale"]) + pb[g]
        weight = torch.where(visible, sigmoid(score), torch.zeros((), dtype=F))
        out[:, g] = weight @ v[:, kv]
    return out.reshape(T, H * dv) @ _w(weights, p + ".o").T


def time_mixing(h, weights, p, m, eps):
    """The right half of the ``parallel`` mixer."""
    T, H, d = h.shape[0], int(m["heads"]), int(m["dim"])
    mix = {s: shifted(h, _w(weights, f"{p}.mu.{s}")) for s in "rkvgw"}
    r = (mix["r"] @ _w(weights, p + ".r").T).view(T, H, d)
    k = (mix["k"] @ _w(weights, p + ".k").T).view(T, H, d)
    v = (mix["v"] @ _w(weights, p + ".v").T).view(T, H, d)
    gate = silu(mix["g"] @ _w(weights, p + ".g").T)
    z = torch.tanh(mix["w"] @ _w(weights, p + ".w1").T) @ _w(weights, p + ".w2").T + _w(weights, p + ".w0")
    w = torch.exp(-torch.exp(z)).view(T, H, d)
    bonus = _w(weights, p + ".u")                # [heads, dim]
    S = torch.zeros(H, d, d, dtype=F)
    o = torch.empty(T, H, d, dtype=F)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S + bonus[:, :, None] * kv, r[t])
        S = w[t][:, :, None] * S + kv
    o = _head_norm(o, eps).reshape(T, H * d) * _w(weights, p + ".norm") * gate
    return o @ _w(weights, p + ".o").T


def side_by_side(h, weights, p, m, eps):
    """The ``parallel`` mixer: half the sum of its two halves, each normed over the width first."""
    left = chunked_sigmoid_attention(h, weights, p + ".left", m["left"], eps)
    right = time_mixing(h, weights, p + ".right", m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * _w(weights, p + ".left.out") + unit_rms(right, eps) * _w(weights, p + ".right.out"))


def dense_feed_forward(h, weights, p):
    return (silu(h @ _w(weights, p + ".gate").T) * (h @ _w(weights, p + ".up").T)) @ _w(weights, p + ".down").T


def layer(x, i, weights, config):
    spec, eps = config["layers"][i], float(config["norm"]["eps"])
    p = f"l{i}"
    h = shifted(dynamic_tanh(x, weights, p + ".norm1"), _w(weights, p + ".shift"))
    kind, m = spec["type"], spec["mixer"]
    if kind == "rglru":
        mixed = real_gated_recurrence(h, weights, p + ".mix", m)
    elif kind == "general_delta":
        mixed = generalized_delta(h, weights, p + ".mix", m, eps)
    elif kind == "parallel":
        mixed = side_by_side(h, weights, p + ".mix", m, eps)
    else:
        raise ValueError(kind)
    if spec.get("mlp") is not None:
        mixed = mixed + dense_feed_forward(dynamic_tanh(x, weights, p + ".norm2"), weights, p + ".mlp")
    return x + mixed


def forward(tokens, weights, config):
    """Logits [T, vocab] and the stream after every layer run [runs, T, width] of one sequence."""
    x0 = embedding(list(tokens), weights, config)
    x, runs = x0, []
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 0}
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(start)] if times else []
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    order += [(i, None) for i in range(stop if times else 0, n)]
    for i, enters in order:
        if enters is not None:
            x = torch.cat([x, x0], dim=-1) @ _w(weights, "loop.in").T + _w(weights, "loop.step")[enters]
        x = layer(x, i, weights, config)
        runs.append(x)
    logits = dynamic_tanh(x, weights, "final.norm") @ _w(weights, "head").T
    return logits, torch.stack(runs)
