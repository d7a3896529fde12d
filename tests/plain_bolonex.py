"""A plain, slow Bolonex: whole sequences in float64, no cache, no batch, one function per mechanism.

Written from the design's equations and sharing no code with the package: the tests compare the engine
(pages, state slots, portions, mixed batches, kernels) with what these functions give for the whole sequence.
`cfg` is the dictionary a config.json holds; `t` maps tensor names to tensors.

Notation: T tokens, width W.  A layer is x <- x + mixer(h) + ff(h) with h = norm1(x), one norm for both branches.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w.to(DT))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def short_conv(u, w, bias=None):
    """Causal convolution per channel: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start.
    u [T, C], w [C, taps]; the last column multiplies the current token."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=DT), u], 0)
    y = torch.zeros(T, C, dtype=DT)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j].to(DT)[None, :]
    if bias is not None:
        y = y + bias.to(DT)[None, :]
    return y


def rotary_frequencies(rot):
    """f_i = base^(-2i/dims), i < dims/2, then the long-context rescaling when `scaling` is given: wavelengths below
    original/high keep f, above original/low use f/factor, and between the two a straight blend in original/wavelength."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=DT)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = sc["factor"], sc["low"], sc["high"], sc["original"]
        out = []
        for fi in f.tolist():
            wl = 2.0 * math.pi / fi
            if wl < orig / high:
                out.append(fi)
            elif wl > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wl - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=DT)
    return f


def rotate_interleaved(x, rot, first_position=0):
    """x [T, heads, dim]: dimensions 2i and 2i+1 (i < dims/2) turn by position * f_i; the rest pass."""
    T = x.shape[0]
    dims = rot["dims"]
    f = rotary_frequencies(rot)
    ang = (torch.arange(T, dtype=DT) + first_position)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def attention_mixer(h, m, t, p, eps):
    """m: the mixer's sizes and constants; t: tensors; p: the layer's tensor prefix ('l0.')."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def proj(name):
        return h @ t[p + "mix." + name].to(DT).T + t[p + "mix." + name + ".b"].to(DT)[None, :]

    q, k, v = proj("q"), proj("k"), proj("v")
    q = short_conv(q, t[p + "mix.q.conv"])
    k = short_conv(k, t[p + "mix.k.conv"])
    v = short_conv(v, t[p + "mix.v.conv"])
    q = rms(q.view(T, H, d), eps) * t[p + "mix.q.norm"].to(DT)
    k = rms(k.view(T, G, d), eps) * t[p + "mix.k.norm"].to(DT)
    v = v.view(T, G, dv)
    if m.get("rot"):
        q, k = rotate_interleaved(q, m["rot"]), rotate_interleaved(k, m["rot"])
    gate = torch.sigmoid(h @ t[p + "mix.g"].to(DT).T)                 # [T, H]
    seen = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.empty(T, H, dv, dtype=DT)
    cap = m.get("softcap")
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        w = torch.softmax(s.masked_fill(~seen, float("-inf")), -1)
        out[:, head] = (w @ v[:, g]) * gate[:, head:head + 1]
    return out.reshape(T, H * dv) @ t[p + "mix.o"].to(DT).T


def mamba2_mixer(h, m, t, p, eps):
    T = h.shape[0]
    nh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = nh * P
    zxbcdt = h @ t[p + "mix.in"].to(DT).T
    z = zxbcdt[:, :inner]
    xbc = zxbcdt[:, inner:2 * inner + 2 * G * N]
    dt = zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, t[p + "mix.conv"], t[p + "mix.conv.b"]))
    x = xbc[:, :inner].reshape(T, nh, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + t[p + "mix.dt_bias"].to(DT)[None, :])          # [T, nh]
    A = -torch.exp(t[p + "mix.A_log"].to(DT))
    D = t[p + "mix.D"].to(DT)
    y = torch.empty(T, nh, P, dtype=DT)
    for head in range(nh):
        g = head // (nh // G)
        S = torch.zeros(N, P, dtype=DT)
        for i in range(T):
            S = torch.exp(A[head] * dt[i, head]) * S + dt[i, head] * torch.outer(B[i, g], x[i, head])
            y[i, head] = S.T @ C[i, g] + D[head] * x[i, head]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * t[p + "mix.norm"].to(DT)
    return y @ t[p + "mix.o"].to(DT).T


def dense_ff(h, t, p):
    return gelu_tanh(h @ t[p + "mlp.up"].to(DT).T) @ t[p + "mlp.down"].to(DT).T


MIXERS = {"attention": attention_mixer, "mamba2": mamba2_mixer}


def forward(cfg, t, tokens, return_layers=False):
    """Logits [T, vocab] (float64) of one whole sequence; with `return_layers` also the residual stream after every
    layer run [runs, T, width]."""
    eps = cfg["norm"]["eps"]
    x = t["embed"].to(DT)[torch.tensor(list(tokens))] * cfg["embedding"]["scale"]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i) if layer.get('weights_of') is not None else i}."
        h = norm_one_plus(x, t[p + "norm1"], eps)
        branch = MIXERS[layer["type"]](h, layer["mixer"], t, p, eps)
        if layer.get("mlp"):
            branch = branch + dense_ff(h, t, p)
        x = x + branch
        streams.append(x)
    logits = norm_one_plus(x, t["final.norm"], eps) @ t["head"].to(DT).T
    return (logits, torch.stack(streams)) if return_layers else logits
