"""A plain, slow Petanex: whole sequences in float64, no cache, no batch, one function per mechanism.

Written from the design's equations and sharing no code with the package: the tests compare the engine
(pages, state slots, portions, mixed batches, kernels) with what these functions give for the whole sequence.
`cfg` is the dictionary a config.json holds; `t` maps tensor names to tensors.

Notation: T tokens, width W.  A layer is
    x <- x + ls1 * mixer(norm1(x));  x <- x + ls2 * ff(norm2(x));  x <- x + side(x, token)
with plain-weight RMS norms; the mixer is latent attention (no positions), a gated delta rule with one decay per head,
or one with a decay per head and key channel; the feed-forward is dense and gated, or a routed mixture with a shared expert.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms(x, eps) * w.to(DT)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def lin(x, w):
    return x @ w.to(DT).T


def short_conv(u, w):
    """y_t[c] = sum_j w[c, j] u_(t - taps + 1 + j)[c]; zeros before the start; the last column is the current token's."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=DT), u], 0)
    y = torch.zeros(T, C, dtype=DT)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j].to(DT)[None, :]
    return y


def latent_attention(h, m, t, p, eps):
    """Causal softmax attention whose keys and values are both expansions of one small latent row per token."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = lin(h, t[p + "q"]).view(T, H, d)
    c = norm(lin(h, t[p + "dkv"]), t[p + "dkv.norm"], eps)
    k = lin(c, t[p + "uk"]).view(T, H, d)
    v = lin(c, t[p + "uv"]).view(T, H, dv)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    s = s.masked_fill(~mask[None], float("-inf"))
    w = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhv->ihv", w, v).reshape(T, H * dv)
    return lin(o, t[p + "o"])


def unit(x):
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, decay, state=None, return_state=False):
    """q, k [T, H, d] (already per value head), v [T, H, dv], beta [T, H], decay [T, H, d] (rows of S by key channel).
    S <- decay * S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=DT) if state is None else state.clone()
    out = torch.zeros(T, H, dv, dtype=DT)
    for i in range(T):
        S = S * decay[i][:, :, None]
        u = beta[i][:, None] * (v[i] - torch.einsum("hdv,hd->hv", S, k[i]))
        S = S + k[i][:, :, None] * u[:, None, :]
        out[i] = torch.einsum("hdv,hd->hv", S, q[i])
    return (out, S) if return_state else out


def delta_mixer(h, m, t, p, eps, per_channel):
    T = h.shape[0]
    H, KH, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(lin(h, t[p + "q"]), t[p + "q.conv"].to(DT))).view(T, KH, d)
    k = silu(short_conv(lin(h, t[p + "k"]), t[p + "k.conv"].to(DT))).view(T, KH, d)
    v = silu(short_conv(lin(h, t[p + "v"]), t[p + "v.conv"].to(DT))).view(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    rep = H // KH
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = sigmoid(lin(h, t[p + "b"]))
    rate = torch.exp(t[p + "A_log"].to(DT))
    if per_channel:
        a = lin(lin(h, t[p + "a1"]), t[p + "a2"]) + t[p + "dt_bias"].to(DT)
        decay = torch.exp(-rate[None, :, None] * softplus(a).view(T, H, d))
        gate = sigmoid(lin(lin(h, t[p + "g1"]), t[p + "g2"]))
    else:
        a = lin(h, t[p + "a"]) + t[p + "dt_bias"].to(DT)
        decay = torch.exp(-rate[None, :] * softplus(a))[:, :, None].expand(T, H, d)
        gate = silu(lin(h, t[p + "g"]))
    o = delta_rule(q, k, v, beta, decay)
    o = rms(o, eps) * t[p + "norm"].to(DT)[None, None, :]
    o = o.reshape(T, H * dv) * gate
    return lin(o, t[p + "o"])


def dense_ff(h, t, p):
    return lin(gelu_tanh(lin(h, t[p + "gate"])) * lin(h, t[p + "up"]), t[p + "down"])


def expert(h, t, p, limit):
    g = torch.clamp(lin(h, t[p + "gate"]), max=limit)
    u = torch.clamp(lin(h, t[p + "up"]), min=-limit, max=limit)
    return lin(g * sigmoid(1.702 * g) * (u + 1.0), t[p + "down"])


def route(h, f, t, p):
    """Chosen experts [T, top] and their weights [T, top]."""
    r = f["router"]
    E, top = r["experts"], r["top"]
    s = sigmoid(lin(h, t[p + "router"]))
    choice = s + t[p + "correction"].to(DT)[None, :]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    G, keep = groups["count"], groups["keep"]
    if G > 1:
        per = E // G
        grouped = choice.view(-1, G, per)
        score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
        best = score.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(-1, G, per).reshape(-1, E), float("-inf"))
    ids = choice.topk(top, dim=-1).indices
    w = s.gather(1, ids)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return ids, w


def moe_ff(h, f, t, p):
    ids, w = route(h, f, t, p)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=DT)
    for i in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[i, j])
            out[i] += w[i, j] * expert(h[i:i + 1], t, f"{p}e{e}.", f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + expert(h, t, p + "shared.", f["shared"]["limit"])
    return out


def token_side(x, tokens, i, cfg, t, eps):
    dim = cfg["token_side"]["dim"]
    p = f"l{i}.side."
    e = t["side.embed"].to(DT)[tokens][:, i * dim:(i + 1) * dim]
    y = lin(gelu_tanh(lin(x, t[p + "gate"])) * e, t[p + "proj"])
    return norm(y, t[p + "norm"], eps)


def forward(cfg, t, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; `layers_out`, a list, receives the residual after every layer."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = t["embed"].to(DT)[tokens] * cfg["embedding"]["scale"]
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm(x, t[p + "norm1"], eps)
        if l["type"] == "latent_attention":
            a = latent_attention(h, l["mixer"], t, p + "mix.", eps)
        else:
            a = delta_mixer(h, l["mixer"], t, p + "mix.", eps, per_channel=l["type"] == "channel_delta")
        x = x + a * t[p + "ls1"].to(DT)
        f = l.get("mlp")
        if f:
            h = norm(x, t[p + "norm2"], eps)
            y = dense_ff(h, t, p + "mlp.") if f["kind"] == "dense" else moe_ff(h, f, t, p + "mlp.")
            x = x + y * t[p + "ls2"].to(DT)
        if cfg.get("token_side"):
            x = x + token_side(x, tokens, i, cfg, t, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(norm(x, t["final.norm"], eps), t["embed"])


def greedy(cfg, t, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(cfg, t, seq)[-1].argmax()))
    return seq[len(prompt):]
