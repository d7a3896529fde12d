"""Petanex put together from parts.

A Petanex model is a list of pre-norm blocks with plain-weight RMS norms whose branch results are scaled column by
column before they join the 32-bit residual (`parts.ScaledBlock`), each followed by a per-token side input
(`parts.TokenSide`, when the file has one).  The mixer of a layer is
* attention over a cached latent without positions (`parts.LatentAttention`), or
* a gated delta rule with one decay per head and a silu gate, or with a decay per head and key channel and a sigmoid
  gate, both of those from factored projections (`parts.GatedDeltaMixer`),
and its feed-forward is a gated one with the tanh form of GELU (`parts.GatedFfn`), a mixture of experts with a shared
expert (`parts.RoutedExperts`), or absent.  The embedding is scaled by a constant of the file; the output is a norm and
the embedding table itself.  Tensor names are those of a Petanex safetensors file: `embed`, `side.embed`,
`l<i>.norm1|norm2|ls1|ls2`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.side.*`, `final.norm`.
"""
from __future__ import annotations

import torch

from ..config.petanex import CHANNEL_DELTA, DEFAULT_RANK, LATENT, PetanexConfig
from ..parts import (DecoderModel, Embedding, GatedDeltaMixer, GatedFfn, LatentAttention, LmHead, RmsNorm, RoutedExperts,
                     ScaledBlock, ShortConv, TokenSide)
from ..weights.store import TensorSpec, WeightStore

NORM_STD = 0.1
MATRIX_STD = 0.02
CONV_STD = 0.3


def _ranks(m) -> tuple:
    """(decay rank, gate rank) of a channel_delta mixer: the file's keys or the stored tensors' shapes
    (`PetanexConfig.with_shapes`), else a default (random weights)."""
    return (m.decay_rank if m.decay_rank is not None else DEFAULT_RANK, m.gate_rank if m.gate_rank is not None else DEFAULT_RANK)


def _expert_specs(p: str, ff: int, W: int) -> list[TensorSpec]:
    return [TensorSpec(p + "gate", (ff, W), MATRIX_STD), TensorSpec(p + "up", (ff, W), MATRIX_STD),
            TensorSpec(p + "down", (W, ff), MATRIX_STD)]


def _layer_specs(cfg: PetanexConfig, i: int) -> list[TensorSpec]:
    l, W, p = cfg.layers[i], cfg.width, f"l{i}."
    m = l.mixer
    out = [TensorSpec(p + "norm1", (W,), 1.0, "norm"), TensorSpec(p + "ls1", (W,), 1.0, "norm")]
    if l.type == LATENT:
        out += [TensorSpec(p + "mix.q", (m.heads * m.dim, W), MATRIX_STD), TensorSpec(p + "mix.dkv", (m.kv_rank, W), MATRIX_STD),
                TensorSpec(p + "mix.dkv.norm", (m.kv_rank,), 1.0, "norm"),
                TensorSpec(p + "mix.uk", (m.heads * m.dim, m.kv_rank), MATRIX_STD),
                TensorSpec(p + "mix.uv", (m.heads * m.vdim, m.kv_rank), MATRIX_STD),
                TensorSpec(p + "mix.o", (W, m.heads * m.vdim), MATRIX_STD)]
    else:
        for name, rows in (("q", m.kv_heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.heads * m.vdim)):
            out += [TensorSpec(f"{p}mix.{name}", (rows, W), MATRIX_STD), TensorSpec(f"{p}mix.{name}.conv", (rows, m.conv), CONV_STD, "norm")]
        out += [TensorSpec(p + "mix.b", (m.heads, W), MATRIX_STD), TensorSpec(p + "mix.A_log", (m.heads,), 0.5, "norm"),
                TensorSpec(p + "mix.norm", (m.vdim,), 1.0, "norm"), TensorSpec(p + "mix.o", (W, m.heads * m.vdim), MATRIX_STD)]
        if l.type == CHANNEL_DELTA:
            ra, rg = _ranks(m)
            out += [TensorSpec(p + "mix.a1", (ra, W), MATRIX_STD), TensorSpec(p + "mix.a2", (m.heads * m.dim, ra), MATRIX_STD),
                    TensorSpec(p + "mix.dt_bias", (m.heads * m.dim,), 0.5, "norm"),
                    TensorSpec(p + "mix.g1", (rg, W), MATRIX_STD), TensorSpec(p + "mix.g2", (m.heads * m.vdim, rg), MATRIX_STD)]
        else:
            out += [TensorSpec(p + "mix.a", (m.heads, W), MATRIX_STD), TensorSpec(p + "mix.dt_bias", (m.heads,), 0.5, "norm"),
                    TensorSpec(p + "mix.g", (m.heads * m.vdim, W), MATRIX_STD)]
    f = l.mlp
    if f is not None:
        out += [TensorSpec(p + "norm2", (W,), 1.0, "norm"), TensorSpec(p + "ls2", (W,), 1.0, "norm")]
        if f.kind == "dense":
            out += _expert_specs(p + "mlp.", f.ff, W)
        else:
            for e in range(f.experts):
                out += _expert_specs(f"{p}mlp.e{e}.", f.expert.ff, W)
            out += [TensorSpec(p + "mlp.router", (f.experts, W), MATRIX_STD), TensorSpec(p + "mlp.correction", (f.experts,), 0.1, "norm")]
            if f.shared is not None:
                out += _expert_specs(p + "mlp.shared.", f.shared.ff, W)
    if cfg.side_dim:
        out += [TensorSpec(p + "side.gate", (cfg.side_dim, W), MATRIX_STD), TensorSpec(p + "side.proj", (W, cfg.side_dim), MATRIX_STD),
                TensorSpec(p + "side.norm", (W,), 1.0, "norm")]
    return out


def tensor_specs(cfg: PetanexConfig) -> list[TensorSpec]:
    """Every tensor a Petanex file holds for `cfg`, with the spread random weights are drawn with."""
    specs = [TensorSpec("embed", (cfg.vocab, cfg.width), MATRIX_STD)]
    if cfg.side_dim:
        specs.append(TensorSpec("side.embed", (cfg.vocab, len(cfg.layers) * cfg.side_dim), 1.0))
    for i in range(len(cfg.layers)):
        specs += _layer_specs(cfg, i)
    specs.append(TensorSpec("final.norm", (cfg.width,), 1.0, "norm"))
    return specs


def _stack(parts: list[torch.Tensor], dim: int = 0) -> torch.Tensor:
    if any(p.numel() == 0 for p in parts) or len({p.dtype for p in parts}) != 1:
        return torch.empty(0)                       # a fault already recorded by the store
    return torch.cat(parts, dim=dim).contiguous()


def _gated(w: WeightStore, p: str, ff: int, W: int) -> tuple:
    gu = _stack([w.take(p + "gate", (ff, W)), w.take(p + "up", (ff, W))])
    w.release(p + "gate", p + "up")
    return gu, w.take(p + "down", (W, ff))


def _mixer(cfg: PetanexConfig, w: WeightStore, i: int):
    l, W, p = cfg.layers[i], cfg.width, f"l{i}."
    m = l.mixer
    if l.type == LATENT:
        return LatentAttention(w.take(p + "mix.q", (m.heads * m.dim, W)), w.take(p + "mix.dkv", (m.kv_rank, W)),
                               w.take(p + "mix.dkv.norm", (m.kv_rank,)), w.take(p + "mix.uk", (m.heads * m.dim, m.kv_rank)),
                               w.take(p + "mix.uv", (m.heads * m.vdim, m.kv_rank)), w.take(p + "mix.o", (W, m.heads * m.vdim)),
                               n_heads=m.heads, dim=m.dim, vdim=m.vdim, rank=m.kv_rank, scale=m.scale, norm_eps=cfg.norm_eps)
    rows = (("q", m.kv_heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.heads * m.vdim))
    mats = [w.take(f"{p}mix.{n}", (r, W)) for n, r in rows] + [w.take(p + "mix.b", (m.heads, W))]
    conv_w = _stack([w.take(f"{p}mix.{n}.conv", (r, m.conv)) for n, r in rows])
    names = [f"{p}mix.{n}" for n, _ in rows] + [p + "mix.b"]
    a2 = g2 = None
    if l.type == CHANNEL_DELTA:
        ra, rg = _ranks(m)
        mats += [w.take(p + "mix.a1", (ra, W)), w.take(p + "mix.g1", (rg, W))]
        names += [p + "mix.a1", p + "mix.g1"]
        a2, g2 = w.take(p + "mix.a2", (m.heads * m.dim, ra)), w.take(p + "mix.g2", (m.heads * m.vdim, rg))
        dt_bias = w.take(p + "mix.dt_bias", (m.heads * m.dim,))
    else:
        mats += [w.take(p + "mix.a", (m.heads, W)), w.take(p + "mix.g", (m.heads * m.vdim, W))]
        names += [p + "mix.a", p + "mix.g"]
        dt_bias = w.take(p + "mix.dt_bias", (m.heads,))
    w_in = _stack(mats)                                             # [q | k | v | b | a | g] rows
    w.release(*names)
    a_log, norm = w.take(p + "mix.A_log", (m.heads,)), w.take(p + "mix.norm", (m.vdim,))
    wo = w.take(p + "mix.o", (W, m.heads * m.vdim))
    if w.faulty:
        w.finish()
    return GatedDeltaMixer(w_in, wo, ShortConv(conv_w, None, "silu"), dt_bias, a_log, norm, heads=m.heads, kv_heads=m.kv_heads,
                           dim=m.dim, vdim=m.vdim, norm_eps=cfg.norm_eps, w_a2=a2, w_g2=g2,
                           gate="sigmoid" if l.type == CHANNEL_DELTA else "silu")


def _feed_forward(cfg: PetanexConfig, w: WeightStore, i: int):
    f, W, p = cfg.layers[i].mlp, cfg.width, f"l{i}.mlp."
    if f.kind == "dense":
        gu, down = _gated(w, p, f.ff, W)
        if w.faulty:
            w.finish()
        return GatedFfn(gu, down, "gelu_tanh")
    gus, downs = [], []
    for e in range(f.experts):
        gu, down = _gated(w, f"{p}e{e}.", f.expert.ff, W)
        gus.append(gu)
        downs.append(down)
    if w.faulty:
        w.finish()
    w_gate_up, w_down = torch.stack(gus).contiguous(), torch.stack(downs).contiguous()
    w.release(*[f"{p}e{e}.down" for e in range(f.experts)])
    shared = None
    if f.shared is not None:
        gu, down = _gated(w, p + "shared.", f.shared.ff, W)
        if w.faulty:
            w.finish()
        shared = GatedFfn(gu, down, "clamped_swish", limit=f.shared.limit)
    router, correction = w.take(p + "router", (f.experts, W)), w.take(p + "correction", (f.experts,))
    if w.faulty:
        w.finish()
    return RoutedExperts(router, correction, w_gate_up, w_down, top=f.top, scale=f.scale, limit=f.expert.limit,
                         groups=f.groups, keep=f.keep, shared=shared)


def build(cfg: PetanexConfig, w: WeightStore) -> DecoderModel:
    cfg = cfg.with_shapes(w.shape_of)
    W, L = cfg.width, len(cfg.layers)
    table = w.take("embed", (cfg.vocab, W))
    side_table = w.take("side.embed", (cfg.vocab, L * cfg.side_dim)) if cfg.side_dim else None
    if w.faulty:
        w.finish()
    blocks = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        mixer = _mixer(cfg, w, i)
        norm1, ls1 = RmsNorm(w.take(p + "norm1", (W,)), cfg.norm_eps), w.take(p + "ls1", (W,))
        ffn = norm2 = ls2 = None
        if l.mlp is not None:
            ffn = _feed_forward(cfg, w, i)
            norm2, ls2 = RmsNorm(w.take(p + "norm2", (W,)), cfg.norm_eps), w.take(p + "ls2", (W,))
        side = None
        if cfg.side_dim:
            side = TokenSide(side_table, i * cfg.side_dim, cfg.side_dim, w.take(p + "side.gate", (cfg.side_dim, W)),
                             w.take(p + "side.proj", (W, cfg.side_dim)), RmsNorm(w.take(p + "side.norm", (W,)), cfg.norm_eps))
        if w.faulty:
            w.finish()
        blocks.append(ScaledBlock(norm1, mixer, ls1, norm2, ffn, ls2, side))
    final_norm = RmsNorm(w.take("final.norm", (W,)), cfg.norm_eps)
    w.finish()
    return DecoderModel(Embedding(table, scale=cfg.embedding_scale), blocks, LmHead(final_norm, table), name=cfg.architecture)
