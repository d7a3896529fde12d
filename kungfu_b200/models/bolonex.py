"""Bolonex put together from parts.

A Bolonex model is a list of parallel blocks: one (1 + w) RMS norm whose output feeds both the mixer and the
feed-forward, whose results are added to the residual together.  The mixer of a layer is either
* attention with biased q, k, v projections, a short causal convolution on each of them, a per-head RMS norm on q and
  k, interleaved rotary positions with long-context frequency rescaling on part of each head, softcapped scores and
  one sigmoid gate per head (`parts.ConvGatedAttention`), or
* a Mamba-2 state-space mixer (`parts.Mamba2Mixer`),
and the feed-forward is dense with the tanh form of GELU (or absent).  A layer may run with another layer's tensors
(`weights_of`): it then shares that layer's part objects and gets a cache slot of its own through the model's
schedule.  The embedding is scaled by a constant of the file; the output is a (1 + w) norm and an untied matrix.
Tensor names are those of a Bolonex safetensors file: `embed`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`,
`final.norm`, `head`.
"""
from __future__ import annotations

import torch

from ..config.bolonex import ATTENTION, BolonexConfig
from ..parts import (ConvGatedAttention, DecoderModel, DenseFfn, Embedding, LayerCall, LmHead, Mamba2Mixer, ParallelBlock,
                     RmsNorm, Rope, ShortConv)
from ..weights.store import TensorSpec, WeightStore

NORM_STD = 0.1
MATRIX_STD = 0.02
CONV_STD = 0.3
BIAS_STD = 0.02


def _layer_specs(p: str, l, W: int) -> list[TensorSpec]:
    m = l.mixer
    out = [TensorSpec(p + "norm1", (W,), NORM_STD, "norm")]
    if l.type == ATTENTION:
        for name, rows in (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)):
            out += [TensorSpec(f"{p}mix.{name}", (rows, W), MATRIX_STD), TensorSpec(f"{p}mix.{name}.b", (rows,), BIAS_STD, "norm")]
        out += [TensorSpec(p + "mix.q.norm", (m.dim,), 1.0, "norm"), TensorSpec(p + "mix.k.norm", (m.dim,), 1.0, "norm")]
        for name, rows in (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)):
            out.append(TensorSpec(f"{p}mix.{name}.conv", (rows, m.conv), CONV_STD, "norm"))
        out += [TensorSpec(p + "mix.g", (m.heads, W), MATRIX_STD), TensorSpec(p + "mix.o", (W, m.heads * m.vdim), MATRIX_STD)]
    else:
        out += [TensorSpec(p + "mix.in", (m.proj_width, W), MATRIX_STD),
                TensorSpec(p + "mix.conv", (m.conv_width, m.conv), CONV_STD, "norm"),
                TensorSpec(p + "mix.conv.b", (m.conv_width,), BIAS_STD, "norm"),
                TensorSpec(p + "mix.dt_bias", (m.heads,), 0.5, "norm"), TensorSpec(p + "mix.A_log", (m.heads,), 0.5, "norm"),
                TensorSpec(p + "mix.D", (m.heads,), 0.5, "norm"), TensorSpec(p + "mix.norm", (m.inner,), 1.0, "norm"),
                TensorSpec(p + "mix.o", (W, m.inner), MATRIX_STD)]
    if l.mlp is not None:
        out += [TensorSpec(p + "mlp.up", (l.mlp.ff, W), MATRIX_STD), TensorSpec(p + "mlp.down", (W, l.mlp.ff), MATRIX_STD)]
    return out


def tensor_specs(cfg: BolonexConfig) -> list[TensorSpec]:
    """Every tensor a Bolonex file holds for `cfg` (layers that use another layer's weights bring none), with the
    spread random weights are drawn with."""
    specs = [TensorSpec("embed", (cfg.vocab, cfg.width), MATRIX_STD)]
    for i, l in enumerate(cfg.layers):
        if l.weights_of is None:
            specs += _layer_specs(f"l{i}.", l, cfg.width)
    specs += [TensorSpec("final.norm", (cfg.width,), NORM_STD, "norm"), TensorSpec("head", (cfg.vocab, cfg.width), MATRIX_STD)]
    return specs


def _stack(parts: list[torch.Tensor]) -> torch.Tensor:
    if any(p.numel() == 0 for p in parts) or len({p.dtype for p in parts}) != 1:
        return torch.empty(0)                       # a fault already recorded by the store
    return torch.cat(parts, dim=0).contiguous()


class _LayerTensors:
    """The tensors of one source layer, taken from the store once and stacked the way the parts want them."""

    def __init__(self, cfg: BolonexConfig, w: WeightStore, i: int):
        l, W, p = cfg.layers[i], cfg.width, f"l{i}."
        m = l.mixer
        self.norm1 = w.take(p + "norm1", (W,))
        if l.type == ATTENTION:
            rows = (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim))
            mats = [w.take(f"{p}mix.{n}", (r, W)) for n, r in rows] + [w.take(p + "mix.g", (m.heads, W))]
            self.w_in = _stack(mats)                                    # [q | k | v | gate] rows
            self.bias = _stack([w.take(f"{p}mix.{n}.b", (r,)) for n, r in rows])
            self.conv_w = _stack([w.take(f"{p}mix.{n}.conv", (r, m.conv)) for n, r in rows])
            w.release(*[f"{p}mix.{n}" for n, _ in rows], p + "mix.g")
            self.q_norm, self.k_norm = w.take(p + "mix.q.norm", (m.dim,)), w.take(p + "mix.k.norm", (m.dim,))
            self.wo = w.take(p + "mix.o", (W, m.heads * m.vdim))
        else:
            self.w_in = w.take(p + "mix.in", (m.proj_width, W))
            self.conv_w = w.take(p + "mix.conv", (m.conv_width, m.conv))
            self.conv_b = w.take(p + "mix.conv.b", (m.conv_width,))
            self.dt_bias, self.a_log = w.take(p + "mix.dt_bias", (m.heads,)), w.take(p + "mix.A_log", (m.heads,))
            self.d_skip, self.norm = w.take(p + "mix.D", (m.heads,)), w.take(p + "mix.norm", (m.inner,))
            self.wo = w.take(p + "mix.o", (W, m.inner))
        if l.mlp is not None:
            self.up, self.down = w.take(p + "mlp.up", (l.mlp.ff, W)), w.take(p + "mlp.down", (W, l.mlp.ff))


def _block(cfg: BolonexConfig, l, t: _LayerTensors, device) -> ParallelBlock:
    m = l.mixer
    if l.type == ATTENTION:
        rope = None
        if m.rot is not None:
            rope = Rope(m.dim, m.rot.base, device, m.rot.dims, interleaved=True, scaling=m.rot.scaling_dict())
        mixer = ConvGatedAttention(t.w_in, t.wo, n_heads=m.heads, n_kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                                   scale=m.scale, softcap=m.softcap, position=rope, bias=t.bias,
                                   conv=ShortConv(t.conv_w),
                                   q_norm=t.q_norm, k_norm=t.k_norm, norm_eps=cfg.norm_eps, gated=True)
    else:
        mixer = Mamba2Mixer(t.w_in, t.wo, ShortConv(t.conv_w, t.conv_b, "silu"), t.dt_bias, t.a_log, t.d_skip, t.norm,
                            heads=m.heads, head_dim=m.vdim, state_dim=m.state, groups=m.groups,
                            norm_groups=m.norm_groups, norm_eps=cfg.norm_eps)
    ffn = DenseFfn(t.up, t.down, "gelu_tanh") if l.mlp is not None else None
    return ParallelBlock(RmsNorm(t.norm1, cfg.norm_eps, plus_one=True), mixer, ffn)


def build(cfg: BolonexConfig, w: WeightStore) -> DecoderModel:
    table = w.take("embed", (cfg.vocab, cfg.width))
    embedding = Embedding(table, scale=cfg.embedding_scale)
    tensors: dict[int, _LayerTensors] = {}
    for i, l in enumerate(cfg.layers):
        if l.weights_of is None:
            tensors[i] = _LayerTensors(cfg, w, i)
    final_norm = RmsNorm(w.take("final.norm", (cfg.width,)), cfg.norm_eps, plus_one=True)
    out = w.take("head", (cfg.vocab, cfg.width))
    w.finish()
    # one block per distinct (source layer, layer description): a layer that uses another layer's weights runs that
    # layer's block, with a cache slot of its own
    blocks, index, schedule, ropes = [], {}, [], {}
    for i, l in enumerate(cfg.layers):
        src = cfg.source_of(i)
        key = (src, l.type, l.mixer, l.mlp)
        if key not in index:
            index[key] = len(blocks)
            blocks.append(_block(cfg, l, tensors[src], w.device))
        schedule.append(LayerCall(index[key], i))
    # layers with the same rotary constants share one table per step
    for b in blocks:
        pos = getattr(b.mixer, "position", None)
        if pos is not None:
            k = (pos.head_dim, pos.base, pos.rotary_dims, pos.interleaved, tuple(sorted((pos.scaling or {}).items())))
            b.mixer.position = ropes.setdefault(k, pos)
    head = LmHead(final_norm, out)
    return DecoderModel(embedding, blocks, head, schedule, name=cfg.architecture)
