"""Small Petanex configurations and weights for the tests.

The configurations differ from one another in every size and option: latent sizes that fill a stored head or not, one
to twenty heads, delta rules with as many query/key heads as heads, fewer, or one, key sizes from 8 to 136, value sizes that are
no multiple of anything, convolutions of 1 to 5 taps, factored decays and gates of unequal ranks, layers without a
feed-forward, mixtures with and without groups, with and without a shared expert, with one choice and with several,
models with and without the per-token side input, either kind of layer first.
"""
from __future__ import annotations

import json
import os

import torch


def latent(heads, dim, vdim, rank, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, scale=1.0, groups=None, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r,
            "shared": {"ff": shared[0], "limit": shared[1]} if shared else None}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, layers, scale=1.0, eps=1e-5, side=0):
    c = {"architecture": "Petanex", "width": width, "vocab": vocab, "embedding": {"scale": scale}, "norm": {"eps": eps},
         "layers": layers}
    if side:
        c["token_side"] = {"dim": side}
    return c


# a delta rule first, fewer query/key heads than heads, values wider than keys; a mixture in groups with a shared expert of
# another width; a latent that does not fill its stored head; a layer without a feed-forward; a mixture without groups or
# shared expert that takes half of its experts
PX_A = config(64, 300, [layer("delta", delta(4, 2, 16, 24, 3), moe(8, 2, 32, 1.0, 2.0, groups=(4, 2), shared=(48, 2.0))),
                        layer("latent_attention", latent(4, 16, 24, 20, 0.3), dense(96)),
                        layer("channel_delta", delta(3, 3, 8, 12, 2)),
                        layer("latent_attention", latent(2, 8, 8, 16, 0.5), moe(6, 3, 40, 3.0))], scale=2.0, side=8)

# no side input; attention first; one query/key head for four heads; a delta rule with a single head and a single tap; a
# mixture that takes one expert of five; another epsilon
PX_B = config(96, 257, [layer("latent_attention", latent(3, 24, 16, 40, 0.2), moe(5, 1, 64, 0.7, 1.5)),
                        layer("channel_delta", delta(4, 1, 20, 10, 4), dense(160)),
                        layer("delta", delta(1, 1, 40, 33, 1), None),
                        layer("delta", delta(6, 6, 8, 8, 4), dense(64))], scale=0.5, eps=1e-6)

# rows that are no multiple of 16 bytes (width 100), odd sizes everywhere, keys of 136 (the widest instance of the
# recurrence), five taps, twenty heads over a latent (more than a tensor-core tile of query rows), two of three groups of four
PX_C = config(100, 333, [layer("channel_delta", delta(2, 1, 136, 20, 5), moe(12, 4, 30, 2.0, 0.8, groups=(3, 2), shared=(30, 2.0))),
                         layer("latent_attention", latent(20, 12, 10, 33, 0.25), dense(150)),
                         layer("delta", delta(6, 3, 12, 7, 2), dense(70))], scale=1.5, side=5)

# sizes at which the tensor-core kernels run: a latent of 128, rows of 512, pages of 64
PX_E = config(512, 3000, [layer("latent_attention", latent(4, 64, 64, 128, 0.11), dense(1024)),
                          layer("delta", delta(4, 2, 64, 64, 4), moe(16, 4, 256, 4.0, 2.5, groups=(4, 2), shared=(256, 4.0))),
                          layer("channel_delta", delta(4, 4, 128, 64, 4), dense(1024)),
                          layer("latent_attention", latent(8, 32, 32, 64, 0.15), moe(16, 2, 128, 4.0, 1.0))], scale=3.0, side=16)

# the smallest of everything, and rows that are no multiple of 8 bytes: width 90, vocabulary 101, a latent of 9, keys of 6 and
# 10, values of 5 and 6, a side input of 3, four experts of which two are taken
PX_D = config(90, 101, [layer("latent_attention", latent(3, 10, 6, 9, 0.4), moe(4, 2, 18, 1.0, 1.0, shared=(10, 1.0))),
                        layer("delta", delta(2, 1, 6, 5, 3), dense(34)),
                        layer("channel_delta", delta(2, 2, 10, 6, 2))], scale=1.0, side=3)

CASES = {"A": (PX_A, [5, 17, 23, 40, 11, 30], 4), "B": (PX_B, [1, 31, 40, 70, 9, 50], 8), "C": (PX_C, [3, 50, 64, 29, 77, 2], 16),
         "D": (PX_D, [4, 19, 1, 33, 8, 12], 4)}
RANKS = {"A": (5, 7), "B": (12, 6), "C": (9, 9), "D": (3, 2), "E": (32, 24)}          # (decay rank, gate rank) of the channel_delta layers


def draw_tensors(cfg_dict: dict, seed: int, sharp: bool = False, ranks=(6, 10)) -> dict:
    """Random weights by tensor name (bfloat16), drawn here with torch's generator.
    sharp: the query matrices of latent attention are four times larger, so that softmax weights differ by factors of
    hundreds and one or two keys carry a row; the decays of the delta rules are slow (exp(A_log) between 0.02 and 0.4, small
    steps), so that tokens hundreds of places back still weigh in the state; router matrices are wide either way, so that
    few choices are close calls."""
    from kungfu_b200.api import load_config
    from kungfu_b200 import registry
    raw = json.loads(json.dumps(cfg_dict))
    for l in raw["layers"]:
        if l["type"] == "channel_delta":
            l["mixer"].update(decay_rank=ranks[0], gate_rank=ranks[1])          # only to size the tensors: files do not carry it
    cfg = load_config(raw)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in registry.find(cfg.architecture).tensor_specs(cfg):
        name = spec.name
        x = torch.randn(tuple(spec.shape), generator=g)
        if name.endswith(("norm1", "norm2", "final.norm", "side.norm", "mix.norm", "dkv.norm")):
            x = 1.0 + 0.2 * x
        elif name.endswith(("ls1", "ls2")):
            x = 0.6 + 0.2 * x
        elif name.endswith(".conv"):
            x = 0.5 * x
        elif name.endswith("A_log"):
            x = (-4.0 + 3.0 * torch.rand(tuple(spec.shape), generator=g)) if sharp else 0.5 * x
        elif name.endswith("dt_bias"):
            x = (-1.0 + 0.5 * x) if sharp else 0.5 * x
        elif name.endswith("correction"):
            x = 0.2 * x
        elif name.endswith("router"):
            x = 4.0 * x / (spec.shape[-1] ** 0.5)
        elif name in ("embed", "side.embed"):
            x = 0.5 * x
        elif name.endswith("mix.q") and sharp and _is_latent(cfg, name):
            x = 4.0 * x / (spec.shape[-1] ** 0.5)
        else:
            x = x / (spec.shape[-1] ** 0.5)                  # projections keep the spread of their input
        out[name] = x.to(torch.bfloat16)
    return out


def _is_latent(cfg, name: str) -> bool:
    return cfg.layers[int(name.split(".")[0][1:])].type == "latent_attention"


def write_model(folder: str, cfg_dict: dict, seed: int, sharp: bool = False, ranks=(6, 10)) -> str:
    from kungfu_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), draw_tensors(cfg_dict, seed, sharp, ranks))
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg_dict, f)
    return folder
