"""Small Bolonex configurations and weights for the tests.

The configurations differ from one another in every size and option: head sizes of keys and values that are equal or
not, one or several key/value heads, rotation of a whole head or part of it, with and without frequency rescaling,
with and without a score cap, scales that are not 1/sqrt(head size), convolutions of 2 to 5 taps, state-space groups
and norm groups that are 1, equal or unequal, layers without a feed-forward, layers that run with another layer's
weights (earlier or later in the list), and first layers of either kind.
"""
from __future__ import annotations

import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, conv, scale, softcap=0.0, rot_dims=None, base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale, "softcap": softcap}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims, "scaling": scaling}
    return m


def mamba2(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def layer(kind, mixer, ff=None, weights_of=None):
    e = {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def config(width, vocab, layers, scale=1.0, eps=1e-5):
    return {"architecture": "Bolonex", "width": width, "vocab": vocab, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "layers": layers}


_AT_A = attention(4, 2, 16, 24, 2, 0.31, 0.0, rot_dims=8, base=10000.0)
_MB_A = mamba2(2, 16, 16, 1, 1, 3)
# first layer a state-space mixer; values wider than keys; half of each key head rotated; no cap; no rescaling; a
# layer without a feed-forward; both kinds of layer run twice
BX_A = config(64, 300, [layer("mamba2", _MB_A, 96), layer("attention", _AT_A, None),
                        layer("mamba2", _MB_A, 96, weights_of=0), layer("attention", _AT_A, None, weights_of=1)], scale=2.0)

_AT_B = attention(3, 3, 32, 16, 4, 0.2, 10.0, rot_dims=32, base=5000.0,
                  scaling={"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64})
_MB_B = mamba2(6, 8, 40, 3, 2, 4)
# as many key/value heads as query heads; keys wider than values; odd vocabulary; rescaled frequencies whose three
# regimes all occur (wavelengths from 6 to 20,000 against 64/4 and 64/1); a layer that uses the weights of a LATER layer
BX_B = config(96, 257, [layer("attention", _AT_B, 160, weights_of=2), layer("mamba2", _MB_B, None),
                        layer("attention", _AT_B, 160), layer("mamba2", _MB_B, None, weights_of=1),
                        layer("mamba2", mamba2(4, 24, 24, 4, 1, 2), 64)], scale=0.5, eps=1e-6)

# rows that are no multiple of 16 bytes (width 100), odd sizes everywhere, five taps, one key/value head for five heads
BX_C = config(100, 333, [layer("attention", attention(5, 1, 20, 20, 5, 0.25, 30.0, rot_dims=20, base=300.0), 150),
                         layer("mamba2", mamba2(3, 12, 10, 3, 3, 5), 70)], scale=1.5)

# sizes at which the tensor-core kernels run: heads of 128, rows of 512 and more, pages of 64
BX_E = config(512, 3000, [layer("attention", attention(4, 2, 128, 128, 4, 0.09, 25.0, rot_dims=64, base=100000.0,
                                                      scaling={"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}), 1024),
                          layer("mamba2", mamba2(8, 64, 128, 2, 2, 4), 1024),
                          layer("attention", attention(4, 2, 128, 128, 4, 0.09, 25.0, rot_dims=64, base=100000.0,
                                                      scaling={"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}),
                                1024, weights_of=0)], scale=3.0)

# the smallest of everything: one tap (the "convolution" is a scale per channel and keeps no tail), no rotation, odd head
# sizes (keys of 6, values of 7, so heads of 8 in the cache), one state-space head of 5 with 7 states, one layer of each
BX_D = config(24, 50, [layer("attention", attention(2, 1, 6, 7, 1, 0.4), 40), layer("mamba2", mamba2(1, 5, 7, 1, 1, 1), None),
                       layer("mamba2", mamba2(3, 5, 9, 1, 3, 2), 16)], scale=1.0)

CASES = {"A": (BX_A, [5, 17, 23, 40, 11, 30], 4), "B": (BX_B, [1, 31, 40, 70, 9, 50], 8), "C": (BX_C, [3, 50, 64, 29, 77, 2], 16),
         "D": (BX_D, [4, 19, 1, 33, 8, 12], 4)}


def draw_tensors(cfg_dict: dict, seed: int, sharp: bool = False) -> dict:
    """Random weights by tensor name (bfloat16), drawn here with torch's generator.
    sharp: the norm weights of q and k are about 2.5, so that scores spread by about +-6 around 0 (a score is the sum
    of `dim` products of unit-rms numbers times scale, i.e. about w_q w_k for scale = 1/sqrt(dim)): softmax weights
    then differ by factors of hundreds, one or two keys carry a row's result, and a key that is read from a wrong
    place, rotated by a wrong angle or masked wrongly moves the logits by far more than the tolerance; the decay of
    the state-space layers is slow (exp(A_log) between 0.02 and 0.4) so that tokens hundreds of places back still
    weigh in the state."""
    from kungfu_b200.api import load_config
    from kungfu_b200 import registry
    cfg = load_config(dict(cfg_dict))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in registry.find(cfg.architecture).tensor_specs(cfg):
        name = spec.name
        x = torch.randn(tuple(spec.shape), generator=g)
        if name.endswith((".q.norm", ".k.norm")):
            x = (2.5 if sharp else 1.0) + 0.3 * x
        elif name.endswith("mix.norm"):
            x = 1.0 + 0.2 * x
        elif name.endswith(("norm1", "final.norm")):
            x = 0.1 * x
        elif name.endswith(".conv"):
            x = 0.5 * x
        elif name.endswith(".b"):
            x = 0.1 * x
        elif name.endswith("A_log"):
            x = (-4.0 + 3.0 * torch.rand(tuple(spec.shape), generator=g)) if sharp else 0.5 * x
        elif name.endswith(("dt_bias", "mix.D")):
            x = 0.5 * x
        elif name == "embed":
            x = 0.5 * x
        else:
            x = x / (spec.shape[-1] ** 0.5)                  # projections keep the spread of their input
        out[name] = x.to(torch.bfloat16)
    return out


def write_model(folder: str, cfg_dict: dict, seed: int, sharp: bool = False) -> str:
    from kungfu_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), draw_tensors(cfg_dict, seed, sharp))
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg_dict, f)
    return folder
