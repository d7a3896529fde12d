"""Bolonex hyperparameters, read from the model's own config.json.

A Bolonex file describes its model layer by layer: `layers` is a list whose entries give the mixer's `type`
('attention' or 'mamba2'), the mixer's sizes and constants (`mixer`), the feed-forward (`mlp`, null for none) and,
for a layer that reuses another layer's tensors with a cache or state of its own, `weights_of`.  Nothing is
implied by a layer's index and no size is fixed by the design: every number below is read from the file.

  architecture            "Bolonex"
  width, vocab            residual width, vocabulary
  embedding.scale         factor on the embedding rows
  norm.eps                epsilon of every RMS norm
  layers[i].type          attention | mamba2
  layers[i].mixer         attention: heads, kv_heads, dim (q/k head size), vdim (value head size), conv (taps), scale,
                                     softcap (0 or absent: none), rot {base, dims, scaling {factor, low, high, original} | null}
                          mamba2:    heads, vdim (head size), state, groups, norm_groups, conv (taps)
  layers[i].mlp           {kind: dense, ff} | null
  layers[i].weights_of    index of the layer whose tensors this layer uses (optional)
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

ATTENTION, MAMBA2 = "attention", "mamba2"


@dataclass(frozen=True)
class RotarySpec:
    base: float
    dims: int
    scaling: tuple | None = None            # (factor, low, high, original) or None

    def scaling_dict(self) -> dict | None:
        if self.scaling is None:
            return None
        return dict(zip(("factor", "low", "high", "original"), self.scaling))


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                                # taps of the short convolution on q, k, v (1: none)
    scale: float
    softcap: float                           # 0: none
    rot: RotarySpec | None

    @property
    def qkv_width(self) -> int:
        return (self.heads + self.kv_heads) * self.dim + self.kv_heads * self.vdim


@dataclass(frozen=True)
class Mamba2Spec:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_width(self) -> int:
        return self.inner + 2 * self.groups * self.state

    @property
    def proj_width(self) -> int:
        return self.inner + self.conv_width + self.heads


@dataclass(frozen=True)
class MlpSpec:
    kind: str                                # dense
    ff: int


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: AttentionSpec | Mamba2Spec
    mlp: MlpSpec | None
    weights_of: int | None = None


def _sub(k: KeyReader, key: str, required: bool = True) -> KeyReader | None:
    raw = k.raw.get(key)
    k.read.add(key)
    if raw is None:
        if required:
            raise ConfigError(f"{k.where}: required key '{key}' is missing")
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"{k.where}: key '{key}' must be an object, found {raw!r}")
    return KeyReader(raw, f"{k.where}: {key}")


def _attention(k: KeyReader) -> AttentionSpec:
    heads = k.int("heads", min=1)
    kv_heads = k.int("kv_heads", heads, min=1)
    dim = k.int("dim", min=1)
    vdim = k.int("vdim", dim, min=1)
    conv = k.int("conv", 1, min=1)
    scale = k.float("scale")
    softcap = k.float("softcap", 0.0)
    r = _sub(k, "rot", required=False)
    rot = None
    if r is not None:
        base, dims = r.float("base"), r.int("dims", dim, min=0)
        s = _sub(r, "scaling", required=False)
        scaling = None if s is None else (s.float("factor"), s.float("low"), s.float("high"), s.float("original"))
        rot = RotarySpec(base, dims, scaling) if dims > 0 else None
    return AttentionSpec(heads, kv_heads, dim, vdim, conv, scale, softcap, rot)


def _mamba2(k: KeyReader) -> Mamba2Spec:
    return Mamba2Spec(k.int("heads", min=1), k.int("vdim", min=1), k.int("state", min=1), k.int("groups", 1, min=1),
                      k.int("norm_groups", 1, min=1), k.int("conv", 1, min=1))


@dataclass(frozen=True)
class BolonexConfig:
    architecture: str
    width: int
    vocab: int
    embedding_scale: float
    norm_eps: float
    layers: tuple = field(default_factory=tuple)         # LayerSpec per layer

    # what the engine and the command line ask of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def source_of(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself unless `weights_of` points elsewhere, followed to its end)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"layers[{i}]: 'weights_of' runs in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "BolonexConfig":
        k = KeyReader(raw, where)
        arch = k.str("architecture")
        width, vocab = k.int("width", min=1), k.int("vocab", min=1)
        emb = _sub(k, "embedding", required=False)
        scale = emb.float("scale", 1.0) if emb is not None else 1.0
        eps = _sub(k, "norm").float("eps")
        entries = k.list("layers")
        layers = []
        for i, e in enumerate(entries):
            lk = KeyReader(e, f"{where}: layers[{i}]")
            kind = lk.str("type", choices=(ATTENTION, MAMBA2))
            mk = _sub(lk, "mixer")
            mixer = _attention(mk) if kind == ATTENTION else _mamba2(mk)
            fk = _sub(lk, "mlp", required=False)
            mlp = None if fk is None else MlpSpec(fk.str("kind", "dense", choices=("dense",)), fk.int("ff", min=1))
            src = lk.int("weights_of", None)
            layers.append(LayerSpec(kind, mixer, mlp, src))
        cfg = cls(arch, width, vocab, scale, eps, tuple(layers))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if not self.layers:
            raise ConfigError(f"{where}: 'layers' is empty")
        if not (self.norm_eps > 0):
            raise ConfigError(f"{where}: norm.eps must be positive, found {self.norm_eps}")
        for i, l in enumerate(self.layers):
            at = f"{where}: layers[{i}]"
            m = l.mixer
            if l.type == ATTENTION:
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{at}: heads {m.heads} is not a multiple of kv_heads {m.kv_heads}")
                if max(m.dim, m.vdim) > 256:
                    raise ConfigError(f"{at}: head sizes above 256 are not supported (dim {m.dim}, vdim {m.vdim})")
                if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                    raise ConfigError(f"{at}: rot.dims {m.rot.dims} must be even and at most dim {m.dim}")
                if not (m.scale > 0) or m.softcap < 0:
                    raise ConfigError(f"{at}: scale must be positive and softcap >= 0")
            else:
                if m.heads % m.groups:
                    raise ConfigError(f"{at}: heads {m.heads} is not a multiple of groups {m.groups}")
                if m.inner % m.norm_groups:
                    raise ConfigError(f"{at}: heads * vdim = {m.inner} is not a multiple of norm_groups {m.norm_groups}")
                if m.state > 256:
                    raise ConfigError(f"{at}: state sizes above 256 are not supported, found {m.state}")
            if m.conv > 8:
                raise ConfigError(f"{at}: a short convolution has at most 8 taps, found {m.conv}")
            if l.weights_of is not None:
                j = l.weights_of
                if not (0 <= j < len(self.layers)) or j == i:
                    raise ConfigError(f"{at}: 'weights_of' {j} names no other layer")
                src = self.layers[self.source_of(i)]
                if src.type != l.type:
                    raise ConfigError(f"{at}: is '{l.type}' but uses the weights of layer {self.source_of(i)}, a '{src.type}'")

    def to_dict(self) -> dict:
        """A config.json dictionary that `from_dict` reads back to this configuration."""
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == ATTENTION:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv,
                         "scale": m.scale, "softcap": m.softcap,
                         "rot": None if m.rot is None else {"base": m.rot.base, "dims": m.rot.dims, "scaling": m.rot.scaling_dict()}}
            else:
                mixer = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups,
                         "norm_groups": m.norm_groups, "conv": m.conv}
            e = {"type": l.type, "mixer": mixer, "mlp": None if l.mlp is None else {"kind": l.mlp.kind, "ff": l.mlp.ff}}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            layers.append(e)
        return {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": layers}

    def replace(self, **kw) -> "BolonexConfig":
        cfg = dataclasses.replace(self, **kw)
        cfg.validate()
        return cfg

    def state_summary(self, element_size: int = 2) -> list:
        """Per layer, what it keeps per request: bytes per token of paged keys and values, and fixed bytes."""
        out = []
        for i, l in enumerate(self.layers):
            m = l.mixer
            if l.type == ATTENTION:
                d = (max(m.dim, m.vdim) + 1) // 2 * 2
                out.append({"layer": i, "kind": "kv_cache+conv_tail", "bytes_per_token": 2 * m.kv_heads * d * element_size,
                            "window": None, "fixed_bytes": 4 * max(m.conv - 1, 0) * m.qkv_width})
            else:
                out.append({"layer": i, "kind": "recurrent+conv_tail", "bytes_per_token": 0, "window": None,
                            "fixed_bytes": 4 * (m.heads * m.vdim * m.state + max(m.conv - 1, 0) * m.conv_width)})
        return out
