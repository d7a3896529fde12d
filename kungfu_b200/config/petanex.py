"""Petanex hyperparameters, read from the model's own config.json.

A Petanex file describes its model layer by layer; nothing is implied by a layer's index and no size is fixed by the
design: every number below is read from the file (or, for the ranks of factored projections, from a tensor's shape).

  architecture            "Petanex"
  width, vocab            residual width, vocabulary
  embedding.scale         factor on the embedding rows
  norm.eps                epsilon of every RMS norm
  token_side.dim          columns of the per-token side table each layer reads (absent: no side input)
  layers[i].type          latent_attention | delta | channel_delta
  layers[i].mixer         latent_attention: heads, dim (query/key head size), vdim, kv_rank (latent size), scale
                          delta, channel_delta: heads, kv_heads, dim, vdim, conv (taps);
                                     channel_delta may name decay_rank and gate_rank (else the tensors' shapes give them)
  layers[i].mlp           null | {kind: dense, ff}
                          | {kind: moe, expert {ff, limit}, router {experts, top, scale, groups {count, keep}}, shared {ff, limit} | null}
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

LATENT, DELTA, CHANNEL_DELTA = "latent_attention", "delta", "channel_delta"
DEFAULT_RANK = 32           # rank of a factored projection when neither the file nor a tensor says (random weights)


@dataclass(frozen=True)
class LatentSpec:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float


@dataclass(frozen=True)
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int | None = None           # channel_delta only
    gate_rank: int | None = None

    @property
    def qkv_width(self) -> int:
        return 2 * self.kv_heads * self.dim + self.heads * self.vdim


@dataclass(frozen=True)
class ExpertSpec:
    ff: int
    limit: float


@dataclass(frozen=True)
class MlpSpec:
    kind: str                                # dense | moe
    ff: int = 0                              # dense
    expert: ExpertSpec | None = None         # moe
    experts: int = 0
    top: int = 0
    scale: float = 1.0
    groups: int = 1
    keep: int = 1
    shared: ExpertSpec | None = None


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: LatentSpec | DeltaSpec
    mlp: MlpSpec | None


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


def _expert(k: KeyReader) -> ExpertSpec:
    return ExpertSpec(k.int("ff", min=1), k.float("limit"))


def _mlp(k: KeyReader | None) -> MlpSpec | None:
    if k is None:
        return None
    kind = k.str("kind", "dense", choices=("dense", "moe"))
    if kind == "dense":
        return MlpSpec("dense", ff=k.int("ff", min=1))
    r = _sub(k, "router")
    g = _sub(r, "groups", required=False)
    sh = _sub(k, "shared", required=False)
    return MlpSpec("moe", expert=_expert(_sub(k, "expert")), experts=r.int("experts", min=1), top=r.int("top", min=1),
                   scale=r.float("scale", 1.0), groups=g.int("count", 1, min=1) if g is not None else 1,
                   keep=g.int("keep", 1, min=1) if g is not None else 1, shared=_expert(sh) if sh is not None else None)


@dataclass(frozen=True)
class PetanexConfig:
    architecture: str
    width: int
    vocab: int
    embedding_scale: float
    norm_eps: float
    side_dim: int = 0                                    # 0: no per-token side input
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

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "PetanexConfig":
        k = KeyReader(raw, where)
        arch = k.str("architecture")
        width, vocab = k.int("width", min=1), k.int("vocab", min=1)
        emb = _sub(k, "embedding", required=False)
        scale = emb.float("scale", 1.0) if emb is not None else 1.0
        eps = _sub(k, "norm").float("eps")
        side = _sub(k, "token_side", required=False)
        side_dim = side.int("dim", 0, min=0) if side is not None else 0
        layers = []
        for i, e in enumerate(k.list("layers")):
            lk = KeyReader(e, f"{where}: layers[{i}]")
            kind = lk.str("type", choices=(LATENT, DELTA, CHANNEL_DELTA))
            mk = _sub(lk, "mixer")
            if kind == LATENT:
                mixer = LatentSpec(mk.int("heads", min=1), mk.int("dim", min=1), mk.int("vdim", min=1),
                                   mk.int("kv_rank", min=1), mk.float("scale"))
            else:
                heads = mk.int("heads", min=1)
                mixer = DeltaSpec(heads, mk.int("kv_heads", heads, min=1), mk.int("dim", min=1), mk.int("vdim", min=1),
                                  mk.int("conv", 1, min=1),
                                  mk.int("decay_rank", None, min=1) if kind == CHANNEL_DELTA else None,
                                  mk.int("gate_rank", None, min=1) if kind == CHANNEL_DELTA else None)
            layers.append(LayerSpec(kind, mixer, _mlp(_sub(lk, "mlp", required=False))))
        cfg = cls(arch, width, vocab, scale, eps, side_dim, tuple(layers))
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
            if l.type == LATENT:
                if m.kv_rank > 256:
                    raise ConfigError(f"{at}: a latent of {m.kv_rank} is above 256, the largest head the attention kernels take")
                if not (m.scale > 0):
                    raise ConfigError(f"{at}: scale must be positive")
            else:
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{at}: heads {m.heads} is not a multiple of kv_heads {m.kv_heads}")
                if m.dim > 256:
                    raise ConfigError(f"{at}: key sizes above 256 are not supported, found {m.dim}")
                if m.conv > 8:
                    raise ConfigError(f"{at}: a short convolution has at most 8 taps, found {m.conv}")
            f = l.mlp
            if f is not None and f.kind == "moe":
                if f.top > f.experts or f.experts % f.groups or not (1 <= f.keep <= f.groups):
                    raise ConfigError(f"{at}: mlp: {f.experts} experts, top {f.top}, groups {f.groups}, keep {f.keep} do not fit")
                if f.groups > 1 and f.keep * (f.experts // f.groups) < f.top:
                    raise ConfigError(f"{at}: mlp: {f.keep} groups of {f.experts // f.groups} experts cannot give {f.top} choices")
                if f.experts > 1024:
                    raise ConfigError(f"{at}: mlp: more than 1024 experts are not supported")

    def to_dict(self) -> dict:
        """A config.json dictionary that `from_dict` reads back to this configuration."""
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == LATENT:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
                if m.decay_rank is not None:
                    mixer["decay_rank"] = m.decay_rank
                if m.gate_rank is not None:
                    mixer["gate_rank"] = m.gate_rank
            f = l.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.expert.ff, "limit": f.expert.limit},
                       "router": {"experts": f.experts, "top": f.top, "scale": f.scale,
                                  "groups": {"count": f.groups, "keep": f.keep}},
                       "shared": None if f.shared is None else {"ff": f.shared.ff, "limit": f.shared.limit}}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out

    def with_shapes(self, shape_of) -> "PetanexConfig":
        """This configuration with the sizes that only tensors give filled in: `shape_of(name)` is a stored tensor's shape
        or None.  The ranks of a channel_delta layer's factored decay and gate are the row counts of `l<i>.mix.a1` and
        `l<i>.mix.g1`."""
        layers = []
        for i, l in enumerate(self.layers):
            if l.type == CHANNEL_DELTA:
                a, g = shape_of(f"l{i}.mix.a1"), shape_of(f"l{i}.mix.g1")
                m = dataclasses.replace(l.mixer, decay_rank=l.mixer.decay_rank if l.mixer.decay_rank is not None else (int(a[0]) if a else None),
                                        gate_rank=l.mixer.gate_rank if l.mixer.gate_rank is not None else (int(g[0]) if g else None))
                l = dataclasses.replace(l, mixer=m)
            layers.append(l)
        return dataclasses.replace(self, layers=tuple(layers))

    def replace(self, **kw) -> "PetanexConfig":
        cfg = dataclasses.replace(self, **kw)
        cfg.validate()
        return cfg

    def state_summary(self, element_size: int = 2) -> list:
        """Per layer, what it keeps per request: bytes per token of the paged latent, and fixed bytes."""
        from ..parts.latent import latent_head_size
        out = []
        for i, l in enumerate(self.layers):
            m = l.mixer
            if l.type == LATENT:
                out.append({"layer": i, "kind": "latent_cache", "bytes_per_token": 2 * latent_head_size(m.kv_rank) * element_size,
                            "window": None, "fixed_bytes": 0})
            else:
                out.append({"layer": i, "kind": "recurrent+conv_tail", "bytes_per_token": 0, "window": None,
                            "fixed_bytes": 4 * (m.heads * m.dim * m.vdim + max(m.conv - 1, 0) * m.qkv_width)})
        return out
