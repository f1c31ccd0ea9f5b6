"""Configuration of the Pemezen design (config.json "architecture": "Pemezen").

A decoder whose layers are listed one by one: each entry of `layers` names its mixer (`type`), the mixer's sizes
(`mixer`) and its feed-forward (`mlp`, or null).  Every size and every constant that can differ between two models
of the design is read here; nothing of them stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ConfigReader

ARCHITECTURE = "Pemezen"
MIXERS = ("latent_attention", "latent_attention_2", "rglru")


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    scaling: dict | None     # {"factor", "original", "fast", "slow"} or None


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                 # per head: query/key entries that are not rotated
    rot_dim: int             # per head: rotated query entries; the width of the one rotated key part
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    gate: str                # "element" or "head"


@dataclass(frozen=True)
class RGLRUConfig:
    width: int
    blocks: int
    conv: int                # taps of its convolution


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object
    ff: int | None           # width of the dense feed-forward, None: the layer has none


@dataclass(frozen=True)
class PemezenConfig:
    vocab: int
    width: int
    layers: tuple
    norm_eps: float
    norm_groups: int
    canon_taps: int
    embedding_scale: float
    logit_softcap: float | None
    raw: dict = field(compare=False, repr=False, default_factory=dict)

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, data: dict, source: str = "config.json") -> "PemezenConfig":
        r = ConfigReader(data, source)
        width = r.integer("width", minimum=1)
        entries = data.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{source}: key 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(entries):
            where = f"{source}: layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} must be an object")
            e = ConfigReader(entry, where)
            kind = e.string("type")
            if kind not in MIXERS:
                raise ConfigError(f"{where}: type '{kind}' is not known (known: {', '.join(MIXERS)})")
            if kind == "rglru":
                mixer = RGLRUConfig(width=e.integer("mixer.width", minimum=1), blocks=e.integer("mixer.blocks", minimum=1),
                                    conv=e.integer("mixer.conv", minimum=1))
                if mixer.width % mixer.blocks:
                    raise ConfigError(f"{where}: mixer.width {mixer.width} is not a multiple of mixer.blocks {mixer.blocks}")
            else:
                rot_dim = e.integer("mixer.rot_dim", minimum=0)
                scaling = entry["mixer"].get("rot", {}).get("scaling") if isinstance(entry.get("mixer"), dict) else None
                if scaling is not None:
                    s = ConfigReader(scaling, where + " mixer.rot.scaling")
                    scaling = dict(factor=s.number("factor", exclusive_minimum=0.0), original=s.number("original", exclusive_minimum=0.0),
                                   fast=s.number("fast", exclusive_minimum=0.0), slow=s.number("slow", exclusive_minimum=0.0))
                rot = RotaryConfig(dims=e.integer("mixer.rot.dims", default=rot_dim, minimum=0),
                                   base=e.number("mixer.rot.base", default=10000.0, exclusive_minimum=1.0), scaling=scaling)
                if rot.dims % 2 or rot.dims > rot_dim:
                    raise ConfigError(f"{where}: mixer.rot.dims {rot.dims} must be even and at most mixer.rot_dim {rot_dim}")
                mixer = LatentAttentionConfig(heads=e.integer("mixer.heads", minimum=1), dim=e.integer("mixer.dim", minimum=1),
                                              rot_dim=rot_dim, vdim=e.integer("mixer.vdim", minimum=1),
                                              kv_rank=e.integer("mixer.kv_rank", minimum=1),
                                              scale=e.number("mixer.scale", exclusive_minimum=0.0), rot=rot,
                                              gate="element" if kind == "latent_attention" else "head")
            ff = None
            if entry.get("mlp") is not None:
                mlp_kind = e.string("mlp.kind", default="dense")
                if mlp_kind != "dense":
                    raise ConfigError(f"{where}: mlp.kind '{mlp_kind}' is not known (known: dense)")
                ff = e.integer("mlp.ff", minimum=1)
            layers.append(LayerConfig(kind, mixer, ff))
        groups = r.integer("norm.groups", default=1, minimum=1)
        if width % groups:
            raise ConfigError(f"{source}: width {width} is not a multiple of norm.groups {groups}")
        return cls(vocab=r.integer("vocab", minimum=1), width=width, layers=tuple(layers),
                   norm_eps=r.number("norm.eps", exclusive_minimum=0.0), norm_groups=groups,
                   canon_taps=r.integer("canon.taps", minimum=1), embedding_scale=r.number("embedding.scale", default=1.0),
                   logit_softcap=r.number("logit_softcap", default=None, exclusive_minimum=0.0), raw=data)

    # (what the command line prints about a loaded model)
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> dict:
        """config.json form of this configuration."""
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "rglru":
                mixer = dict(width=m.width, blocks=m.blocks, conv=m.conv)
            else:
                rot = dict(dims=m.rot.dims, base=m.rot.base)
                if m.rot.scaling:
                    rot["scaling"] = dict(m.rot.scaling)
                mixer = dict(heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale, rot=rot)
            layers.append(dict(type=l.type, mixer=mixer, mlp=None if l.ff is None else dict(kind="dense", ff=l.ff)))
        d = dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, layers=layers,
                 norm=dict(eps=self.norm_eps, groups=self.norm_groups), canon=dict(taps=self.canon_taps),
                 embedding=dict(scale=self.embedding_scale))
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d

    def describe(self) -> dict:
        return self.to_dict()
