"""Configuration of the Novunex design (config.json "architecture": "Novunex").

A decoder whose layers are listed one by one: each entry of `layers` names its mixer (`type`), the mixer's sizes
(`mixer`) and its feed-forward (`mlp`, or null).  Both mixers are grouped-query attention over keys and values of
different widths; they differ in how queries and keys are normed, in the frequency scaling of the rotation and in the
softmax (one has a sink).  A layer may read the keys and values of an earlier layer (`mixer.kv_from`) instead of making
its own.  The feed-forward is a mixture of small experts with identity experts and an optional shared expert.  Every size
and every constant that can differ between two models of the design is read here; nothing of them stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ConfigReader

ARCHITECTURE = "Novunex"
MIXERS = ("attention", "attention_2")
SCALING_KEYS = ("factor", "low", "high", "original")


@dataclass(frozen=True)
class RotaryConfig:
    dims: int                # rotated entries of every head (the first ones), even
    base: float
    scaling: dict | None     # {"factor", "low", "high", "original"} or None


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int                 # per head: query/key entries
    vdim: int                # per head: value entries
    scale: float
    rot: RotaryConfig
    kv_from: int | None      # the layer whose keys and values this one reads; None: its own


@dataclass(frozen=True)
class MixtureConfig:
    experts: int             # experts with tensors
    identity: int            # router outputs behind them whose expert returns its input
    top: int
    ff: int                  # inner width of an expert
    shared_ff: int | None    # inner width of the shared expert, None: the layer has none


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: AttentionConfig
    mlp: MixtureConfig | None


@dataclass(frozen=True)
class NovunexConfig:
    vocab: int
    width: int
    layers: tuple
    norm_eps: float
    raw: dict = field(compare=False, repr=False, default_factory=dict)

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, data: dict, source: str = "config.json") -> "NovunexConfig":
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
            dim = e.integer("mixer.dim", minimum=1)
            scaling = entry["mixer"].get("rot", {}).get("scaling") if isinstance(entry.get("mixer"), dict) else None
            if scaling is not None:
                if kind != "attention_2":
                    raise ConfigError(f"{where}: mixer.rot.scaling belongs to layers of type 'attention_2'")
                s = ConfigReader(scaling, where + " mixer.rot.scaling")
                scaling = {k: s.number(k, exclusive_minimum=0.0) for k in SCALING_KEYS}
                if scaling["high"] == scaling["low"]:
                    raise ConfigError(f"{where}: mixer.rot.scaling.high must differ from mixer.rot.scaling.low")
            rot = RotaryConfig(dims=e.integer("mixer.rot.dims", default=0, minimum=0),
                               base=e.number("mixer.rot.base", default=10000.0, exclusive_minimum=0.0), scaling=scaling)
            if rot.dims % 2 or rot.dims > dim:
                raise ConfigError(f"{where}: mixer.rot.dims {rot.dims} must be even and at most mixer.dim {dim}")
            mixer = AttentionConfig(heads=e.integer("mixer.heads", minimum=1), kv_heads=e.integer("mixer.kv_heads", minimum=1), dim=dim,
                                    vdim=e.integer("mixer.vdim", minimum=1), scale=e.number("mixer.scale", exclusive_minimum=0.0),
                                    rot=rot, kv_from=e.integer("mixer.kv_from", default=None, minimum=0))
            if mixer.heads % mixer.kv_heads:
                raise ConfigError(f"{where}: mixer.heads {mixer.heads} is not a multiple of mixer.kv_heads {mixer.kv_heads}")
            if mixer.kv_from is not None:
                if mixer.kv_from >= i:
                    raise ConfigError(f"{where}: mixer.kv_from {mixer.kv_from} must name an earlier layer")
                src = layers[mixer.kv_from]
                if src.mixer.kv_from is not None:
                    raise ConfigError(f"{where}: mixer.kv_from names layer {mixer.kv_from}, which has no keys and values of its own")
                if (src.type, src.mixer.kv_heads, src.mixer.dim, src.mixer.vdim) != (kind, mixer.kv_heads, mixer.dim, mixer.vdim):
                    raise ConfigError(f"{where}: mixer.kv_from names layer {mixer.kv_from}, whose keys and values are of another kind or size")
            mlp = None
            if entry.get("mlp") is not None:
                mlp_kind = e.string("mlp.kind", default="moe")
                if mlp_kind != "moe":
                    raise ConfigError(f"{where}: mlp.kind '{mlp_kind}' is not known (known: moe)")
                mlp = MixtureConfig(experts=e.integer("mlp.router.experts", minimum=0),
                                    identity=e.integer("mlp.router.identity", default=0, minimum=0),
                                    top=e.integer("mlp.router.top", minimum=1), ff=e.integer("mlp.expert.ff", minimum=1),
                                    shared_ff=e.integer("mlp.shared.ff", minimum=1) if entry["mlp"].get("shared") is not None else None)
                if mlp.experts + mlp.identity < mlp.top:
                    raise ConfigError(f"{where}: mlp.router.top {mlp.top} is more than the router's {mlp.experts + mlp.identity} outputs")
            layers.append(LayerConfig(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=width, layers=tuple(layers),
                   norm_eps=r.number("norm.eps", exclusive_minimum=0.0), raw=data)

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
            rot = dict(dims=m.rot.dims, base=m.rot.base)
            if m.rot.scaling:
                rot["scaling"] = dict(m.rot.scaling)
            mixer = dict(heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, rot=rot)
            if m.kv_from is not None:
                mixer["kv_from"] = m.kv_from
            mlp = None
            if l.mlp is not None:
                mlp = dict(kind="moe", expert=dict(ff=l.mlp.ff),
                           router=dict(experts=l.mlp.experts, identity=l.mlp.identity, top=l.mlp.top))
                if l.mlp.shared_ff is not None:
                    mlp["shared"] = dict(ff=l.mlp.shared_ff)
            layers.append(dict(type=l.type, mixer=mixer, mlp=mlp))
        return dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, layers=layers, norm=dict(eps=self.norm_eps))

    def describe(self) -> dict:
        return self.to_dict()
