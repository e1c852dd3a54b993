"""MuvoraxConfig: the sizes, constants and order of layers of a Muvorax decoder, from config.json.

The file is nested: `layers` is a list whose entries give the layer's `type` (which mixer:
`lightning`, linear attention with a decay per head; `latent_attention`, softmax attention over a
cached latent; `mamba1`, the selective scan), the mixer's sizes and constants under `mixer`, and its
feed-forward under `mlp` (null: none; `kind` dense or moe). Model-wide: `vocab`, `width`,
`norm.eps`. Nothing about a model of this family is written anywhere else: tensors' shapes follow
from these.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

LAYER_TYPES = ("lightning", "latent_attention", "mamba1")


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int                 # width of a query/key head
    vdim: int                # width of a value head
    decay: tuple[float, ...]  # one per head


@dataclass(frozen=True)
class RotationConfig:
    dims: int                # leading dims of the rotated part that turn, in adjacent pairs
    base: float
    scaling: dict | None     # {"factor", "original", "fast", "slow"} or None


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                 # unrotated query/key dims per head
    rot_dim: int             # rotated query/key dims per head (the key's are shared by all heads)
    vdim: int
    kv_rank: int             # width of the cached latent
    scale: float             # multiplies q . k
    rot: RotationConfig
    kv_from: int | None      # the layer whose cached latent and key part this layer reads (None: its own)


@dataclass(frozen=True)
class Mamba1Config:
    inner: int
    state: int
    dt_rank: int
    conv: int


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int


@dataclass(frozen=True)
class MoeFFConfig:
    ff: int                  # an expert's intermediate width
    experts: int
    top: int
    groups: int
    keep: int
    scale: float


@dataclass(frozen=True)
class MuvoraxLayerConfig:
    type: str
    mixer: LightningConfig | LatentAttentionConfig | Mamba1Config
    mlp: DenseFFConfig | MoeFFConfig | None


@dataclass(frozen=True)
class MuvoraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[MuvoraxLayerConfig, ...]
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    def to_json_dict(self) -> dict:
        """The config.json that reads back as this record."""
        def mixer(l):
            m = l.mixer
            if l.type == "lightning":
                return {"decay": list(m.decay), "dim": m.dim, "heads": m.heads, "vdim": m.vdim}
            if l.type == "mamba1":
                return {"conv": m.conv, "dt_rank": m.dt_rank, "inner": m.inner, "state": m.state}
            rot = {"base": m.rot.base, "dims": m.rot.dims}
            if m.rot.scaling is not None:
                rot["scaling"] = dict(m.rot.scaling)
            out = {"dim": m.dim, "heads": m.heads, "kv_rank": m.kv_rank, "rot": rot, "rot_dim": m.rot_dim, "scale": m.scale,
                   "vdim": m.vdim}
            if m.kv_from is not None:
                out["kv_from"] = m.kv_from
            return out

        def mlp(f):
            if f is None:
                return None
            if isinstance(f, DenseFFConfig):
                return {"ff": f.ff, "kind": "dense"}
            return {"expert": {"ff": f.ff}, "kind": "moe",
                    "router": {"experts": f.experts, "groups": {"count": f.groups, "keep": f.keep}, "scale": f.scale, "top": f.top}}
        return {"architecture": self.architecture,
                "layers": [{"mixer": mixer(l), "mlp": mlp(l.mlp), "type": l.type} for l in self.layers],
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "MuvoraxConfig":
        r = KeyReader(raw, where)
        name = r.string("architecture", default=None)
        if name is None:
            archs = r.any("architectures")
            if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
                raise ConfigError(f"{where}: 'architecture' must name the model")
            name = archs[0]
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = KeyReader(_obj(r, "norm", where), where + ":norm").number("eps", positive=True)
        entries = r.any("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{where}: 'layers' must be a list with an entry per layer")
        layers = tuple(_layer(e, f"{where}:layers[{i}]") for i, e in enumerate(entries))
        for i, l in enumerate(layers):
            src = l.mixer.kv_from if l.type == "latent_attention" else None
            if src is None:
                continue
            at = f"{where}:layers[{i}]:mixer"
            if not 0 <= src < i or layers[src].type != "latent_attention" or layers[src].mixer.kv_from is not None:
                raise ConfigError(f"{at}: 'kv_from' ({src}) must name an earlier latent_attention layer with a cache of its own")
            a, b = l.mixer, layers[src].mixer
            if (a.kv_rank, a.rot_dim, a.rot) != (b.kv_rank, b.rot_dim, b.rot):
                raise ConfigError(f"{at}: kv_rank, rot_dim and rot must equal those of layer {src}, whose cache it reads")
        return cls(name, vocab, width, eps, layers, raw)


def _obj(r: KeyReader, key: str, where: str) -> dict:
    v = r.any(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object")
    return v


def _layer(e, where: str) -> MuvoraxLayerConfig:
    r = KeyReader(e, where)
    kind = r.string("type", choices=LAYER_TYPES)
    mw = where + ":mixer"
    m = KeyReader(_obj(r, "mixer", where), mw)
    if kind == "lightning":
        decay = m.any("decay")
        heads = m.integer("heads", minimum=1)
        if not isinstance(decay, list) or len(decay) != heads or any(isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
            raise ConfigError(f"{mw}: 'decay' must list one number per head ({heads})")
        if any(not 0.0 <= float(g) <= 1.0 for g in decay):
            raise ConfigError(f"{mw}: every 'decay' lies in 0..1")
        mixer = LightningConfig(heads, m.integer("dim", minimum=1), m.integer("vdim", minimum=1), tuple(float(g) for g in decay))
    elif kind == "mamba1":
        mixer = Mamba1Config(m.integer("inner", minimum=1), m.integer("state", minimum=1), m.integer("dt_rank", minimum=1),
                             m.integer("conv", minimum=1))
    else:
        rw = mw + ":rot"
        rot = KeyReader(_obj(m, "rot", mw), rw)
        scaling = rot.any("scaling")
        if scaling is not None:
            s = KeyReader(scaling, rw + ":scaling")
            scaling = {"factor": s.number("factor", positive=True), "fast": s.number("fast", positive=True),
                       "original": s.number("original", positive=True), "slow": s.number("slow", positive=True)}
        rotation = RotationConfig(rot.integer("dims", minimum=0), rot.number("base", positive=True), scaling)
        mixer = LatentAttentionConfig(m.integer("heads", minimum=1), m.integer("dim", minimum=1), m.integer("rot_dim", minimum=0),
                                      m.integer("vdim", minimum=1), m.integer("kv_rank", minimum=1), m.number("scale"), rotation,
                                      m.integer("kv_from", default=None, minimum=0))
        if rotation.dims % 2 or rotation.dims > mixer.rot_dim:
            raise ConfigError(f"{rw}: 'dims' ({rotation.dims}) must be even and at most rot_dim ({mixer.rot_dim})")
    mlp = r.any("mlp")
    ff = None
    if mlp is not None:
        fw = where + ":mlp"
        f = KeyReader(mlp, fw)
        if f.string("kind", choices=("dense", "moe")) == "dense":
            ff = DenseFFConfig(f.integer("ff", minimum=1))
        else:
            ro = KeyReader(_obj(f, "router", fw), fw + ":router")
            groups = ro.any("groups")
            g = KeyReader(groups, fw + ":router:groups") if groups is not None else None
            ff = MoeFFConfig(KeyReader(_obj(f, "expert", fw), fw + ":expert").integer("ff", minimum=1),
                             ro.integer("experts", minimum=1), ro.integer("top", minimum=1),
                             g.integer("count", minimum=1) if g else 1, g.integer("keep", minimum=1) if g else 1,
                             ro.number("scale", default=1.0))
            if ff.experts % ff.groups or ff.keep > ff.groups or ff.top > ff.keep * (ff.experts // ff.groups):
                raise ConfigError(f"{fw}:router: {ff.experts} experts in {ff.groups} groups, {ff.keep} kept, cannot give {ff.top} a token")
    return MuvoraxLayerConfig(kind, mixer, ff)
