"""SozilixConfig: the sizes, constants and order of layers of a Sozilix decoder, from config.json.

The file is nested: `layers` is a list whose entries give the layer's `type` (which mixer: two
side by side, attention over a window and a gated delta rule, or a gated linear recurrence), the
mixer's sizes under `mixer`, and its feed-forward under `mlp` (null: none). Model-wide: `vocab`,
`width`, `norm.eps`, `residual_mult`, `canon.taps` (the short convolution in front of every mixer).
Nothing about a model of this family is written anywhere else: tensors' shapes follow from these.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

LAYER_TYPES = ("parallel", "rglru")


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                 # width of a query/key head
    vdim: int                # width of a value head
    window: int              # keys visible to a query: its own position and the window - 1 positions behind it
    rot_dims: int            # leading dims of a head that are rotated, in adjacent pairs
    rot_base: float
    scale: float             # multiplies q . k


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int
    kv_heads: int            # query/key heads
    dim: int
    vdim: int
    conv: int                # taps of the short convolutions on q, k, v


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: DeltaRuleConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class RGLRUConfig:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int


@dataclass(frozen=True)
class SozilixLayerConfig:
    type: str
    mixer: ParallelMixerConfig | RGLRUConfig
    mlp: DenseFFConfig | None


@dataclass(frozen=True)
class SozilixConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    canon_taps: int
    layers: tuple[SozilixLayerConfig, ...]
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    def to_json_dict(self) -> dict:
        """The config.json that reads back as this record."""
        def mixer(l):
            m = l.mixer
            if l.type == "rglru":
                return {"blocks": m.blocks, "conv": m.conv, "width": m.width}
            a, d = m.left, m.right
            return {"left": {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "mask": {"size": a.window},
                             "rot": {"base": a.rot_base, "dims": a.rot_dims}, "scale": a.scale, "vdim": a.vdim},
                    "left_scale": m.left_scale,
                    "right": {"conv": d.conv, "dim": d.dim, "heads": d.heads, "kv_heads": d.kv_heads, "vdim": d.vdim},
                    "right_scale": m.right_scale}
        return {"architecture": self.architecture, "canon": {"taps": self.canon_taps},
                "layers": [{"mixer": mixer(l), "mlp": None if l.mlp is None else {"ff": l.mlp.ff, "kind": "dense"}, "type": l.type}
                           for l in self.layers],
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "SozilixConfig":
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
        mult = r.number("residual_mult", default=1.0)
        taps = KeyReader(_obj(r, "canon", where), where + ":canon").integer("taps", minimum=1)
        entries = r.any("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{where}: 'layers' must be a list with an entry per layer")
        layers = tuple(_layer(e, f"{where}:layers[{i}]") for i, e in enumerate(entries))
        return cls(name, vocab, width, eps, mult, taps, layers, raw)


def _obj(r: KeyReader, key: str, where: str) -> dict:
    v = r.any(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object")
    return v


def _layer(e, where: str) -> SozilixLayerConfig:
    r = KeyReader(e, where)
    kind = r.string("type", choices=LAYER_TYPES)
    m = KeyReader(_obj(r, "mixer", where), where + ":mixer")
    if kind == "rglru":
        mixer = RGLRUConfig(m.integer("width", minimum=1), m.integer("blocks", minimum=1), m.integer("conv", minimum=1))
        if mixer.width % mixer.blocks:
            raise ConfigError(f"{where}: a width of {mixer.width} cannot be cut into {mixer.blocks} equal blocks")
    else:
        a = KeyReader(_obj(m, "left", where + ":mixer"), where + ":mixer:left")
        rot = KeyReader(_obj(a, "rot", a.where), a.where + ":rot")
        mask = KeyReader(_obj(a, "mask", a.where), a.where + ":mask")
        left = WindowAttentionConfig(a.integer("heads", minimum=1), a.integer("kv_heads", minimum=1), a.integer("dim", minimum=1),
                                     a.integer("vdim", minimum=1), mask.integer("size", minimum=1), rot.integer("dims", minimum=0),
                                     rot.number("base", positive=True), a.number("scale"))
        if left.heads % left.kv_heads:
            raise ConfigError(f"{a.where}: heads ({left.heads}) must be a multiple of kv_heads ({left.kv_heads})")
        if left.rot_dims % 2 or left.rot_dims > left.dim:
            raise ConfigError(f"{a.where}: rot.dims ({left.rot_dims}) must be even and at most dim ({left.dim})")
        d = KeyReader(_obj(m, "right", where + ":mixer"), where + ":mixer:right")
        right = DeltaRuleConfig(d.integer("heads", minimum=1), d.integer("kv_heads", minimum=1), d.integer("dim", minimum=1),
                                d.integer("vdim", minimum=1), d.integer("conv", minimum=1))
        if right.heads % right.kv_heads:
            raise ConfigError(f"{d.where}: heads ({right.heads}) must be a multiple of kv_heads ({right.kv_heads})")
        mixer = ParallelMixerConfig(left, right, m.number("left_scale", default=1.0), m.number("right_scale", default=1.0))
    mlp = r.any("mlp")
    ff = None
    if mlp is not None:
        f = KeyReader(mlp, where + ":mlp")
        f.string("kind", default="dense", choices=("dense",))
        ff = DenseFFConfig(f.integer("ff", minimum=1))
    return SozilixLayerConfig(kind, mixer, ff)
