"""Layout of the Muvorax decoder: which parts, with which numbers and tensor names.

Every layer is x += norm1b(mixer(norm1(x))) and, where it has a feed-forward, x += norm2b(ff(norm2(x))):
a norm in front of and behind each sublayer, all of the kind without statistics
(tanh(alpha v) w + b; tensors `<name>`, `<name>.b`, `<name>.alpha`). The mixer (`l<i>.mix.*`) is linear
attention with a decay per head, softmax attention over a cached latent (a layer may read the latent
another layer cached: it then runs on that layer's cache unit without writing), or the selective
scan. The feed-forward (`l<i>.mlp.*`) is dense with the tanh form of gelu, or routed experts
(`e<j>.up`, `e<j>.down`, `router`, `correction`) with the square of relu. The embedding `embed` is
also the output head, behind the model's last norm `final.norm`.
"""
from __future__ import annotations

from ..config.muvorax import DenseFFConfig, MuvoraxConfig
from ..config.registry import register_architecture
from ..engine.layout import ModelLayout, ScheduleEntry
from ..parts.base import PartSpec
from ..parts.block import LayerSpec
from ..parts.embedding import linear_head, token_embedding
from ..parts.rotary import YarnScaling

MAX_POSITIONS = 1 << 20      # the family states no longest sequence; the cache's size bounds it


def _norm(cfg: MuvoraxConfig, name: str) -> PartSpec:
    return PartSpec("dynamic_tanh", dict(width=cfg.width, weight_name=name, bias_name=name + ".b", alpha_name=name + ".alpha"))


def _mixer(cfg: MuvoraxConfig, layer, p: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "lightning":
        return PartSpec("decay_linear_attention", dict(
            hidden=cfg.width, n_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, decay=list(m.decay), norm_eps=cfg.norm_eps,
            q_name=p + "q", k_name=p + "k", v_name=p + "v", gate_name=p + "g", norm_name=p + "norm", o_name=p + "o"))
    if layer.type == "mamba1":
        return PartSpec("selective_scan", dict(
            hidden=cfg.width, inner=m.inner, n_state=m.state, dt_rank=m.dt_rank, conv_taps=m.conv, in_name=p + "in",
            conv_name=p + "conv", conv_bias_name=p + "conv.b", x_name=p + "x", dt_name=p + "dt", dt_bias_name=p + "dt.b",
            a_log_name=p + "A_log", d_name=p + "D", o_name=p + "o"))
    position = None
    if m.rot.dims >= 2:
        s = m.rot.scaling
        scaling = YarnScaling(s["factor"], s["original"], s["fast"], s["slow"]) if s is not None else None
        position = PartSpec("rotary", dict(head_dim=m.rot_dim, rotary_dim=m.rot.dims, theta=m.rot.base, scaling=scaling,
                                           pairing="interleaved"))
    own = m.kv_from is None
    return PartSpec("latent_attention", dict(
        hidden=cfg.width, n_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, v_dim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
        position=position, norm_eps=cfg.norm_eps, q_name=p + "q", uk_name=p + "uk", uv_name=p + "uv", o_name=p + "o",
        dkv_name=p + "dkv" if own else None, dkv_norm_name=p + "dkv.norm" if own else None, shares_cache=not own))


def _feed_forward(cfg: MuvoraxConfig, f, p: str) -> PartSpec:
    if isinstance(f, DenseFFConfig):
        return PartSpec("act_feed_forward", dict(hidden=cfg.width, intermediate=f.ff, up_name=p + "up", down_name=p + "down",
                                                 act="gelu_tanh"))
    return PartSpec("routed_experts", dict(
        hidden=cfg.width, intermediate=f.ff, experts=f.experts, top=f.top, n_groups=f.groups, keep_groups=f.keep, scale=f.scale,
        router_name=p + "router", correction_name=p + "correction", up_names=[f"{p}e{j}.up" for j in range(f.experts)],
        down_names=[f"{p}e{j}.down" for j in range(f.experts)], act="relu_squared"))


def muvorax_layout(cfg: MuvoraxConfig) -> ModelLayout:
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, layer, p + "mix."),
                 "mixer_post_norm": _norm(cfg, p + "norm1b")}
        if layer.mlp is not None:
            parts.update(feed_forward_norm=_norm(cfg, p + "norm2"), feed_forward=_feed_forward(cfg, layer.mlp, p + "mlp."),
                         feed_forward_post_norm=_norm(cfg, p + "norm2b"))
        layers.append(LayerSpec("sandwich_norm", parts))
        src = layer.mixer.kv_from if layer.type == "latent_attention" else None
        schedule.append(ScheduleEntry(i, i, True) if src is None else ScheduleEntry(i, src, False))
    return ModelLayout(
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS,
        embedding=token_embedding(cfg.vocab, cfg.width, "embed"), layers=tuple(layers), schedule=tuple(schedule),
        final_norm=_norm(cfg, "final.norm"), head=linear_head(cfg.vocab, cfg.width, "embed", tied=True))


register_architecture("Muvorax", MuvoraxConfig, muvorax_layout)
