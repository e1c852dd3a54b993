"""Layout of the Sozilix decoder: which parts, with which numbers and tensor names.

Every layer is x += m * mixer(c(norm1(x))) and, where it has a feed-forward, x += m *
ff(norm2(x)): layer norms with a weight and no bias, m the model's residual multiplier, c the
short causal convolution with its input added back (`l<i>.canon1`). The mixer is either two side by
side on the same input (`l<i>.mix.left.*`: grouped-query softmax attention over a sliding window,
queries and keys partly rotated in adjacent pairs, values of their own width divided by their root
mean square before they are cached; `l<i>.mix.right.*`: the gated delta rule), added with a
coefficient each, or a gated linear recurrence (`l<i>.mix.*`). The feed-forward is the SiLU-gated
one. A final layer norm (`final.norm`) and an untied head (`head`) follow; the embedding is `embed`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sozilix import SozilixConfig
from ..engine.layout import ModelLayout, sequential_schedule
from ..parts.base import PartSpec
from ..parts.block import LayerSpec
from ..parts.embedding import linear_head, token_embedding

MAX_POSITIONS = 1 << 20      # the family states no longest sequence; the cache's size bounds it


def _norm(cfg: SozilixConfig, name: str, out_dtype=None) -> PartSpec:
    return PartSpec("weighted_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=name, center=True, out_dtype=out_dtype))


def _mixer(cfg: SozilixConfig, layer, p: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "rglru":
        return PartSpec("rglru", dict(
            hidden=cfg.width, width=m.width, blocks=m.blocks, conv_taps=m.conv, y_name=p + "y", y_bias_name=p + "y.b",
            x_name=p + "x", x_bias_name=p + "x.b", conv_name=p + "conv", conv_bias_name=p + "conv.b", ra_name=p + "ra",
            ra_bias_name=p + "ra.b", ri_name=p + "ri", ri_bias_name=p + "ri.b", lam_name=p + "lam", o_name=p + "o"))
    a, d = m.left, m.right
    la, ra = p + "left.", p + "right."
    position = PartSpec("rotary", dict(head_dim=a.dim, rotary_dim=a.rot_dims, theta=a.rot_base, scaling=None,
                                       pairing="interleaved")) if a.rot_dims >= 2 else None
    left = PartSpec("attention", dict(
        hidden=cfg.width, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim, v_dim=a.vdim, position=position,
        window=a.window, scale=a.scale, value_norm_eps=cfg.norm_eps, q_name=la + "q", k_name=la + "k", v_name=la + "v",
        o_name=la + "o"))
    right = PartSpec("gated_delta_rule", dict(
        hidden=cfg.width, n_heads=d.heads, n_kv_heads=d.kv_heads, key_dim=d.dim, value_dim=d.vdim, conv_taps=d.conv,
        norm_eps=cfg.norm_eps, q_name=ra + "q", k_name=ra + "k", v_name=ra + "v", q_conv_name=ra + "q.conv",
        k_conv_name=ra + "k.conv", v_conv_name=ra + "v.conv", beta_name=ra + "b", decay_name=ra + "a", a_log_name=ra + "A_log",
        dt_bias_name=ra + "dt_bias", gate_name=ra + "g", norm_name=ra + "norm", o_name=ra + "o"))
    return PartSpec("parallel", dict(branches=[("left", left, m.left_scale), ("right", right, m.right_scale)]))


def sozilix_layout(cfg: SozilixConfig) -> ModelLayout:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": _norm(cfg, p + "norm1", out_dtype="float32"), "mixer": _mixer(cfg, layer, p + "mix.")}
        if layer.mlp is not None:
            parts["feed_forward_norm"] = _norm(cfg, p + "norm2")
            parts["feed_forward"] = PartSpec("swiglu", dict(hidden=cfg.width, intermediate=layer.mlp.ff, gate_name=p + "mlp.gate",
                                                            up_name=p + "mlp.up", down_name=p + "mlp.down"))
        layers.append(LayerSpec("scaled_pre_norm", parts, dict(
            residual_scale=cfg.residual_mult, input_conv=dict(name=p + "canon1", channels=cfg.width, taps=cfg.canon_taps))))
    return ModelLayout(
        vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=MAX_POSITIONS,
        embedding=token_embedding(cfg.vocab, cfg.width, "embed"), layers=tuple(layers),
        schedule=sequential_schedule(len(layers)), final_norm=_norm(cfg, "final.norm"),
        head=linear_head(cfg.vocab, cfg.width, "head"))


register_architecture("Sozilix", SozilixConfig, sozilix_layout)
