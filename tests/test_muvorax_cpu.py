"""What of the Muvorax decoder needs no GPU: its configuration, its layout, tensor names, cache
units and schedule, the rotation's rescaled table, and the plain statement against second
statements of the same formulas."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_muvorax as plain
from scriptling_llm_lib_b200 import models  # noqa: F401
from scriptling_llm_lib_b200.config.base import ConfigError
from scriptling_llm_lib_b200.config.registry import architecture_for, architecture_name
from scriptling_llm_lib_b200.engine.model import DecoderModel

YARN = {"factor": 4.0, "fast": 16.0, "original": 64, "slow": 2.0}
RAW = {
    "architecture": "Muvorax", "norm": {"eps": 1e-5}, "vocab": 90, "width": 48,
    "layers": [
        {"type": "latent_attention", "mlp": {"ff": 64, "kind": "dense"},
         "mixer": {"dim": 8, "heads": 3, "kv_rank": 20, "rot": {"base": 300.0, "dims": 4, "scaling": YARN}, "rot_dim": 4, "scale": 0.3, "vdim": 12}},
        {"type": "mamba1", "mlp": None, "mixer": {"conv": 3, "dt_rank": 5, "inner": 40, "state": 6}},
        {"type": "lightning", "mixer": {"decay": [0.5, 0.99], "dim": 8, "heads": 2, "vdim": 16},
         "mlp": {"expert": {"ff": 24}, "kind": "moe", "router": {"experts": 6, "groups": {"count": 3, "keep": 2}, "scale": 1.5, "top": 2}}},
        {"type": "latent_attention", "mlp": None,
         "mixer": {"dim": 6, "heads": 5, "kv_from": 0, "kv_rank": 20, "rot": {"base": 300.0, "dims": 4, "scaling": YARN}, "rot_dim": 4,
                   "scale": 0.2, "vdim": 10}},
    ],
}


def test_the_configuration_reads_back_and_names_the_model():
    arch = architecture_for(architecture_name(RAW))
    cfg = arch.config_class.from_dict(RAW)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (90, 48, 1e-5)
    assert [l.type for l in cfg.layers] == ["latent_attention", "mamba1", "lightning", "latent_attention"]
    a = cfg.layers[0].mixer
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.scale, a.kv_from, a.rot.dims, a.rot.base) == (3, 8, 4, 12, 20, 0.3, None, 4, 300.0)
    assert cfg.layers[3].mixer.kv_from == 0 and cfg.layers[1].mlp is None and cfg.layers[0].mlp.ff == 64
    e = cfg.layers[2].mlp
    assert (e.ff, e.experts, e.top, e.groups, e.keep, e.scale) == (24, 6, 2, 3, 2, 1.5)
    assert cfg.layers[2].mixer.decay == (0.5, 0.99)
    assert arch.config_class.from_dict(cfg.to_json_dict()) == cfg
    assert cfg.to_json_dict() == RAW


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "gru", "type"), (("layers", 2, "mixer", "decay"), [0.5], "decay"),
    (("layers", 2, "mixer", "decay"), [0.5, 1.5], "decay"), (("layers", 3, "mixer", "kv_from"), 1, "kv_from"),
    (("layers", 3, "mixer", "kv_from"), 3, "kv_from"), (("layers", 3, "mixer", "kv_rank"), 24, "kv_rank"),
    (("layers", 0, "mixer", "rot", "dims"), 3, "dims"), (("layers", 2, "mlp", "router", "top"), 5, "experts"),
    (("layers", 2, "mlp", "router", "groups", "count"), 4, "groups"), (("layers", 2, "mlp", "kind"), "glu", "kind"),
    (("layers",), [], "layers"), (("norm",), 3, "norm"),
])
def test_a_wrong_configuration_names_its_key(path, value, word):
    raw = copy.deepcopy(RAW)
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        architecture_for("Muvorax").config_class.from_dict(raw)
    assert word in str(e.value)


def test_the_layout_asks_for_every_tensor_once_and_shares_a_cache_unit():
    arch = architecture_for("Muvorax")
    lay = arch.layout(arch.config_class.from_dict(RAW))
    m = DecoderModel(lay)
    specs = {s.name: tuple(s.shape) for s in m.tensor_specs()}
    assert specs["embed"] == (90, 48) and "head" not in specs
    assert specs["l0.mix.q"] == (3 * 12, 48) and specs["l0.mix.dkv"] == (24, 48) and specs["l0.mix.dkv.norm"] == (20,)
    assert specs["l0.mix.uk"] == (24, 20) and specs["l0.mix.uv"] == (36, 20) and specs["l0.mix.o"] == (48, 36)
    assert "l3.mix.dkv" not in specs and "l3.mix.dkv.norm" not in specs and specs["l3.mix.uk"] == (30, 20)
    assert specs["l1.mix.in"] == (80, 48) and specs["l1.mix.conv"] == (40, 3) and specs["l1.mix.x"] == (5 + 12, 40)
    assert specs["l1.mix.dt"] == (40, 5) and specs["l1.mix.A_log"] == (40, 6) and specs["l1.mix.D"] == (40,)
    assert specs["l2.mix.q"] == (16, 48) and specs["l2.mix.v"] == (32, 48) and specs["l2.mix.norm"] == (32,)
    assert specs["l2.mlp.router"] == (6, 48) and specs["l2.mlp.correction"] == (6,) and specs["l2.mlp.e5.down"] == (48, 24)
    assert specs["l0.norm1.alpha"] == () and specs["l0.norm2b.b"] == (48,) and "l1.norm2" not in specs and specs["final.norm"] == (48,)
    assert [(e.layer, e.cache_unit, e.writes_cache) for e in lay.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False)]
    needs = m.cache_needs()
    assert needs[0].kv_heads == 1 and needs[0].head_dim == 24 and needs[0].value_dim == 0 and needs[1] is None
    states = m.state_needs()
    assert states[0] is None and set(states[1]) == {"S", "conv"} and states[1]["S"].shape == (40, 6) and states[1]["conv"].shape == (2, 40)
    assert states[2]["S"].shape == (2, 8, 16) and 3 not in states
    assert m.graph_safe()


def test_the_rescaled_rotation_table_against_values_worked_by_hand():
    from scriptling_llm_lib_b200.parts.rotary import RotaryEncoding, YarnScaling
    dims, base = 8, 100.0
    enc = RotaryEncoding(8, dims, base, YarnScaling(4.0, 64.0, 16.0, 2.0), "interleaved")
    # index(t) = 8 ln(64 / (2 pi t)) / (2 ln 100): fast 16 -> -0.39 -> lo 0; slow 2 -> 1.41 -> hi 2
    f = [100.0 ** (-2 * i / 8) for i in range(4)]
    ramp = [0.0, 0.5, 1.0, 1.0]
    want = [fi / 4.0 * r + fi * (1 - r) for fi, r in zip(f, ramp)]
    assert np.allclose(enc.inv_freq, want, rtol=1e-12)
    assert abs(enc.amplitude - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    pf, mult = plain.yarn_frequencies(dims, base, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0})
    assert np.allclose(pf, want, rtol=1e-12) and abs(mult - enc.amplitude) < 1e-12
    enc.prepare(10, "cpu")
    t = enc.cos_sin
    assert abs(float(t[3, 1, 0]) - enc.amplitude * math.cos(3 * want[1])) < 1e-6
    assert abs(float(t[3, 1, 1]) - enc.amplitude * math.sin(3 * want[1])) < 1e-6


def _weights(seed=0):
    arch = architecture_for("Muvorax")
    specs = DecoderModel(arch.layout(arch.config_class.from_dict(RAW))).tensor_specs()
    g = torch.Generator().manual_seed(seed)
    return {s.name: (torch.randn(s.shape, generator=g) * 0.3 + (1.0 if s.init in ("norm_weight", "slope") else 0.0)).double() for s in specs}


def test_plain_linear_attention_is_attention_with_decayed_scores():
    W = _weights()
    c = RAW["layers"][2]["mixer"]
    h = torch.randn(9, 48, dtype=torch.float64)
    got = plain.lightning(h, W, "l2.mix.", c, 1e-5)
    T, H, D, V = 9, 2, 8, 16
    q = plain.silu(h @ W["l2.mix.q"].T).view(T, H, D)
    k = plain.silu(h @ W["l2.mix.k"].T).view(T, H, D)
    v = plain.silu(h @ W["l2.mix.v"].T).view(T, H, V)
    o = torch.zeros(T, H, V, dtype=torch.float64)
    for hd in range(H):
        for i in range(T):
            for j in range(i + 1):
                o[i, hd] += c["decay"][hd] ** (i - j) * (q[i, hd] @ k[j, hd]) * v[j, hd]
    o = o.reshape(T, H * V)
    y = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5) * W["l2.mix.norm"] * torch.sigmoid(h @ W["l2.mix.g"].T)
    assert torch.allclose(got, y @ W["l2.mix.o"].T, rtol=1e-10, atol=1e-12)


def test_plain_latent_attention_equals_asking_the_latent_directly():
    """q . (Wuk c) = (Wuk^T q) . c and sum p (Wuv c) = Wuv (sum p c): the form the kernels use."""
    W = _weights(1)
    c = RAW["layers"][0]["mixer"]
    h = torch.randn(11, 48, dtype=torch.float64)
    got = plain.latent_attention(h, W, "l0.mix.", c, 1e-5)
    T, H, D, P, V, R = 11, 3, 8, 4, 12, 20
    lat, kr = plain.latent_pair(h, W, "l0.mix.", c, 1e-5)
    q = (h @ W["l0.mix.q"].T).view(T, H, D + P)
    qr = plain.rotate_pairs(q[..., D:], torch.arange(T), 4, 300.0, YARN)
    out = torch.zeros(T, H, V, dtype=torch.float64)
    for hd in range(H):
        wuk = W["l0.mix.uk"][hd * D:(hd + 1) * D]
        wuv = W["l0.mix.uv"][hd * V:(hd + 1) * V]
        for i in range(T):
            s = ((q[i, hd, :D] @ wuk) @ lat[:i + 1].T + qr[i, hd] @ kr[:i + 1].T) * 0.3
            out[i, hd] = wuv @ (torch.softmax(s, -1) @ lat[:i + 1])
    assert torch.allclose(got, out.reshape(T, H * V) @ W["l0.mix.o"].T, rtol=1e-9, atol=1e-12)


def test_plain_convolution_and_scan_against_second_statements():
    x = torch.randn(7, 5, dtype=torch.float64)
    w = torch.randn(5, 3, dtype=torch.float64)
    b = torch.randn(5, dtype=torch.float64)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T[None], (2, 0)), w[:, None, :], b, groups=5)[0].T
    assert torch.allclose(plain.causal_conv(x, w, b), want, atol=1e-12)
    # the scan with a constant step and one state: a geometric sum
    W = {"m.in": torch.zeros(2, 3, dtype=torch.float64), "m.conv": torch.ones(1, 1, dtype=torch.float64), "m.conv.b": torch.zeros(1, dtype=torch.float64),
         "m.x": torch.zeros(3, 1, dtype=torch.float64), "m.dt": torch.zeros(1, 1, dtype=torch.float64), "m.dt.b": torch.tensor([0.3], dtype=torch.float64),
         "m.A_log": torch.tensor([[0.1]], dtype=torch.float64), "m.D": torch.tensor([2.0], dtype=torch.float64), "m.o": torch.ones(1, 1, dtype=torch.float64)}
    got = plain.mamba1(torch.zeros(4, 3, dtype=torch.float64), W, "m.", {"inner": 1, "state": 1, "dt_rank": 1})
    assert torch.allclose(got, torch.zeros(4, 1, dtype=torch.float64))      # x = silu(0) = 0 all the way


def test_plain_router_keeps_to_the_best_groups_and_weighs_without_the_correction():
    W = {"r.router": torch.eye(6, dtype=torch.float64), "r.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 5.0], dtype=torch.float64)}
    h = torch.tensor([[3.0, 2.9, 0.0, 0.0, 2.0, -4.0]], dtype=torch.float64)
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    idx, w = plain.route(h, W, "r.", r)
    # groups (0,1) (2,3) (4,5): the correction lifts expert 5 and with it its group above group 0
    assert set(idx[0].tolist()) == {4, 5}
    s = torch.sigmoid(h[0])
    assert torch.allclose(w[0].sum(), torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(w[0, idx[0].tolist().index(5)], 2.0 * s[5] / (s[4] + s[5]))      # weighed by the plain score
    r["groups"] = {"count": 3, "keep": 2}
    idx, w = plain.route(h, W, "r.", r)
    assert set(idx[0].tolist()) == {0, 5}             # groups 2 and 0 are kept; chosen by the corrected score
    assert torch.allclose(w[0, idx[0].tolist().index(5)], 2.0 * s[5] / (s[0] + s[5]))
    r["groups"] = {"count": 1, "keep": 1}
    r["top"] = 3
    idx, w = plain.route(h, W, "r.", r)
    assert set(idx[0].tolist()) == {5, 0, 1}
