"""What of the Sozilix decoder needs no GPU: its configuration, its layout and tensor names, the
cache's per-sequence state under names, values of a width of their own, and the plain statement
against second statements of the same formulas."""
import copy

import pytest
import torch

import plain_sozilix as plain
from scriptling_llm_lib_b200 import models  # noqa: F401
from scriptling_llm_lib_b200.cache import CacheNeed, SequenceCache, StateNeed
from scriptling_llm_lib_b200.config.base import ConfigError
from scriptling_llm_lib_b200.config.registry import architecture_for, architecture_name
from scriptling_llm_lib_b200.engine.model import DecoderModel

RAW = {
    "architecture": "Sozilix", "canon": {"taps": 3}, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "vocab": 90, "width": 48,
    "layers": [
        {"type": "rglru", "mixer": {"width": 36, "blocks": 3, "conv": 2}, "mlp": {"ff": 64, "kind": "dense"}},
        {"type": "parallel", "mlp": None, "mixer": {
            "left": {"dim": 16, "heads": 6, "kv_heads": 2, "mask": {"size": 11}, "rot": {"base": 300.0, "dims": 4}, "scale": 0.2, "vdim": 8},
            "left_scale": 0.6, "right": {"conv": 4, "dim": 8, "heads": 4, "kv_heads": 2, "vdim": 12}, "right_scale": 1.2}},
    ],
}


def test_the_configuration_reads_back_and_names_the_model():
    arch = architecture_for(architecture_name(RAW))
    cfg = arch.config_class.from_dict(RAW)
    assert (cfg.vocab, cfg.width, cfg.canon_taps, cfg.residual_mult, cfg.norm_eps) == (90, 48, 3, 0.5, 1e-6)
    assert [l.type for l in cfg.layers] == ["rglru", "parallel"]
    assert cfg.layers[0].mlp.ff == 64 and cfg.layers[1].mlp is None
    left = cfg.layers[1].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.window, left.rot_dims, left.rot_base, left.scale) == \
        (6, 2, 16, 8, 11, 4, 300.0, 0.2)
    assert arch.config_class.from_dict(cfg.to_json_dict()) == cfg
    assert architecture_name({"architectures": ["LlamaForCausalLM"]}) == "LlamaForCausalLM"
    with pytest.raises(ConfigError):
        architecture_name({})


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "lstm", "type"), (("layers", 0, "mixer", "blocks"), 5, "blocks"),
    (("layers", 1, "mixer", "left", "kv_heads"), 4, "kv_heads"), (("layers", 1, "mixer", "left", "rot", "dims"), 5, "rot.dims"),
    (("canon",), 3, "canon"), (("layers", 1, "mixer", "right", "kv_heads"), 3, "kv_heads"), (("layers",), [], "layers"),
])
def test_a_wrong_configuration_names_its_key(path, value, word):
    raw = copy.deepcopy(RAW)
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        architecture_for("Sozilix").config_class.from_dict(raw)
    assert word in str(e.value)


def test_the_layout_asks_for_every_tensor_once_and_for_state_and_cache_by_layer():
    arch = architecture_for("Sozilix")
    m = DecoderModel(arch.layout(arch.config_class.from_dict(RAW)))
    shapes = {s.name: tuple(s.shape) for s in m.tensor_specs()}
    assert shapes["embed"] == (90, 48) and shapes["head"] == (90, 48) and shapes["final.norm"] == (48,)
    assert shapes["l0.canon1"] == (48, 3) and shapes["l1.canon1"] == (48, 3) and "l1.norm2" not in shapes
    assert shapes["l0.mix.ra"] == (3, 12, 12) and shapes["l0.mix.conv"] == (36, 2) and shapes["l0.mix.o"] == (48, 36)
    assert shapes["l1.mix.left.q"] == (96, 48) and shapes["l1.mix.left.k"] == (32, 48) and shapes["l1.mix.left.v"] == (16, 48)
    assert shapes["l1.mix.left.o"] == (48, 48)
    assert shapes["l1.mix.right.q"] == (16, 48) and shapes["l1.mix.right.v"] == (48, 48) and shapes["l1.mix.right.v.conv"] == (48, 4)
    assert shapes["l1.mix.right.b"] == (4, 48) and shapes["l1.mix.right.A_log"] == (4,) and shapes["l1.mix.right.norm"] == (12,)
    needs = m.cache_needs()
    assert needs[0] is None and needs[1] == CacheNeed("window", 2, 16, 11, v_dim=8)
    st = m.state_needs()
    assert st[0]["input_conv"].shape == (2, 48) and st[0]["mixer"]["S"].shape == (36,) and st[0]["mixer"]["conv"].shape == (1, 36)
    assert st[1]["mixer"]["right"]["S"].shape == (4, 8, 12) and st[1]["mixer"]["right"]["conv"].shape == (3, 16 + 16 + 48)
    assert m.graph_safe()


def test_the_cache_keeps_named_state_per_slot_and_values_of_their_own_width():
    needs = {0: CacheNeed("window", 2, 16, 11, v_dim=8), 1: None}
    states = {0: {"a": StateNeed((3,)), "deep": {"b": StateNeed((2, 2), torch.float32)}}, 1: StateNeed((5,))}
    c = SequenceCache(needs, states, n_slots=2, n_pages=4, dtype=torch.float32, device="cpu")
    assert c.groups[0].k.shape == (1, 5, 2, 64, 16) and c.groups[0].v.shape == (1, 5, 2, 64, 8)
    s0 = c.open()
    c.state[0]["a"][s0] += 1
    c.state[0]["deep"]["b"][s0] += 2
    c.state[1][s0] += 3
    s1 = c.open()
    c.state[0]["a"][s1] += 5
    c.close(s0)
    again = c.open()
    assert again == s0
    assert float(c.state[0]["a"][again].abs().sum()) == 0 and float(c.state[0]["deep"]["b"][again].abs().sum()) == 0
    assert float(c.state[1][again].abs().sum()) == 0 and float(c.state[0]["a"][s1].sum()) == 15


# ------------------------------------------------------------------ the plain statement against second statements
def test_plain_convolution_is_torch_s_padded_convolution():
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(19, 5, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T[None], (3, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(plain.causal_conv(x, w), ref, atol=1e-12)


def test_plain_norm_rotation_and_activations():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, 10, generator=g, dtype=torch.float64)
    w = torch.randn(10, generator=g, dtype=torch.float64)
    assert torch.allclose(plain.layer_norm(x, w, 1e-5), torch.nn.functional.layer_norm(x, (10,), w, None, 1e-5), atol=1e-12)
    assert torch.allclose(plain.gelu_tanh(x), torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-12)
    assert torch.allclose(plain.softplus(x * 20), torch.nn.functional.softplus(x * 20), atol=1e-9)
    q = torch.randn(6, 2, 8, generator=g, dtype=torch.float64)
    pos = torch.arange(3, 9)
    r = plain.rotate_interleaved(q, pos, 4, 100.0)
    assert torch.allclose(r[..., 4:], q[..., 4:]) and torch.allclose((r ** 2).sum(-1), (q ** 2).sum(-1))
    # a rotation makes scores depend on the distance only
    a = plain.rotate_interleaved(q[:1], torch.tensor([5]), 4, 100.0)[0, 0] @ plain.rotate_interleaved(q[1:2], torch.tensor([2]), 4, 100.0)[0, 0]
    b = plain.rotate_interleaved(q[:1], torch.tensor([13]), 4, 100.0)[0, 0] @ plain.rotate_interleaved(q[1:2], torch.tensor([10]), 4, 100.0)[0, 0]
    assert abs(float(a - b)) < 1e-12


def test_plain_delta_rule_in_its_closed_form_for_two_tokens():
    """After two writes along orthogonal unit keys the state is decay * k1 (b1 v1)^T + k2 (b2 v2)^T."""
    c = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "conv": 1}
    g = torch.Generator().manual_seed(2)
    W = {n: torch.randn(s, generator=g, dtype=torch.float64) for n, s in {
        "q": (4, 6), "k": (4, 6), "v": (3, 6), "b": (1, 6), "a": (1, 6), "g": (3, 6), "o": (6, 3), "A_log": (1,), "dt_bias": (1,),
        "norm": (3,)}.items()}
    for n in ("q", "k", "v"):
        W[n + ".conv"] = torch.ones((W[n].shape[0], 1), dtype=torch.float64)
    h = torch.randn(2, 6, generator=g, dtype=torch.float64)
    out = plain.gated_delta(h, W, "", c, 1e-6)
    unit = lambda x: x / torch.sqrt((x * x).sum() + 1e-6)
    q = [unit(plain.silu(h[t] @ W["q"].T)) * 0.5 for t in range(2)]
    k = [unit(plain.silu(h[t] @ W["k"].T)) for t in range(2)]
    v = [plain.silu(h[t] @ W["v"].T) for t in range(2)]
    beta = [torch.sigmoid(h[t] @ W["b"].T) for t in range(2)]
    dec = [torch.exp(-torch.exp(W["A_log"]) * plain.softplus(h[t] @ W["a"].T + W["dt_bias"])) for t in range(2)]
    S1 = torch.outer(k[0], beta[0] * v[0])
    S2 = dec[1] * S1 + torch.outer(k[1], beta[1] * (v[1] - (dec[1] * S1).T @ k[1]))
    o = torch.stack([S1.T @ q[0], S2.T @ q[1]])
    want = (plain.rms_unit(o, 1e-6) * W["norm"] * plain.silu(h @ W["g"].T)) @ W["o"].T
    assert torch.allclose(out, want, atol=1e-12)
