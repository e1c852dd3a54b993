"""A plain, slow statement of the Muvorax decoder in float64, one function per mechanism.

Nothing here is shared with the library: tensors come in as a dict name -> torch tensor, the
configuration as the parsed config.json, and every function works on one sequence given as a whole
([tokens, channels]) with explicit loops over time where the mechanism is a recurrence; there is no
cache and no carried state, so whatever the library does with portions, batches, pages and slots
has to agree with this.

Notation: x_t the residual stream at token t, h what a mixer reads, rows times W^T for a stored
[out, in] matrix. `rnd` (default: identity) is applied wherever a version of the library working in
a 16-bit type writes an activation to memory, so that the same functions give the rounding oracle.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

F64 = torch.float64


def ident(t):
    return t


def bf16_round(t):
    return t.to(torch.float32).to(torch.bfloat16).to(F64)


# --------------------------------------------------------------------------- small functions
def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dynamic_tanh(x, W, name):
    """tanh(alpha x) * w + b: a norm that takes no statistics of the row."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


# --------------------------------------------------------------------------- rotation
def yarn_frequencies(dims, base, scaling):
    """(frequency per pair, multiplier of cos and sin). Pair i has f_i = base^(-2i/dims); with a
    scaling, pairs that turn slowly are slowed down by `factor`, fast ones are kept, and a linear
    ramp over the pair index joins the two."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turns_to_index(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turns_to_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_to_index(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, dims, base, scaling=None):
    """x [T, ..., width]: the leading `dims` of the last axis are turned in adjacent pairs
    (2i, 2i+1) by positions * frequency_i; cos and sin carry the scaling's multiplier."""
    freq, mult = yarn_frequencies(dims, base, scaling)
    out = x.clone()
    shape = [x.shape[0]] + [1] * (x.dim() - 2)
    for i, f in enumerate(freq):
        a = positions.to(F64) * f
        c, s = (torch.cos(a) * mult).view(shape), (torch.sin(a) * mult).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# --------------------------------------------------------------------------- mixers
def lightning(h, W, pre, c, eps, rnd=ident):
    """Linear attention with a fixed decay per head: S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t,
    all of q, k, v through SiLU; the heads' outputs together are divided by their root mean square,
    weighted, gated by sigmoid(Wg h) and projected."""
    T = h.shape[0]
    H, D, V = c["heads"], c["dim"], c["vdim"]
    q = rnd(silu(h @ W[pre + "q"].T)).view(T, H, D)
    k = rnd(silu(h @ W[pre + "k"].T)).view(T, H, D)
    v = rnd(silu(h @ W[pre + "v"].T)).view(T, H, V)
    g = rnd(h @ W[pre + "g"].T)
    o = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=F64)
        decay = float(c["decay"][hd])
        for t in range(T):
            S = decay * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    y = rms_unit(o.reshape(T, H * V), eps) * W[pre + "norm"] * torch.sigmoid(g)
    return rnd(y) @ W[pre + "o"].T


def latent_pair(h, W, pre, c, eps, rnd=ident):
    """What a latent-attention layer keeps per position: the normed latent [T, kv_rank] and the
    rotated key part [T, rot_dim] that all heads share."""
    T = h.shape[0]
    R, P = c["kv_rank"], c["rot_dim"]
    d = rnd(h @ W[pre + "dkv"].T)
    lat = rnd(rms_unit(d[:, :R], eps) * W[pre + "dkv.norm"])
    rot = c["rot"]
    kr = rotate_pairs(d[:, R:R + P], torch.arange(T), rot["dims"], rot["base"], rot.get("scaling"))
    return lat, rnd(kr)


def latent_attention(h, W, pre, c, eps, shared=None, rnd=ident):
    """Causal softmax attention whose keys and values are made per head from a cached latent:
    k_h = [Wuk_h c | rotated part], v_h = Wuv_h c; queries [unrotated | rotated] per head.
    `shared`: the (latent, rotated key part) of another layer to use instead of this one's."""
    T = h.shape[0]
    H, D, P, V, R = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    lat, kr = shared if shared is not None else latent_pair(h, W, pre, c, eps, rnd)
    q = rnd(h @ W[pre + "q"].T).view(T, H, D + P)
    rot = c["rot"]
    q_rot = rotate_pairs(q[..., D:], torch.arange(T), rot["dims"], rot["base"], rot.get("scaling"))
    kn = (lat @ W[pre + "uk"].T).view(T, H, D)
    vv = (lat @ W[pre + "uv"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        s = (q[:, hd, :D] @ kn[:, hd].T + q_rot[:, hd] @ kr.T) * float(c["scale"])
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ vv[:, hd]
    return rnd(out.reshape(T, H * V)) @ W[pre + "o"].T


def causal_conv(x, w, bias=None):
    """y_t[c] = sum_j w[c, j] x_{t - taps + 1 + j}[c] (+ bias[c]); x before the start is zero."""
    T = x.shape[0]
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y if bias is None else y + bias


def mamba1(h, W, pre, c, rnd=ident):
    """Selective scan: per channel a state vector that decays by exp(dt A) and takes dt x B, read
    with C, plus a skip D x; dt, B, C are functions of the token."""
    T = h.shape[0]
    I, N, K = c["inner"], c["state"], c["dt_rank"]
    xz = rnd(h @ W[pre + "in"].T)
    x, z = xz[:, :I], xz[:, I:]
    x = rnd(silu(causal_conv(x, W[pre + "conv"], W[pre + "conv.b"])))
    p = x @ W[pre + "x"].T
    dt = softplus(rnd(p[:, :K]) @ W[pre + "dt"].T + W[pre + "dt.b"])
    Bm, Cm = p[:, K:K + N], p[:, K + N:K + 2 * N]
    A = -torch.exp(W[pre + "A_log"])
    S = torch.zeros(I, N, dtype=F64)
    y = torch.zeros(T, I, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * Bm[t][None, :]
        y[t] = S @ Cm[t] + W[pre + "D"] * x[t]
    y = y * silu(z)
    return rnd(y) @ W[pre + "o"].T


# --------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, pre, rnd=ident):
    return rnd(gelu_tanh(h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(h, W, pre, r):
    """(picked experts [T, top], their factors [T, top]). s = sigmoid(logits); c = s + correction picks:
    experts in runs of equal length, a run rated by its best two c, only the best-rated runs open, the
    highest c among the open; the factors are the picked experts' s over their sum, times a scale."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ W[pre + "router"].T)
    choice = s + W[pre + "correction"]
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = choice.view(-1, n, E // n)
        gscore = per.topk(min(2, E // n), dim=-1).values.sum(-1)
        best = gscore.topk(keep, dim=-1).indices
        allowed = torch.zeros(h.shape[0], n, dtype=torch.bool)
        allowed.scatter_(1, best, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(E // n, dim=1), float("-inf"))
    idx = choice.topk(top, dim=-1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20) * float(r["scale"])


def moe_ff(h, W, pre, m, rnd=ident, router_input=None):
    idx, w = route(h if router_input is None else router_input, W, pre, m["router"])
    out = torch.zeros(h.shape[0], W[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            a = rnd(relu_squared(h[t] @ W[f"{pre}e{e}.up"].T))
            out[t] += w[t, j] * (a @ W[f"{pre}e{e}.down"].T)
    return out


# --------------------------------------------------------------------------- the model
class PlainMuvorax:
    def __init__(self, cfg: dict, weights: dict, rnd=ident):
        self.cfg, self.rnd = cfg, rnd
        self.W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}

    def layer(self, i, x, kept):
        W, L, eps, rnd = self.W, self.cfg["layers"][i], float(self.cfg["norm"]["eps"]), self.rnd
        p, m = f"l{i}.", L["mixer"]
        h = rnd(dynamic_tanh(x, W, p + "norm1"))
        if L["type"] == "lightning":
            a = lightning(h, W, p + "mix.", m, eps, rnd)
        elif L["type"] == "mamba1":
            a = mamba1(h, W, p + "mix.", m, rnd)
        elif L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_pair(h, W, p + "mix.", m, eps, rnd)
            a = latent_attention(h, W, p + "mix.", m, eps, shared=kept[i if src is None else src], rnd=rnd)
        else:
            raise ValueError(f"layer type {L['type']!r}")
        x = x + dynamic_tanh(rnd(a), W, p + "norm1b")
        if L.get("mlp") is not None:
            h32 = dynamic_tanh(x, W, p + "norm2")
            h = rnd(h32)
            if L["mlp"]["kind"] == "dense":
                f = dense_ff(h, W, p + "mlp.", rnd)
            else:
                f = moe_ff(h, W, p + "mlp.", L["mlp"], rnd, router_input=h32)
            x = x + dynamic_tanh(rnd(f), W, p + "norm2b")
        return x

    def forward(self, ids, layers_out: list | None = None):
        """Logits [T, vocab] of one sequence; `layers_out` collects the stream after every layer."""
        x = self.W["embed"][torch.as_tensor(ids, dtype=torch.long)]
        kept = {}
        for i in range(len(self.cfg["layers"])):
            x = self.layer(i, x, kept)
            if layers_out is not None:
                layers_out.append(x.clone())
        n = self.rnd(dynamic_tanh(x, self.W, "final.norm"))
        return n @ self.W["embed"].T


def load_folder(model_dir):
    """(config dict, tensors) of a model folder, read with a reader of its own."""
    import numpy as np
    d = Path(model_dir)
    cfg = json.loads((d / "config.json").read_text())
    blob = (d / "model.safetensors").read_bytes()
    n = int.from_bytes(blob[:8], "little")
    header = json.loads(blob[8:8 + n])
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        a, b = rec["data_offsets"]
        raw = blob[8 + n + a:8 + n + b]
        if rec["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif rec["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        elif rec["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {rec['dtype']}")
        out[name] = t.reshape(rec["shape"])
    return cfg, out
