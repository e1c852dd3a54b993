"""A plain, slow statement of the Sozilix decoder in float64, one function per mechanism.

Nothing here is shared with the library: tensors come in as a dict name -> torch tensor, the
configuration as the parsed config.json, and every function works on one sequence given as a whole
([tokens, channels]); there is no cache and no state, so whatever the library does with portions,
batches, pages and slots has to agree with this.

Notation: x_t the residual stream at token t, h what a mixer reads, W x a stored [out, in] matrix
applied to a column vector (here: rows times W^T).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w; var = mean squared deviation; no bias."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def causal_conv(x, w, bias=None):
    """y_t[c] = sum_j w[c, j] x_{t - taps + 1 + j}[c] (+ bias[c]); x before the start is zero.
    x [T, C], w [C, taps]: the last column multiplies the current token."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    if bias is not None:
        y = y + bias
    return y


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotate_interleaved(x, positions, rot_dims, base):
    """x [T, heads, dim]: dims (2i, 2i+1), i < rot_dims / 2, turned by positions * base^(-2i / rot_dims)."""
    out = x.clone()
    for i in range(rot_dims // 2):
        f = float(base) ** (-2.0 * i / rot_dims)
        a = positions.to(F64) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def windowed_attention(h, W, pre, c, eps):
    """Softmax attention over a sliding window with grouped heads, partly rotated queries and keys
    and unit-rms values. h [T, width]."""
    T = h.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    pos = torch.arange(T)
    q = (h @ W[pre + "q"].T).view(T, H, D)
    k = (h @ W[pre + "k"].T).view(T, G, D)
    v = (h @ W[pre + "v"].T).view(T, G, V)
    q = rotate_interleaved(q, pos, c["rot"]["dims"], c["rot"]["base"])
    k = rotate_interleaved(k, pos, c["rot"]["dims"], c["rot"]["base"])
    v = rms_unit(v, eps)
    out = torch.zeros(T, H, V, dtype=F64)
    size = c["mask"]["size"]
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * c["scale"]
        i = pos[:, None]
        j = pos[None, :]
        seen = (i - j >= 0) & (i - j < size)
        s = s.masked_fill(~seen, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * V) @ W[pre + "o"].T


def gated_delta(h, W, pre, c, eps):
    """The gated delta rule with short convolutions, unit queries and keys and a gated unit-rms read-out."""
    T = h.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(causal_conv(h @ W[pre + "q"].T, W[pre + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ W[pre + "k"].T, W[pre + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ W[pre + "v"].T, W[pre + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[pre + "b"].T)                                   # [T, H]
    decay = torch.exp(-torch.exp(W[pre + "A_log"]) * softplus(h @ W[pre + "a"].T + W[pre + "dt_bias"]))
    gate = silu(h @ W[pre + "g"].T).view(T, H, V)
    o = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(D, V, dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    o = rms_unit(o, eps) * W[pre + "norm"] * gate
    return o.reshape(T, H * V) @ W[pre + "o"].T


def parallel_mixer(h, W, pre, c, eps):
    return c["left_scale"] * windowed_attention(h, W, pre + "left.", c["left"], eps) + \
        c["right_scale"] * gated_delta(h, W, pre + "right.", c["right"], eps)


def rglru_mixer(h, W, pre, c, eps):
    """Two branches: a gelu gate, and a convolved one run through a real-gated linear recurrence
    whose gates are block-diagonal."""
    T = h.shape[0]
    width, nb = c["width"], c["blocks"]
    bs = width // nb
    y = gelu_tanh(h @ W[pre + "y"].T + W[pre + "y.b"])
    u = causal_conv(h @ W[pre + "x"].T + W[pre + "x.b"], W[pre + "conv"], W[pre + "conv.b"])
    ub = u.view(T, nb, bs)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W[pre + "ra"]) + W[pre + "ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W[pre + "ri"]) + W[pre + "ri.b"]).reshape(T, width)
    log_a = -8.0 * r * softplus(W[pre + "lam"])
    a = torch.exp(log_a)
    S = torch.zeros(width, dtype=F64)
    out = torch.zeros(T, width, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ W[pre + "o"].T


def dense_ff(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


MIXERS = {"parallel": parallel_mixer, "rglru": rglru_mixer}


def layer(x, W, i, lc, cfg):
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    p = f"l{i}."
    h = layer_norm(x, W[p + "norm1"], eps)
    h = h + causal_conv(h, W[p + "canon1"])
    x = x + m * MIXERS[lc["type"]](h, W, p + "mix.", lc["mixer"], eps)
    if lc.get("mlp") is not None:
        x = x + m * dense_ff(layer_norm(x, W[p + "norm2"], eps), W, p + "mlp.")
    return x


def forward(tokens, W, cfg, streams=None):
    """Logits [T, vocab] of one whole sequence; `streams` (a list) receives the stream after each layer."""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, lc in enumerate(cfg["layers"]):
        x = layer(x, W, i, lc, cfg)
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
