"""The gated delta rule: a linear-attention mixer whose per-head state is a matrix S [dk, dv] that
decays, is corrected towards the new value along the new key, and is read with the query.

From the mixer's input h (no biases): q = Wq h and k = Wk h with n_kv_heads heads of width dk,
v = Wv h with n_heads heads of width dv; head i reads q/k head i // (n_heads / n_kv_heads). Each of
q, k, v passes a short causal convolution per channel and SiLU; q and k then become unit vectors per
head, x / sqrt(sum x^2 + 1e-6), and q is multiplied by dk^-1/2. beta = sigmoid(Wb h) and
decay = exp(-exp(A_log) * softplus(Wa h + dt_bias)), one each per head. For every head and row the
state is first shrunk, S = decay * S; then corrected, u = beta * (v - S^T k), S = S + k u^T; then read,
o = S^T q, i.e. a row's output already contains what the row wrote. The output per head is
o / rms(o) (over dv, with eps) times a weight vector [dv] that all heads share, times silu(Wg h) taken
as [heads, dv]; Wo maps the heads' outputs back to the hidden width.

State per sequence: S in float32 and the last taps - 1 inputs of the three convolutions. The
projections run in the engine's dtype; everything from the convolutions' outputs to the read-out
(unit norms, beta, decay, the recurrence, the output norm) is float32.
"""
from __future__ import annotations

import torch

from ..cache.needs import StateNeed
from ..weights.spec import TensorSpec
from .base import MIXERS, Mixer
from .conv import CausalConv
from .linear import Linear


class GatedDeltaRule(Mixer):
    graph_safe = True
    MAX_KEY_WIDTH = 512

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, conv_taps: int, norm_eps: float,
                 q_name: str, k_name: str, v_name: str, q_conv_name: str, k_conv_name: str, v_conv_name: str, beta_name: str,
                 decay_name: str, a_log_name: str, dt_bias_name: str, gate_name: str, norm_name: str, o_name: str):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} query/key heads")
        if key_dim > self.MAX_KEY_WIDTH:
            raise ValueError(f"key width {key_dim}: the recurrence kernel keeps a state column in registers, at most {self.MAX_KEY_WIDTH}")
        self.hidden, self.H, self.G, self.dk, self.dv, self.eps = hidden, n_heads, n_kv_heads, key_dim, value_dim, float(norm_eps)
        qk, vw = n_kv_heads * key_dim, n_heads * value_dim
        self.qk_width, self.v_width = qk, vw
        # one product for everything that is a row of h: q | k | v | gate, and a small one for beta | decay
        self.wide = Linear([q_name, k_name, v_name, gate_name], [qk, qk, vw, vw], hidden)
        self.small = Linear([beta_name, decay_name], [n_heads, n_heads], hidden)
        self.conv = CausalConv([q_conv_name, k_conv_name, v_conv_name], [qk, qk, vw], conv_taps, act="silu")
        self.out = Linear([o_name], [hidden], vw)
        self.a_log_name, self.dt_bias_name, self.norm_name = a_log_name, dt_bias_name, norm_name

    def tensor_specs(self):
        return (self.wide.tensor_specs() + self.small.tensor_specs() + self.conv.tensor_specs() + self.out.tensor_specs() +
                [TensorSpec(self.a_log_name, (self.H,), init="log_rate"), TensorSpec(self.dt_bias_name, (self.H,), init="bias"),
                 TensorSpec(self.norm_name, (self.dv,), init="norm_weight")])

    def bind(self, tensors, dtype, device):
        for p in (self.wide, self.small, self.conv, self.out):
            p.bind(tensors, dtype, device)
        # the small product's rows padded to a multiple of 8 with zero rows: every product kernel takes that
        w = self.small.weight
        pad = -w.shape[0] % 8
        if pad:
            self.small.weight = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)]).contiguous()
        self.a_log, self.dt_bias, self.norm_w = tensors[self.a_log_name], tensors[self.dt_bias_name], tensors[self.norm_name]

    def state_need(self):
        need = {"S": StateNeed((self.H, self.dk, self.dv), torch.float32)}
        conv = self.conv.state_need()
        if conv is not None:
            need["conv"] = conv
        return need

    def forward(self, x, ctx, unit, writes, state=None):
        st = state if state is not None else ctx.unit_state(unit)
        k = ctx.kernels.seq
        T = x.shape[0]
        proj = self.wide.forward(x, ctx)                                        # [T, q | k | v | gate] in the engine's dtype
        ba = self.small.forward(x, ctx, out_dtype=torch.float32)                # [T, beta | decay (| padding)] float32
        n_conv = 2 * self.qk_width + self.v_width
        qkv = self.conv.forward(proj[:, :n_conv], st.get("conv"), ctx, torch.float32)       # float32 [T, q | k | v]
        bd = torch.empty((T, 2 * self.H + self.G), dtype=torch.float32, device=x.device)    # beta | decay | k . q
        k.delta_prepare(qkv[:, :2 * self.qk_width], ba, self.a_log, self.dt_bias, bd, self.H, self.G, self.dk)
        o = torch.empty((T, self.v_width), dtype=torch.float32, device=x.device)
        k.delta_rule(qkv[:, :2 * self.qk_width], qkv[:, 2 * self.qk_width:], bd, st["S"], ctx, o, self.H, self.G, self.dk, self.dv)
        y = torch.empty((T, self.v_width), dtype=x.dtype, device=x.device)
        k.gated_unit_rms(o, proj[:, n_conv:], self.norm_w, y, self.H, self.dv, self.eps)
        return self.out.forward(y, ctx)


MIXERS.register("gated_delta_rule", GatedDeltaRule)
