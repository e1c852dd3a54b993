"""Linear attention with a fixed decay per head (the recurrence of "lightning attention").

From the mixer's input h (no biases): q = silu(Wq h), k = silu(Wk h) with n_heads heads of width
dk, v = silu(Wv h) with heads of width dv. Per head a matrix state S [dk, dv], zero at the start of
a sequence: S_t = g S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, with g the head's decay (a constant of the
model, no other scale). The heads' outputs side by side are divided by the root mean square of the
whole row, sqrt(mean(o^2) + eps), multiplied by a weight [n_heads dv] and by sigmoid(Wg h), and Wo
maps them back to the hidden width.

The kernel works a step's rows in pieces: inside a piece the rows see each other through their
decayed scores (q_i . k_j) g^(i-j), and the pieces before them through the state, so a prompt
costs matrix products instead of one dependent update per row; a decode step is a piece of one
row. State per sequence: S in float32. The projections run in the engine's dtype; SiLU, scores,
decay powers, state and the read-out norm are float32.
"""
from __future__ import annotations

import torch

from ..cache.needs import StateNeed
from ..weights.spec import TensorSpec
from .base import MIXERS, Mixer
from .linear import Linear


class DecayLinearAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, decay: list, norm_eps: float, q_name: str,
                 k_name: str, v_name: str, gate_name: str, norm_name: str, o_name: str, gate_act: str = "sigmoid"):
        if len(decay) != n_heads:
            raise ValueError(f"{len(decay)} decays for {n_heads} heads")
        if any(not 0.0 <= float(g) <= 1.0 for g in decay):
            raise ValueError("a head's decay lies in 0..1")
        self.hidden, self.H, self.dk, self.dv, self.eps, self.gate_act = hidden, n_heads, key_dim, value_dim, float(norm_eps), gate_act
        self.decay_values = [float(g) for g in decay]
        qk, vw = n_heads * key_dim, n_heads * value_dim
        self.qk_width, self.v_width = qk, vw
        self.wide = Linear([q_name, k_name, v_name, gate_name], [qk, qk, vw, vw], hidden)
        self.out = Linear([o_name], [hidden], vw)
        self.norm_name = norm_name

    def tensor_specs(self):
        return self.wide.tensor_specs() + self.out.tensor_specs() + [TensorSpec(self.norm_name, (self.v_width,), init="norm_weight")]

    def bind(self, tensors, dtype, device):
        self.wide.bind(tensors, dtype, device)
        self.out.bind(tensors, dtype, device)
        self.norm_w = tensors[self.norm_name].float().contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(device)

    def state_need(self):
        return {"S": StateNeed((self.H, self.dk, self.dv), torch.float32)}

    def forward(self, x, ctx, unit, writes, state=None):
        st = state if state is not None else ctx.unit_state(unit)
        k = ctx.kernels.mix
        T = x.shape[0]
        proj = self.wide.forward(x, ctx)                                         # [T, q | k | v | gate] raw, the engine's dtype
        o = torch.empty((T, self.v_width), dtype=torch.float32, device=x.device)
        k.lin_attn_decay(proj, 0, self.qk_width, 2 * self.qk_width, self.decay, st["S"], ctx, o, self.H, self.dk, self.dv)
        y = torch.empty((T, self.v_width), dtype=x.dtype, device=x.device)
        k.gated_row_rms(o, proj[:, 2 * self.qk_width + self.v_width:], self.norm_w, y, self.eps, self.gate_act)
        return self.out.forward(y, ctx, partials_ok=True)


MIXERS.register("decay_linear_attention", DecayLinearAttention)
