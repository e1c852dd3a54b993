"""A recurrent block around a real-gated linear recurrent unit (the RG-LRU of Griffin).

Two branches of width W from the mixer's input h: y = gelu_tanh(Wy h + by), and u = conv(Wx h + bx),
a short causal convolution per channel with a bias and no activation. u is cut into `blocks` equal
parts; in part b, r = sigmoid(Ra[b] u_b + ra_b[b]) and i = sigmoid(Ri[b] u_b + ri_b[b]) with square
matrices Ra[b], Ri[b] (block-diagonal gates). Per channel: log a = -8 r softplus(lam), a = exp(log a),
S_t = a S_{t-1} + sqrt(1 - a^2) * i * u, starting from S = 0 with the same formula for row 0 as for any row. The mixer's
output is Wo (S * y).

State per sequence: S [W] in float32 and the convolution's last taps - 1 inputs. Projections run in
the engine's dtype; the gates' products accumulate and stay in float32, as do u, the gates, the
decay and the recurrence.
"""
from __future__ import annotations

import torch

from ..cache.needs import StateNeed
from ..weights.spec import TensorSpec
from .base import MIXERS, Mixer
from .conv import CausalConv
from .linear import Linear


class RGLRU(Mixer):
    graph_safe = True

    def __init__(self, hidden: int, width: int, blocks: int, conv_taps: int, y_name: str, y_bias_name: str, x_name: str,
                 x_bias_name: str, conv_name: str, conv_bias_name: str, ra_name: str, ra_bias_name: str, ri_name: str,
                 ri_bias_name: str, lam_name: str, o_name: str):
        if blocks < 1 or width % blocks:
            raise ValueError(f"a width of {width} cannot be cut into {blocks} equal blocks")
        self.hidden, self.width, self.blocks, self.bs = hidden, width, blocks, width // blocks
        self.yx = Linear([y_name, x_name], [width, width], hidden)
        self.conv = CausalConv([conv_name], [width], conv_taps, bias_name=conv_bias_name)
        self.out = Linear([o_name], [hidden], width)
        self.names = dict(y_b=y_bias_name, x_b=x_bias_name, ra=ra_name, ra_b=ra_bias_name, ri=ri_name, ri_b=ri_bias_name, lam=lam_name)

    def tensor_specs(self):
        n, W, nb, bs = self.names, self.width, self.blocks, self.bs
        return (self.yx.tensor_specs() + self.conv.tensor_specs() + self.out.tensor_specs() +
                [TensorSpec(n["y_b"], (W,), init="bias"), TensorSpec(n["x_b"], (W,), init="bias"),
                 TensorSpec(n["ra"], (nb, bs, bs), init="gate_matrix"), TensorSpec(n["ra_b"], (nb, bs), init="bias"),
                 TensorSpec(n["ri"], (nb, bs, bs), init="gate_matrix"), TensorSpec(n["ri_b"], (nb, bs), init="bias"),
                 TensorSpec(n["lam"], (W,), init="log_rate")])

    def bind(self, tensors, dtype, device):
        for p in (self.yx, self.conv, self.out):
            p.bind(tensors, dtype, device)
        n = self.names
        self.y_b, self.x_b, self.lam = tensors[n["y_b"]], tensors[n["x_b"]], tensors[n["lam"]]
        self.ra_b, self.ri_b = tensors[n["ra_b"]].reshape(-1).contiguous(), tensors[n["ri_b"]].reshape(-1).contiguous()
        # per block one product for both gates: rows [Ra[b] ; Ri[b]]
        self.gate_w = torch.cat([tensors[n["ra"]], tensors[n["ri"]]], dim=1).contiguous()        # [blocks, 2 bs, bs]
        self.gates = []
        for b in range(self.blocks):
            lin = Linear([f"{n['ra']}[{b}]|{n['ri']}[{b}]"], [2 * self.bs], self.bs)
            lin.weight = self.gate_w[b]
            self.gates.append(lin)

    def state_need(self):
        need = {"S": StateNeed((self.width,), torch.float32)}
        conv = self.conv.state_need()
        if conv is not None:
            need["conv"] = conv
        return need

    def forward(self, x, ctx, unit, writes, state=None):
        st = state if state is not None else ctx.unit_state(unit)
        T, W, bs = x.shape[0], self.width, self.bs
        yx = self.yx.forward(x, ctx)                                           # [T, y | x] raw, engine dtype
        u_low = torch.empty((T, W), dtype=x.dtype, device=x.device) if x.dtype != torch.float32 else None
        u = self.conv.forward(yx[:, W:], st.get("conv"), ctx, torch.float32, in_bias=self.x_b, also=u_low)
        src = u if u_low is None else u_low
        gates = torch.empty((self.blocks, T, 2 * bs), dtype=torch.float32, device=x.device)
        for b, lin in enumerate(self.gates):
            lin.forward(src[:, b * bs:(b + 1) * bs], ctx, out_dtype=torch.float32, out=gates[b])
        out = torch.empty((T, W), dtype=x.dtype, device=x.device)
        ctx.kernels.seq.rglru_scan(gates, u, yx[:, :W], self.ra_b, self.ri_b, self.lam, self.y_b, st["S"], ctx, out, bs)
        return self.out.forward(out, ctx)


MIXERS.register("rglru", RGLRU)
