"""The selective scan (the mixer of Mamba): a state vector per channel whose decay, input and
read-out depend on the token.

The input projection Win h gives two halves of `inner` channels, x and z. On x runs a short causal
convolution over time, one filter and one bias per channel, followed by SiLU. Wx x = [dt_low (dt_rank) | B (n_state) | C (n_state)];
dt = softplus(Wdt dt_low + dt_bias), one per channel; A = -exp(A_log) [inner, n_state]. Per channel c
and state n: S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c. The
output is Wo (y * silu(z)).

State per sequence: S [inner, n_state] in float32 (zero at the start) and the convolution's last
taps - 1 inputs. The projections and the convolution with its SiLU run in the engine's dtype; the
step size with its softplus, the decay's exponentials, the state and the read-out are float32 (the
step size's product writes float32).
"""
from __future__ import annotations

import torch

from ..cache.needs import StateNeed
from ..weights.spec import TensorSpec
from .base import MIXERS, Mixer
from .conv import CausalConv
from .linear import Linear


class SelectiveScan(Mixer):
    graph_safe = True
    MAX_STATE = 256

    def __init__(self, hidden: int, inner: int, n_state: int, dt_rank: int, conv_taps: int, in_name: str, conv_name: str,
                 conv_bias_name: str, x_name: str, dt_name: str, dt_bias_name: str, a_log_name: str, d_name: str, o_name: str):
        if not 1 <= n_state <= self.MAX_STATE:
            raise ValueError(f"{n_state} states per channel: the scan kernel keeps them in registers, 1..{self.MAX_STATE}")
        self.hidden, self.I, self.N, self.K = hidden, inner, n_state, dt_rank
        self.in_proj = Linear([in_name], [2 * inner], hidden)
        self.conv = CausalConv([conv_name], [inner], conv_taps, bias_name=conv_bias_name, act="silu")
        self.x_proj = Linear([x_name], [dt_rank + 2 * n_state], inner)
        self.dt_proj = Linear([dt_name], [inner], dt_rank)
        self.out = Linear([o_name], [hidden], inner)
        self.names = dict(dt_b=dt_bias_name, a_log=a_log_name, d=d_name)

    def _linears(self):
        return (self.in_proj, self.x_proj, self.dt_proj, self.out)

    def tensor_specs(self):
        n = self.names
        specs = [s for p in self._linears() for s in p.tensor_specs()] + self.conv.tensor_specs()
        return specs + [TensorSpec(n["dt_b"], (self.I,), init="bias"), TensorSpec(n["a_log"], (self.I, self.N), init="log_rate"),
                        TensorSpec(n["d"], (self.I,), init="norm_weight")]

    def bind(self, tensors, dtype, device):
        for p in self._linears() + (self.conv,):
            p.bind(tensors, dtype, device)
        n = self.names
        self.dt_b, self.a_log, self.d = (tensors[n[k]].float().contiguous() for k in ("dt_b", "a_log", "d"))

    def state_need(self):
        need = {"S": StateNeed((self.I, self.N), torch.float32)}
        conv = self.conv.state_need()
        if conv is not None:
            need["conv"] = conv
        return need

    def forward(self, x, ctx, unit, writes, state=None):
        st = state if state is not None else ctx.unit_state(unit)
        I, N, K = self.I, self.N, self.K
        xz = self.in_proj.forward(x, ctx)                                        # [T, x | z] raw
        xc = self.conv.forward(xz[:, :I], st.get("conv"), ctx, x.dtype)          # convolution + bias + SiLU
        p = self.x_proj.forward(xc, ctx)                                         # [T, dt_low | B | C]
        dt_raw = self.dt_proj.forward(p[:, :K], ctx, out_dtype=torch.float32)    # [T, I] float32, before bias and softplus
        y = torch.empty((x.shape[0], I), dtype=x.dtype, device=x.device)
        ctx.kernels.mix.selective_scan(xc, dt_raw, self.dt_b, self.a_log, self.d, p, K, K + N, xz[:, I:], st["S"], ctx, y, I, N)
        return self.out.forward(y, ctx, partials_ok=True)


MIXERS.register("selective_scan", SelectiveScan)
