"""Several mixers side by side on the same input, their outputs added with a coefficient each:
y = sum_i scale_i * mixer_i(h). The branches are named parts of the MIXERS registry; at most one
may keep keys and values (a cache unit has one paged store), every one may keep state, which the
unit holds under the branch's name. The sum is not formed here: the branches' outputs go on as
weighted addends, and the norm that reads the residual stream next adds them in float32.
"""
from __future__ import annotations

from .base import MIXERS, Mixer, PartSpec


class ParallelMixer(Mixer):
    def __init__(self, branches: list):
        """`branches`: (name, PartSpec of a mixer, scale) each."""
        if not branches:
            raise ValueError("a parallel mixer needs at least one branch")
        self.names = [n for n, _, _ in branches]
        if len(set(self.names)) != len(self.names):
            raise ValueError(f"branch names must differ: {self.names}")
        self.mixers = [MIXERS.build(spec) for _, spec, _ in branches]
        self.scales = [float(s) for _, _, s in branches]
        if sum(m.cache_need() is not None for m in self.mixers) > 1:
            raise ValueError("at most one branch of a parallel mixer may keep keys and values")

    @property
    def graph_safe(self) -> bool:
        return all(getattr(m, "graph_safe", False) for m in self.mixers)

    def tensor_specs(self):
        return [s for m in self.mixers for s in m.tensor_specs()]

    def bind(self, tensors, dtype, device):
        for m in self.mixers:
            m.bind(tensors, dtype, device)

    def prepare(self, max_positions, device):
        for m in self.mixers:
            m.prepare(max_positions, device)

    def cache_need(self):
        for m in self.mixers:
            if m.cache_need() is not None:
                return m.cache_need()
        return None

    def state_need(self):
        need = {n: m.state_need() for n, m in zip(self.names, self.mixers) if m.state_need() is not None}
        return need or None

    def forward(self, x, ctx, unit, writes, state=None):
        st = state if state is not None else (ctx.unit_state(unit) if self.state_need() is not None else None)
        out = []
        for n, m, s in zip(self.names, self.mixers, self.scales):
            y = m.forward(x, ctx, unit, writes, state=st[n]) if m.state_need() is not None else m.forward(x, ctx, unit, writes)
            out.append((y, s))
        return out


MIXERS.register("parallel", ParallelMixer)
