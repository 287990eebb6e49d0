"""Mixers side by side: every branch reads the same input and the result is a scaled sum of the
branches' outputs, each first RMS-normed over the model width with a weight of its own.

    out = scale * sum_b rmsnorm(branch_b(x)) * w_b          (``<branch>.out`` [D], a plain weight)

The branches are mixers from the registry; their tensors and states live under the branch's name
(``left.q``, ``right.S``).  Their input projections run as one stacked product where every branch
exposes its own, the first branch runs on a side stream beside the others, and the norms and the
sum are one launch.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Sequence

import torch

from ..kernels import ops as K
from . import streaming
from . import branches as side_streams
from .base import Mixer, ParamSpec, PartSpec, StateSpec, build_part, register_mixer

Tensor = torch.Tensor


class NormedParallelMixer(Mixer):
    def __init__(self, hidden_size: int, branches: Sequence[Dict[str, Any]], eps: float, scale: float):
        """``branches``: [{"name", "kind", "params"}], at most four."""
        if not 1 <= len(branches) <= 4:
            raise ValueError("one to four branches")
        self.hidden_size = int(hidden_size)
        self.eps, self.scale = float(eps), float(scale)
        self.branch_names = [str(b["name"]) for b in branches]
        self.mixers: List[Mixer] = [build_part("mixer", PartSpec(b["kind"], b["name"], dict(b.get("params", {}))),
                                               hidden_size=hidden_size) for b in branches]
        self._name = ""
        self._fused = None
        self._cols: List[tuple] = []

    # the branches find their state under "<this mixer>.<branch>.<state>"
    @property
    def name(self) -> str:
        return self._name

    @name.setter
    def name(self, value: str) -> None:
        self._name = value
        for b, m in zip(self.branch_names, self.mixers):
            m.name = f"{value}.{b}" if value else b

    def param_specs(self) -> List[ParamSpec]:
        specs = []
        for b, m in zip(self.branch_names, self.mixers):
            specs += [dataclasses.replace(ps, name=f"{b}.{ps.name}" if ps.name else b) for ps in m.param_specs()]
            specs.append(ParamSpec(f"{b}.out", (self.hidden_size,), kind="vector", init=("ones",)))
        return specs

    def state_specs(self) -> List[StateSpec]:
        return [dataclasses.replace(s, name=f"{b}.{s.name}") for b, m in zip(self.branch_names, self.mixers)
                for s in m.state_specs()]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.out_w = []
        for b, m in zip(self.branch_names, self.mixers):
            m.bind({ps.name: params[f"{b}.{ps.name}" if ps.name else b] for ps in m.param_specs()})
            self.out_w.append(params[f"{b}.out"].contiguous())

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        for m in self.mixers:
            m.finalize(dtype, device)
        if len(self.mixers) > 1 and all(m.input_rows() > 0 for m in self.mixers):
            self._fused = torch.cat([m.input_weight() for m in self.mixers], dim=0).contiguous()
            start = 0
            for m in self.mixers:
                rows = m.input_rows()
                m.adopt_input_weight(self._fused[start:start + rows])
                self._cols.append((start, start + rows))
                start += rows

    def forward(self, x: Tensor, ctx, cache, out: Tensor) -> None:
        ws = ctx.workspace
        T = x.shape[0]
        outs = [ws.alloc((T, self.hidden_size), x.dtype) for _ in self.mixers]
        proj = None
        if self._fused is not None:
            proj = ws.alloc((T, self._fused.shape[0]), x.dtype)
            streaming.linear(x, self._fused, proj, ctx)
        main = torch.cuda.current_stream(x.device)
        side = side_streams.branch_stream(x.device, "mixer") if len(self.mixers) > 1 else None
        # a branch's output bias is added where the branch is normed, not by a launch of its own
        biases = [m.output_bias() for m in self.mixers]
        ctx.defer_output_bias = True
        for i, m in enumerate(self.mixers):
            def run():
                if proj is not None:
                    c0, c1 = self._cols[i]
                    m.forward_projected(proj[:, c0:c1], ctx, cache, outs[i])
                else:
                    m.forward(x, ctx, cache, outs[i])
            if i == 0 and side is not None:
                with side_streams.fork(main, side):
                    run()
            else:
                run()
        if side is not None:
            main.wait_stream(side)
        ctx.defer_output_bias = False
        K.normed_sum(list(zip(outs, self.out_w)), self.eps, self.scale, out, biases=biases)


register_mixer("normed_parallel", NormedParallelMixer)
