"""Hyper-connections: a layer whose residual state is several lanes instead of one stream.

The residual state is n lanes x_0..x_{n-1} of [T, D] floats, all equal to the embedding's output
at the start of the model and summed at its end.  Every sublayer q (the mixer, then the
feed-forward if the layer has one) owns three small tensors ``hc<q>.in`` [n], ``hc<q>.out`` [n]
and ``hc<q>.mix`` [n, n] (indexed [from, to]):

    u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y

with all lanes updated at once from the old ones.  As in the single-stream arrangement a
sublayer's result is not added by a launch of its own: it waits on the stream and is folded
into the lanes by the launch that norms the next sublayer's input.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .base import (FeedForward, LayerCache, LayerSpec, Mixer, Norm, ParamSpec, Part, PartSpec, StateSpec,
                   build_part, register_arrangement)

Tensor = torch.Tensor


class LaneWeights(Part):
    """The three tensors of one sublayer's connection to the lanes."""

    def __init__(self, n: int):
        self.n = int(n)

    def param_specs(self) -> List[ParamSpec]:
        n = self.n
        return [ParamSpec("in", (n,), kind="vector", init=("uniform", 0.5 / n, 1.5 / n)),
                ParamSpec("out", (n,), kind="vector", init=("uniform", 0.5, 1.0)),
                ParamSpec("mix", (n, n), kind="vector", init=("uniform", 0.5 / n, 1.5 / n))]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.in_w = params["in"].contiguous()
        self.out_w = params["out"].contiguous()
        self.mix = params["mix"].reshape(-1).contiguous()


def hyper_layer(prefix: str, lanes: int, mixer_norm: PartSpec, mixer: PartSpec,
                ffn_norm: Optional[PartSpec] = None, ffn: Optional[PartSpec] = None) -> LayerSpec:
    """The LayerSpec of a ``hyper_prenorm`` layer."""
    return LayerSpec("hyper_prenorm", prefix, {"lanes": int(lanes), "mixer_norm": mixer_norm, "mixer": mixer,
                                               "ffn_norm": ffn_norm, "ffn": ffn})


class HyperPreNormBlock(Part):
    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.prefix = spec.prefix
        self.hidden_size = hidden_size
        unknown = set(spec.parts) - {"lanes", "mixer_norm", "mixer", "ffn_norm", "ffn"}
        if unknown or spec.part("mixer_norm") is None or spec.part("mixer") is None or not spec.part("lanes"):
            raise ValueError("hyper_prenorm takes the parts lanes, mixer_norm, mixer, ffn_norm and ffn"
                             + (f"; got also {sorted(unknown)}" if unknown else ""))
        self.n_lanes = int(spec.part("lanes"))
        self.mixer_norm: Norm = build_part("norm", spec.part("mixer_norm"), width=hidden_size)
        self.mixer: Mixer = build_part("mixer", spec.part("mixer"), hidden_size=hidden_size)
        self.mixer_lanes = LaneWeights(self.n_lanes)
        self.mixer_lanes.name = "hc1"
        self.ffn_norm: Optional[Norm] = None
        self.ffn: Optional[FeedForward] = None
        self.ffn_lanes: Optional[LaneWeights] = None
        if spec.part("ffn") is not None:
            if spec.part("ffn_norm") is None:
                raise ValueError("a feed-forward needs its norm")
            self.ffn_norm = build_part("norm", spec.part("ffn_norm"), width=hidden_size)
            self.ffn = build_part("feed_forward", spec.part("ffn"), hidden_size=hidden_size)
            self.ffn_lanes = LaneWeights(self.n_lanes)
            self.ffn_lanes.name = "hc2"

    def parts(self) -> List[Part]:
        out: List[Part] = [self.mixer_norm, self.mixer, self.mixer_lanes]
        if self.ffn is not None:
            out += [self.ffn_norm, self.ffn, self.ffn_lanes]
        return out

    def branch_buffers_needed(self) -> int:
        return 1

    def state_specs(self) -> List[Tuple[str, StateSpec]]:
        return [(f"{self.mixer.name}.{s.name}", s) for s in self.mixer.state_specs()]

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        for p in self.parts():
            p.finalize(dtype, device)
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and norm.rms_prologue() is None:
                raise ValueError("hyper_prenorm norms its sublayers' inputs in the launch that mixes the lanes: "
                                 "it takes RMS-form norms only")

    def forward(self, stream, ctx, cache: LayerCache) -> None:
        if stream.lanes is None or stream.lanes.shape[0] != self.n_lanes:
            raise RuntimeError(f"hyper_prenorm needs a residual state of {self.n_lanes} lanes "
                               "(ModelSpec.residual_lanes)")
        ws = ctx.workspace
        mark = ws.mark()
        n = stream.lanes_normed(self.mixer_lanes.in_w, self.mixer_norm)
        out = stream.take_branch()
        self.mixer.forward(n, ctx, cache, out)
        stream.lane_add(out, self.mixer_lanes.mix, self.mixer_lanes.out_w)
        if self.ffn is not None:
            f = stream.lanes_normed(self.ffn_lanes.in_w, self.ffn_norm)
            out = stream.take_branch()
            self.ffn.forward(f, ctx, out)
            stream.lane_add(out, self.ffn_lanes.mix, self.ffn_lanes.out_w)
        ws.release(mark)


register_arrangement("hyper_prenorm", HyperPreNormBlock)
