"""Causal softmax attention with biased projections, rotation of part of every head and an output gate.

    q = Wq x + bq (heads x dim), k = Wk x + bk (kv_heads x dim), v = Wv x + bv (kv_heads x vdim);
    among the first rot_dims entries of every q and k head, entry i < rot_dims/2 and entry
    i + rot_dims/2 turn together by the angle p * f_i, f_i = rot_base^(-2i / rot_dims) / rot_factor
    (``rot_layout`` "pairs": entries 2i and 2i+1 instead); entries from rot_dims on pass unchanged;
    score = (q . k) * scale; token i sees every j <= i (``window`` > 0: only 0 <= i - j < window);
    plain softmax; the concatenated heads are multiplied by sigmoid(Wg x) per channel (``gate``);
    out = Wo [heads].

Query head h reads key/value head h // (heads / kv_heads).  All projections that read x (q, k, v and
the gate) are row blocks of one stacked matrix.  State per request: the rotated keys and the values
in cache pages; every head is Dp = max(dim, vdim) (rounded up to a multiple of 16) wide there and in
the attention kernels, padded with zeros; the gate drops the padding again.  Positions, angles,
sines and cosines, scores and softmax weights are float arithmetic in both storage types.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from . import streaming
from .base import ParamSpec, StateSpec, register_mixer
from .window_attention import PagedSoftmaxAttention

Tensor = torch.Tensor


class GatedRotaryAttention(PagedSoftmaxAttention):
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, rot_dims: int, rot_base: float,
                 scale: float, rot_factor: float = 1.0, rot_layout: str = "halves", bias: bool = True, gate: bool = True,
                 window: int = 0, out_multiplier: float = 1.0):
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ValueError("rot_dims must be even and at most dim")
        if rot_layout not in ("halves", "pairs"):
            raise ValueError("rot_layout is 'halves' or 'pairs'")
        if rot_factor <= 0.0:
            raise ValueError("rot_factor must be positive")
        self.hidden_size = int(hidden_size)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.rot_dims, self.rot_base, self.rot_factor = int(rot_dims), float(rot_base), float(rot_factor)
        self.half_layout = rot_layout == "halves"
        self.scale, self.window = float(scale), int(window)
        self.has_bias, self.has_gate = bool(bias), bool(gate)
        self.out_scale = float(out_multiplier)
        self.padded_dim = (max(self.dim, self.vdim) + 15) // 16 * 16
        K.check_head_dim(self.padded_dim)
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.o_dim = self.heads * self.vdim
        self.inv_freq: Optional[Tensor] = None
        self.biases = None

    def param_specs(self) -> List[ParamSpec]:
        D = self.hidden_size
        specs = []
        for name, rows in (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim)):
            specs.append(ParamSpec(name, (rows, D)))
            if self.has_bias:
                specs.append(ParamSpec(name + ".b", (rows,), kind="vector", init=("normal", 0.1)))
        if self.has_gate:
            specs.append(ParamSpec("g", (self.o_dim, D)))
        specs.append(ParamSpec("o", (D, self.o_dim)))
        return specs

    def state_specs(self) -> List[StateSpec]:
        return [StateSpec.paged("kv", planes=2, width=self.kv_heads * self.padded_dim, window=self.window)]

    def bind(self, params: Dict[str, Tensor]) -> None:
        blocks = [params["q"], params["k"], params["v"]] + ([params["g"]] if self.has_gate else [])
        self.w_in = torch.cat(blocks, dim=0).contiguous()
        if self.has_bias:
            self.biases = tuple(params[n + ".b"].contiguous() for n in ("q", "k", "v"))
        self.w_out = params["o"].contiguous()

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        if self.rot_dims > 0:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / float(self.rot_dims))
            self.inv_freq = (inv / self.rot_factor).to(device=device, dtype=torch.float32).contiguous()
        self._make_split_counter(device)

    def forward_projected(self, proj: Tensor, ctx, cache, out: Tensor) -> None:
        streaming.linear(self._gated_heads(proj, ctx, cache, None, 1.0), self.w_out, out, ctx)

    def output_weight(self) -> Tensor:
        return self.w_out

    def joins_output_products(self) -> bool:
        return self.has_gate

    def pre_output_into(self, proj: Tensor, ctx, cache, into: Tensor, scale: float) -> bool:
        if not self.has_gate:
            return False
        self._gated_heads(proj, ctx, cache, into, scale)
        return True

    def _gated_heads(self, proj: Tensor, ctx, cache, into: Optional[Tensor], scale: float) -> Tensor:
        """The concatenated heads after the output gate (times ``scale``), [T, heads * vdim]."""
        T = proj.shape[0]
        ws = ctx.workspace
        kv = cache.paged(f"{self.name}.kv")
        H, Dp = self.heads, self.padded_dim
        c_k, c_v, c_g = self.q_dim, self.q_dim + self.k_dim, self.q_dim + self.k_dim + self.v_dim
        q_rot = ws.alloc((T, H * Dp), proj.dtype)
        K.rope_pairs_store(proj[:, :c_k], proj[:, c_k:c_v], proj[:, c_v:c_g], self.inv_freq, self.rot_dims, ctx.positions,
                           ctx.seq_of, kv.block_table, kv.pool, q_rot, H, self.kv_heads, self.dim, self.vdim, Dp,
                           half_layout=self.half_layout, biases=self.biases)
        attn = ws.alloc((T, H * Dp), proj.dtype)
        self._attend(q_rot, kv, ctx, attn)
        if self.has_gate:
            gated = into if into is not None else ws.alloc((T, self.o_dim), proj.dtype)
            K.sigmoid_gate(attn, proj[:, c_g:c_g + self.o_dim], scale, gated, H, Dp, self.vdim)
        elif Dp != self.vdim:
            gated = ws.alloc((T, self.o_dim), proj.dtype)
            gated.view(T, H, self.vdim).copy_(attn.view(T, H, Dp)[:, :, :self.vdim])
        else:
            gated = attn
        return gated


register_mixer("rotary_gated_attention", GatedRotaryAttention)
