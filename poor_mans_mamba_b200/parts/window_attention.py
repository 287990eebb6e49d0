"""Softmax attention over a sliding window with a sink, a short convolution after the
projections and pair-rotated positions.

    q = Wq x + bq (heads x dim), k = Wk x + bk (kv_heads x dim), v = Wv x + bv (kv_heads x vdim);
    each passes a short causal convolution per channel (no activation), directly after the projection;
    the first rot_dims entries of every q and k head are rotated in neighbouring pairs (2i, 2i+1) by
    the angle p * base^(-2i / rot_dims);  score = (q . k) * scale;  token i sees j with
    0 <= i - j < window (``window`` 0: all earlier tokens);  the softmax's denominator also holds
    exp(sink_h), a learned score per head without key or value;  out = Wo [heads] + bo.

State per request: the rotated keys and the values in cache pages (a windowed group, so pages the
window has passed are given back) and the last taps - 1 projected rows of the convolution (float32,
in a slot).  Key size and value size may differ: in the pages and in the attention kernel every
head is Dp = max(dim, vdim) (rounded up to a multiple of 16) wide, padded with zeros, and the
output projection's matrix gets zero columns to match.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from .base import ParamSpec, StateSpec, register_mixer
from .recurrent import _StackedInput, causal_conv

Tensor = torch.Tensor

_TARGET_BLOCKS = 592   # the float kernel's key ranges are sized for about this many blocks


def plan_key_ranges(n_tokens: int, n_heads: int, kv_len_bound: int, window: int):
    """(number of key ranges, their length) for the float attention kernel (four heads a block)."""
    blocks = n_tokens * ((n_heads + 3) // 4)
    reach = min(kv_len_bound, window) if window > 0 else kv_len_bound
    if blocks >= _TARGET_BLOCKS or reach <= 128:
        return 1, 0
    want = min((_TARGET_BLOCKS + blocks - 1) // blocks, (reach + 127) // 128)
    if want <= 1:
        return 1, 0
    split_len = ((kv_len_bound + want - 1) // want + 63) // 64 * 64
    n_splits = (kv_len_bound + split_len - 1) // split_len
    return (n_splits, split_len) if n_splits > 1 else (1, 0)


class WindowSinkAttention(_StackedInput):
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, window: int,
                 rot_dims: int, rot_base: float, scale: float):
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ValueError("rot_dims must be even and at most dim")
        if conv < 1:
            raise ValueError("the convolution needs at least one tap")
        self.hidden_size = int(hidden_size)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.taps, self.window = int(conv), int(window)
        self.rot_dims, self.rot_base, self.scale = int(rot_dims), float(rot_base), float(scale)
        self.padded_dim = (max(self.dim, self.vdim) + 15) // 16 * 16
        K.check_head_dim(self.padded_dim)
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.conv_dim = self.q_dim + self.k_dim + self.v_dim
        self.inv_freq: Optional[Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        D = self.hidden_size
        conv = ("normal", 0.5)
        specs = []
        for name, rows in (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim)):
            specs += [ParamSpec(name, (rows, D)), ParamSpec(name + ".b", (rows,), kind="vector"),
                      ParamSpec(name + ".conv", (rows, self.taps), kind="vector", init=conv)]
        specs += [ParamSpec("sink", (self.heads,), kind="vector", init=("normal", 1.0)),
                  ParamSpec("o", (D, self.heads * self.vdim)), ParamSpec("o.b", (D,), kind="vector")]
        return specs

    def state_specs(self) -> List[StateSpec]:
        return [StateSpec.paged("kv", planes=2, width=self.kv_heads * self.padded_dim, window=self.window),
                StateSpec.fixed("conv", (self.taps - 1, self.conv_dim), "float32")]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.w_in = torch.cat([params["q"], params["k"], params["v"]], dim=0).contiguous()
        self.in_bias = torch.cat([params["q.b"], params["k.b"], params["v.b"]]).contiguous()
        self.conv_w = torch.cat([params["q.conv"], params["k.conv"], params["v.conv"]], dim=0).contiguous()
        self.conv_w_t = self.conv_w.t().contiguous()
        self.conv_ones = torch.ones(self.conv_dim, dtype=torch.float32, device=self.conv_w.device)
        self.sink = params["sink"].contiguous()
        self.out_bias = params["o.b"].contiguous()
        w_o = params["o"]
        if self.padded_dim != self.vdim:  # zero columns where the attention kernel's heads are padded
            w = torch.zeros((w_o.shape[0], self.heads, self.padded_dim), dtype=w_o.dtype, device=w_o.device)
            w[:, :, :self.vdim] = w_o.view(w_o.shape[0], self.heads, self.vdim)
            w_o = w.view(w_o.shape[0], self.heads * self.padded_dim)
        self.w_out = w_o.contiguous()

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        if self.rot_dims > 0:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / float(self.rot_dims))
            self.inv_freq = inv.to(device=device, dtype=torch.float32).contiguous()

    def forward_projected(self, proj: Tensor, ctx, cache, out: Tensor) -> None:
        T = proj.shape[0]
        ws = ctx.workspace
        kv = cache.paged(f"{self.name}.kv")
        # the projection's bias is added where the convolution reads its input (and kept in the window)
        qkv = causal_conv(proj, self.conv_ones, self.in_bias, self.conv_w, self.conv_w_t,
                          cache.fixed(f"{self.name}.conv"), ctx, activation=False)
        Dp = self.padded_dim
        q_rot = ws.alloc((T, self.heads * Dp), proj.dtype)
        K.rope_pairs_store(qkv[:, :self.q_dim], qkv[:, self.q_dim:self.q_dim + self.k_dim],
                           qkv[:, self.q_dim + self.k_dim:], self.inv_freq, self.rot_dims, ctx.positions, ctx.seq_of,
                           kv.block_table, kv.pool, q_rot, self.heads, self.kv_heads, self.dim, self.vdim, Dp)
        n_splits, split_len = plan_key_ranges(T, self.heads, ctx.kv_len_bound, self.window)
        scratch = None
        if n_splits > 1:
            scratch = ws.alloc((K.attention_scratch_floats(T, self.heads, Dp, n_splits),), torch.float32)
        attn = ws.alloc((T, self.heads * Dp), proj.dtype)
        K.paged_attention(q_rot, kv.pool, kv.block_table, ctx.positions, ctx.seq_of, attn, self.heads, self.kv_heads,
                          Dp, self.scale, window=self.window, n_splits=n_splits, split_len=split_len, scratch=scratch,
                          sink=self.sink)
        K.linear(attn, self.w_out, out)
        K.add_row_bias_(out, self.out_bias)


register_mixer("window_sink_attention", WindowSinkAttention)
