"""Mixers whose per-request state is one matrix per head, updated token by token.

``GatedDeltaMixer`` ("gated_delta"): the gated delta rule with a decay per head and key channel.
    q = Wq x, k = Wk x (kv_heads x dim), v = Wv x (heads x vdim); each passes a short causal
    convolution per channel and SiLU; q and k are scaled to unit length per head
    (x / sqrt(sum x^2 + unit_eps), q also by dim^-1/2); head h reads q/k head h // (heads / kv_heads);
    beta = sigmoid(Wb x) per head;  g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 x) + dt_bias)) per head
    and key channel;  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
    out = Wo [ rmsnorm_head(o) * norm * sigmoid(Wg2 (Wg1 x)) ].
``DecayLinearAttention`` ("decay_linear_attention"): linear attention with a fixed decay per head.
    q, k = silu(W x) (heads x dim), v = silu(Wv x) (heads x vdim);  S <- decay_h S + k v^T;  o = S^T q;
    out = Wo [ rmsnorm(o over all heads) * norm * sigmoid(Wg x) ].

State per request (float32, in a slot, zero for a new request): S [heads, dim, vdim]; the gated
delta mixer also keeps the last taps - 1 inputs of its convolution.  Decays, gates, unit lengths,
the state and the norm are float arithmetic in both storage types; the projections, the convolution
and SiLU have the storage type.  Every projection that reads x is a row block of one stacked matrix.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import ops as K
from . import streaming
from . import branches
from .base import Mixer, ParamSpec, StateSpec, register_mixer

Tensor = torch.Tensor

# Steps whose longest portion has at least this many tokens walk it in chunks (two launches with a
# fixed cost of tens of microseconds) instead of token by token (about a microsecond a token).
_CHUNKED_FROM = 32


def _chunked(ctx, dim: int, delta: bool) -> bool:
    return (not ctx.decode_only and max(ctx.new_lens) >= _CHUNKED_FROM and K.recurrent_chunked_supported(dim, delta))


class _StackedInput(Mixer):
    """Shares the stacked input projection with mixers that run beside this one."""
    w_in: Optional[Tensor] = None

    def input_rows(self) -> int:
        return int(self.w_in.shape[0])

    def input_weight(self) -> Tensor:
        return self.w_in

    def adopt_input_weight(self, view: Tensor) -> None:
        self.w_in = view

    def forward(self, x: Tensor, ctx, cache, out: Tensor) -> None:
        proj = ctx.workspace.alloc((x.shape[0], self.input_rows()), x.dtype)
        streaming.linear(x, self.w_in, proj, ctx)
        self.forward_projected(proj, ctx, cache, out)


def causal_conv(raw: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], weight: Tensor, weight_t: Tensor,
                window: Tensor, ctx, activation: bool) -> Tensor:
    """Short causal convolution per channel over the step's tokens, from and into the requests'
    windows (the last taps - 1 inputs of each); returns [T, C] in the storage type."""
    T, C = raw.shape
    out = ctx.workspace.alloc((T, C), raw.dtype)
    if ctx.decode_only:
        K.conv1d_decode(raw, pre_scale, pre_bias, weight, None, window, ctx.slots, out, activation=activation)
        return out
    K.conv1d_fwd(raw, pre_scale, pre_bias, weight, None, window, ctx.seq_of, ctx.cu_seqlens, ctx.slots, out,
                 weight_t=weight_t, activation=activation)
    # the window is next read by the next step; the write follows the read on the same stream
    K.conv1d_window_update(raw, pre_scale, pre_bias, window, ctx.cu_seqlens, ctx.slots, ctx.n_seq, weight.shape[1])
    return out


class GatedDeltaMixer(_StackedInput):
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int,
                 decay_rank: int, gate_rank: int, norm_eps: float, unit_eps: float = 1e-6):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if dim > K.RECURRENT_MAX_KEY_DIM:
            raise ValueError(f"the recurrence kernels take key sizes up to {K.RECURRENT_MAX_KEY_DIM}, got {dim}")
        if conv < 1:
            raise ValueError("the convolution needs at least one tap")
        self.hidden_size = int(hidden_size)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.taps, self.decay_rank, self.gate_rank = int(conv), int(decay_rank), int(gate_rank)
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.qk_dim = self.kv_heads * self.dim
        self.v_dim = self.heads * self.vdim
        self.conv_dim = 2 * self.qk_dim + self.v_dim

    def param_specs(self) -> List[ParamSpec]:
        D, H, d = self.hidden_size, self.heads, self.dim
        conv = ("normal", 0.5)
        return [
            ParamSpec("q", (self.qk_dim, D)), ParamSpec("q.conv", (self.qk_dim, self.taps), kind="vector", init=conv),
            ParamSpec("k", (self.qk_dim, D)), ParamSpec("k.conv", (self.qk_dim, self.taps), kind="vector", init=conv),
            ParamSpec("v", (self.v_dim, D)), ParamSpec("v.conv", (self.v_dim, self.taps), kind="vector", init=conv),
            ParamSpec("b", (H, D)),
            ParamSpec("A_log", (H,), kind="vector", init=("log_uniform", 0.5, 4.0)),
            ParamSpec("norm", (self.vdim,), kind="vector", init=("ones",)),
            ParamSpec("a1", (self.decay_rank, D)), ParamSpec("a2", (H * d, self.decay_rank)),
            ParamSpec("dt_bias", (H * d,), kind="vector", init=("inv_softplus_log_uniform", 1e-3, 0.1)),
            ParamSpec("g1", (self.gate_rank, D)), ParamSpec("g2", (self.v_dim, self.gate_rank)),
            ParamSpec("o", (D, self.v_dim)),
        ]

    def state_specs(self) -> List[StateSpec]:
        return [StateSpec.fixed("conv", (self.taps - 1, self.conv_dim), "float32"),
                StateSpec.fixed("S", (self.heads, self.dim, self.vdim), "float32")]

    def bind(self, params: Dict[str, Tensor]) -> None:
        # the low-rank inputs before the per-head beta: their column blocks then start on 16-byte boundaries
        self.w_in = torch.cat([params["q"], params["k"], params["v"], params["a1"], params["g1"], params["b"]],
                              dim=0).contiguous()
        self.conv_w = torch.cat([params["q.conv"], params["k.conv"], params["v.conv"]], dim=0).contiguous()
        self.conv_w_t = self.conv_w.t().contiguous()
        self.conv_ones = torch.ones(self.conv_dim, dtype=torch.float32, device=self.conv_w.device)
        self.a2, self.g2, self.w_out = params["a2"].contiguous(), params["g2"].contiguous(), params["o"].contiguous()
        self.a_log, self.dt_bias = params["A_log"].contiguous(), params["dt_bias"].contiguous()
        self.norm_w = params["norm"].repeat(self.heads).contiguous()  # one weight per channel of every head

    def forward_projected(self, proj: Tensor, ctx, cache, out: Tensor) -> None:
        T = proj.shape[0]
        ws = ctx.workspace
        c0 = self.conv_dim
        c1 = c0 + self.decay_rank
        c2 = c1 + self.gate_rank
        beta = proj[:, c2:c2 + self.heads]
        a = ws.alloc((T, self.heads * self.dim), proj.dtype)
        gate = ws.alloc((T, self.v_dim), proj.dtype)
        # The second halves of the low-rank projections run beside the convolution (a parallel branch
        # of a recorded step): the decays are needed by the recurrence, the output gate only after it.
        here = torch.cuda.current_stream(proj.device)
        side = branches.branch_stream(proj.device, "gate")
        with branches.fork(here, side):
            streaming.linear(proj[:, c0:c1], self.a2, a, ctx)
            decays_ready = torch.cuda.Event()
            decays_ready.record(side)
            streaming.linear(proj[:, c1:c2], self.g2, gate, ctx)
        qkv = causal_conv(proj[:, :c0], self.conv_ones, None, self.conv_w, self.conv_w_t,
                          cache.fixed(f"{self.name}.conv"), ctx, activation=True)
        o = ws.alloc((T, self.v_dim), torch.float32)
        q, k, v = qkv[:, :self.qk_dim], qkv[:, self.qk_dim:2 * self.qk_dim], qkv[:, 2 * self.qk_dim:]
        state = cache.fixed(f"{self.name}.S")
        here.wait_event(decays_ready)
        if _chunked(ctx, self.dim, True):
            scratch = ws.alloc((K.recurrent_chunked_scratch_floats(ctx.new_lens, self.heads, self.dim, self.vdim, True),),
                               torch.float32)
            K.recurrent_chunked(q, k, v, state, ctx.cu_seqlens, ctx.slots, ctx.new_lens, o, scratch, self.heads,
                                self.kv_heads, self.dim, self.vdim, beta=beta, a=a, dt_bias=self.dt_bias,
                                a_log=self.a_log, unit_eps=self.unit_eps, q_scale=float(self.dim) ** -0.5)
        else:
            K.delta_scan(q, k, v, beta, a, self.dt_bias, self.a_log, state, ctx.cu_seqlens, ctx.slots, ctx.n_seq, o,
                         self.heads, self.kv_heads, self.dim, self.vdim, self.unit_eps, float(self.dim) ** -0.5)
        y = ws.alloc((T, self.v_dim), proj.dtype)
        here.wait_stream(side)
        K.gated_norm(o, gate, 1.0, None, self.norm_w, self.norm_eps, self.heads, True, y, gate="sigmoid")
        streaming.linear(y, self.w_out, out, ctx)


class DecayLinearAttention(_StackedInput):
    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, decay: Sequence[float], norm_eps: float):
        if len(decay) != heads:
            raise ValueError("one decay per head")
        if dim > K.RECURRENT_MAX_KEY_DIM:
            raise ValueError(f"the recurrence kernels take key sizes up to {K.RECURRENT_MAX_KEY_DIM}, got {dim}")
        self.hidden_size = int(hidden_size)
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        self.decay_values = tuple(float(a) for a in decay)
        self.norm_eps = float(norm_eps)
        self.qk_dim, self.v_dim = self.heads * self.dim, self.heads * self.vdim

    def param_specs(self) -> List[ParamSpec]:
        D = self.hidden_size
        return [ParamSpec("q", (self.qk_dim, D)), ParamSpec("k", (self.qk_dim, D)), ParamSpec("v", (self.v_dim, D)),
                ParamSpec("g", (self.v_dim, D)), ParamSpec("o", (D, self.v_dim)),
                ParamSpec("norm", (self.v_dim,), kind="vector", init=("ones",))]

    def state_specs(self) -> List[StateSpec]:
        return [StateSpec.fixed("S", (self.heads, self.dim, self.vdim), "float32")]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.w_in = torch.cat([params["q"], params["k"], params["v"], params["g"]], dim=0).contiguous()
        self.w_out = params["o"].contiguous()
        self.norm_w = params["norm"].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.norm_w.device)

    def forward_projected(self, proj: Tensor, ctx, cache, out: Tensor) -> None:
        T = proj.shape[0]
        ws = ctx.workspace
        qk, vd = self.qk_dim, self.v_dim
        o = ws.alloc((T, vd), torch.float32)
        q, k, v = proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vd]
        state = cache.fixed(f"{self.name}.S")
        if _chunked(ctx, self.dim, False):
            scratch = ws.alloc((K.recurrent_chunked_scratch_floats(ctx.new_lens, self.heads, self.dim, self.vdim, False),),
                               torch.float32)
            K.recurrent_chunked(q, k, v, state, ctx.cu_seqlens, ctx.slots, ctx.new_lens, o, scratch, self.heads,
                                self.heads, self.dim, self.vdim, decay=self.decay)
        else:
            K.decay_scan(q, k, v, self.decay, state, ctx.cu_seqlens, ctx.slots, ctx.n_seq, o, self.heads, self.dim,
                         self.vdim)
        y = ws.alloc((T, vd), proj.dtype)
        K.gated_norm(o, proj[:, 2 * qk + vd:], 1.0, None, self.norm_w, self.norm_eps, 1, True, y, gate="sigmoid")
        streaming.linear(y, self.w_out, out, ctx)


register_mixer("gated_delta", GatedDeltaMixer)
register_mixer("decay_linear_attention", DecayLinearAttention)
