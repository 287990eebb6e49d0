"""Plain, slow Tafesun forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Tafesun tests.  It shares no code with the package: the configuration is a
plain dict, the weights a ``name -> tensor`` dict, and every formula runs directly on the CPU in
one floating-point type (float64 by default).  Notation: T tokens, D model width, linear weights
stored [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------- small functions
def silu(x: Tensor) -> Tensor:
    return x * torch.sigmoid(x)


def softplus(x: Tensor) -> Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None) -> Tensor:
    y = x @ w.t()
    return y if b is None else y + b


def tanh_norm(x: Tensor, alpha: Tensor, w: Tensor, b: Tensor) -> Tensor:
    """The statistic-free norm: w * tanh(alpha x) + b, element by element."""
    return torch.tanh(alpha * x) * w + b


def rms_parts(x: Tensor, parts: int, eps: float) -> Tensor:
    """x [T, C] cut into ``parts`` equal pieces along C, each divided by sqrt(mean(piece^2) + eps)."""
    T, C = x.shape
    xs = x.reshape(T, parts, C // parts)
    xs = xs / torch.sqrt((xs * xs).mean(dim=-1, keepdim=True) + eps)
    return xs.reshape(T, C)


def causal_conv(u: Tensor, w: Tensor, b: Tensor) -> Tensor:
    """u [T, C], w [C, taps]: y[t] = b + sum_j w[:, j] u[t - (taps - 1) + j], zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = b.expand(T, C).clone()
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def rotate_halves(x: Tensor, positions: Tensor, dims: int, base: float, factor: float) -> Tensor:
    """x [T, H, d]: among the first ``dims`` entries of a head, entry i < dims/2 and entry i + dims/2
    turn by the angle p * base^(-2i/dims) / factor; entries from ``dims`` on stay."""
    half = dims // 2
    if half == 0:
        return x.clone()
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims) / factor
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# --------------------------------------------------------------------------- the left mixer
def causal_attention(q: Tensor, k: Tensor, v: Tensor, scale: float) -> Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H/G); token i
    sees every j <= i; plain softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def gated_attention(h: Tensor, w: Dict[str, Tensor], pre: str, c: dict, positions: Tensor) -> Tensor:
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = linear(h, w[pre + "q"], w[pre + "q.b"]).reshape(T, H, d)
    k = linear(h, w[pre + "k"], w[pre + "k.b"]).reshape(T, G, d)
    v = linear(h, w[pre + "v"], w[pre + "v.b"]).reshape(T, G, dv)
    rot = c["rot"]
    factor = float(rot.get("scaling", {}).get("factor", 1.0)) if rot.get("scaling") else 1.0
    q = rotate_halves(q, positions, rot["dims"], rot["base"], factor)
    k = rotate_halves(k, positions, rot["dims"], rot["base"], factor)
    o = causal_attention(q, k, v, c["scale"]).reshape(T, H * dv)
    o = o * torch.sigmoid(linear(h, w[pre + "g"]))
    return linear(o, w[pre + "o"])


# --------------------------------------------------------------------------- the right mixer
def selective_scan(x: Tensor, B: Tensor, C: Tensor, dt: Tensor, a_log: Tensor, d_skip: Tensor) -> Tensor:
    """x [T, H, P], B and C [T, G, N], dt [T, H] (already positive).  Per head, with its group's B, C:
    S_t = exp(-exp(a_log) dt_t) S_{t-1} + dt_t B_t x_t^T,  y_t = S_t^T C_t + d_skip x_t."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(x)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=x.dtype)
        a = torch.exp(a_log[hd])
        for t in range(T):
            S = torch.exp(-a * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.t() @ C[t, g] + d_skip[hd] * x[t, hd]
    return y


def state_space_mixer(h: Tensor, w: Dict[str, Tensor], pre: str, c: dict, eps: float) -> Tensor:
    T = h.shape[0]
    H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner, gn = H * P, G * N
    p = linear(h, w[pre + "in"])
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * gn], p[:, 2 * inner + 2 * gn:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + gn].reshape(T, G, N)
    C = xbc[:, inner + gn:].reshape(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    y = selective_scan(x, B, C, dt, w[pre + "A_log"], w[pre + "D"]).reshape(T, inner)
    y = rms_parts(y * silu(z), c["norm_groups"], eps) * w[pre + "norm"]
    return linear(y, w[pre + "o"])


# --------------------------------------------------------------------------- the feed-forward
def clamped_expert(h: Tensor, gate: Tensor, up: Tensor, down: Tensor, limit: float) -> Tensor:
    g = torch.clamp(linear(h, gate), max=limit)
    u = torch.clamp(linear(h, up), min=-limit, max=limit)
    return linear(g * torch.sigmoid(1.702 * g) * (u + 1.0), down)


def routed_experts(h: Tensor, w: Dict[str, Tensor], pre: str, c: dict) -> Tensor:
    E, top = c["router"]["experts"], c["router"]["top"]
    z = linear(h, w[pre + "router"], w[pre + "router.b"])
    val, idx = torch.topk(z, top, dim=-1)
    p = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += p[t, j] * clamped_expert(h[t:t + 1], w[f"{pre}e{e}.gate"], w[f"{pre}e{e}.up"],
                                               w[f"{pre}e{e}.down"], c["expert"]["limit"])[0]
    if c.get("shared"):
        out = out + clamped_expert(h, w[pre + "shared.gate"], w[pre + "shared.up"], w[pre + "shared.down"],
                                   c["shared"]["limit"])
    return out


# --------------------------------------------------------------------------- the model
def _norm(x: Tensor, w: Dict[str, Tensor], name: str) -> Tensor:
    return tanh_norm(x, w[name + ".alpha"], w[name], w[name + ".b"])


def forward(config: dict, weights: Dict[str, Tensor], tokens, dtype=torch.float64, layer_outputs: Optional[List] = None) -> Tensor:
    """Logits [T, vocab] of one whole sequence."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    eps = float(config["norm"]["eps"])
    x = w["embed"][tokens]
    for i, layer in enumerate(config["layers"]):
        src = i
        while config["layers"][src].get("weights_of") is not None:  # a layer may use another layer's tensors
            src = config["layers"][src]["weights_of"]
        L = f"l{src}."
        m = layer["mixer"]
        hn = _norm(x, w, L + "norm1")
        left = gated_attention(hn, w, L + "mix.left.", m["left"], positions)
        right = state_space_mixer(hn, w, L + "mix.right.", m["right"], eps)
        x = x + _norm(m["left_scale"] * left + m["right_scale"] * right, w, L + "norm1b")
        if layer.get("mlp") is not None:
            hn = _norm(x, w, L + "norm2")
            x = x + _norm(routed_experts(hn, w, L + "mlp.", layer["mlp"]), w, L + "norm2b")
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return linear(_norm(x, w, "final.norm"), w["embed"]) * float(config["logit_scale"])
