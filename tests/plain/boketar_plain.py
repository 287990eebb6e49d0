"""Plain, slow Boketar forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Boketar tests.  It shares no code with the package: the configuration is a
plain dict, the weights a ``name -> tensor`` dict, and every formula runs directly on the CPU
in one floating-point type (float64 by default).  Notation: T tokens, D model width, linear
weights stored [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

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


def rms_unit(x: Tensor, eps: float) -> Tensor:
    """x over the root of (its mean square + eps), over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: Tensor, w: Tensor, eps: float) -> Tensor:
    """RMS norm whose weight is stored around zero."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x: Tensor, w: Tensor, eps: float) -> Tensor:
    return rms_unit(x, eps) * w


def causal_conv(u: Tensor, w: Tensor) -> Tensor:
    """u [T, C], w [C, taps]; the last column weighs the current token, zeros before the start:
    y[t] = sum_j w[:, j] * u[t - (taps - 1) + j]."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def rotate_pairs(x: Tensor, positions: Tensor, dims: int, base: float) -> Tensor:
    """x [T, H, d]: the first ``dims`` entries of every head are rotated in neighbouring pairs
    (2i, 2i+1) by the angle p * base^(-2i/dims); the rest pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# --------------------------------------------------------------------------- mixers
def windowed_sink_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, window: int, sink: Tensor) -> Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; token i sees j with 0 <= i - j < window; the softmax's
    denominator holds exp(sink_h) once more, a term without key or value."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + torch.exp(sink[h] - m)
            out[i, h] = (e[:, None] * v[lo:i + 1, g]).sum(dim=0) / den
    return out


def decayed_linear_attention(q: Tensor, k: Tensor, v: Tensor, decay: Sequence[float]) -> Tensor:
    """Per head S <- decay_h S + k v^T, o = S^T q.  q, k [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(d, v.shape[2], dtype=q.dtype)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.t() @ q[t, h]
    return out


def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, g: Tensor) -> Tensor:
    """q, k, g [T, H, d], v [T, H, dv], beta [T, H].  Per head, with S [d, dv]:
    S <- g S (row-wise); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, d = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(d, v.shape[2], dtype=q.dtype)
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.t() @ k[t, h])
            S = S + torch.outer(k[t, h], u)
            out[t, h] = S.t() @ q[t, h]
    return out


def channel_delta_mixer(h: Tensor, W: Dict[str, Tensor], p: str, m: dict, eps: float) -> Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(linear(h, W[p + "q"]), W[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(linear(h, W[p + "k"]), W[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(linear(h, W[p + "v"]), W[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(linear(h, W[p + "b"]))
    a = linear(linear(h, W[p + "a1"]), W[p + "a2"]) + W[p + "dt_bias"]
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * softplus(a).view(T, H, d))
    o = gated_delta_rule(q, k, v, beta, g)
    gate = torch.sigmoid(linear(linear(h, W[p + "g1"]), W[p + "g2"])).view(T, H, dv)
    o = rms_unit(o, eps) * W[p + "norm"] * gate
    return linear(o.reshape(T, H * dv), W[p + "o"])


def parallel_mixer(h: Tensor, W: Dict[str, Tensor], p: str, m: dict, eps: float, positions: Tensor) -> Tensor:
    T = h.shape[0]
    L, R = m["left"], m["right"]
    lp, rp = p + "left.", p + "right."
    H, G, d, dv = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
    q = causal_conv(linear(h, W[lp + "q"], W[lp + "q.b"]), W[lp + "q.conv"]).view(T, H, d)
    k = causal_conv(linear(h, W[lp + "k"], W[lp + "k.b"]), W[lp + "k.conv"]).view(T, G, d)
    v = causal_conv(linear(h, W[lp + "v"], W[lp + "v.b"]), W[lp + "v.conv"]).view(T, G, dv)
    q = rotate_pairs(q, positions, L["rot"]["dims"], L["rot"]["base"])
    k = rotate_pairs(k, positions, L["rot"]["dims"], L["rot"]["base"])
    a = windowed_sink_attention(q, k, v, L["scale"], L["mask"]["size"], W[lp + "sink"])
    left = linear(a.reshape(T, H * dv), W[lp + "o"], W[lp + "o.b"])

    Hr, dr, dvr = R["heads"], R["dim"], R["vdim"]
    qr = silu(linear(h, W[rp + "q"])).view(T, Hr, dr)
    kr = silu(linear(h, W[rp + "k"])).view(T, Hr, dr)
    vr = silu(linear(h, W[rp + "v"])).view(T, Hr, dvr)
    o = decayed_linear_attention(qr, kr, vr, R["decay"]).reshape(T, Hr * dvr)
    o = norm_plain(o, W[rp + "norm"], eps) * torch.sigmoid(linear(h, W[rp + "g"]))
    right = linear(o, W[rp + "o"])
    return 0.5 * (norm_plain(left, W[lp + "out"], eps) + norm_plain(right, W[rp + "out"], eps))


def dense_ff(h: Tensor, W: Dict[str, Tensor], p: str) -> Tensor:
    return linear(silu(linear(h, W[p + "gate"])) * linear(h, W[p + "up"]), W[p + "down"])


# --------------------------------------------------------------------------- the model
def forward(cfg: dict, W: Dict[str, Tensor], tokens: Sequence[int], dtype=torch.float64,
            layer_outputs: Optional[List[Tensor]] = None) -> Tensor:
    """Logits [T, vocab] of one sequence from position 0.  ``layer_outputs`` (a list) receives the
    residual stream (the sum of the streams) after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x0 = W["embed"][torch.tensor(list(tokens), dtype=torch.long)] * float(cfg["embedding"]["scale"])
    n_streams = cfg.get("streams")
    xs = [x0.clone() for _ in range(n_streams or 1)]

    def sublayer(xs, prefix, q, fn):
        if n_streams is None:
            return [xs[0] + fn(norm_one_plus(xs[0], W[f"{prefix}norm{q}"], eps))]
        w_in, w_out, w_mix = W[f"{prefix}hc{q}.in"], W[f"{prefix}hc{q}.out"], W[f"{prefix}hc{q}.mix"]
        u = sum(w_in[s] * xs[s] for s in range(n_streams))
        y = fn(norm_one_plus(u, W[f"{prefix}norm{q}"], eps))
        return [sum(w_mix[s, t] * xs[s] for s in range(n_streams)) + w_out[t] * y for t in range(n_streams)]

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "channel_delta":
            mix = lambda h: channel_delta_mixer(h, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            mix = lambda h: parallel_mixer(h, W, p + "mix.", layer["mixer"], eps, positions)
        else:
            raise ValueError(layer["type"])
        xs = sublayer(xs, p, 1, mix)
        if layer.get("mlp") is not None:
            xs = sublayer(xs, p, 2, lambda h: dense_ff(h, W, p + "mlp."))
        if layer_outputs is not None:
            layer_outputs.append(sum(xs))
    x = sum(xs)
    return linear(norm_one_plus(x, W["final.norm"], eps), W["head"])
