"""Tiny Tafesun configurations of the test-suite and model folders with random weights for them.

They differ in every size and option: widths that are and are not multiples of 8 (the routed
products then run on the tensor cores or in float), grouped and ungrouped heads, key sizes smaller
and larger than value sizes, rotation of a part of the head, of all of it and of none, with and
without scaled frequencies, state groups and norm parts of one and of several, convolutions of 1 to
5 taps, routers that choose one expert, some and all, layers with and without a feed-forward or a
shared expert, and layers that use the tensors of an earlier or a later layer.
"""
from __future__ import annotations

import copy
import json
import math
import os
import random
from typing import Dict, List, Tuple

import torch


def _layer(left, right, ls, rs, mlp, weights_of=None):
    d = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


_A_LEFT = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3,
           "rot": {"dims": 8, "base": 1000.0, "scaling": {"factor": 2.0}}}
_A_RIGHT = {"heads": 3, "vdim": 16, "state": 24, "groups": 1, "conv": 3, "norm_groups": 3}
_A_MLP = {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 40, "limit": 1.5},
          "shared": {"ff": 56, "limit": 3.0}}
_A_LEFT2 = {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 16, "scale": 0.2,
            "rot": {"dims": 32, "base": 50000.0, "scaling": {"factor": 8.0}}}
_A_RIGHT2 = {"heads": 4, "vdim": 8, "state": 16, "groups": 2, "conv": 4, "norm_groups": 2}

TF_A = {
    "architecture": "Tafesun", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "layers": [
        _layer(_A_LEFT, _A_RIGHT, 0.8, 1.3, _A_MLP),
        _layer(_A_LEFT2, _A_RIGHT2, 1.5, 0.6, None),
        _layer(_A_LEFT, _A_RIGHT, 0.8, 1.3, _A_MLP, weights_of=0),
    ],
}

_B_LEFT = {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 32, "scale": 0.15, "rot": {"dims": 16, "base": 100.0}}
_B_RIGHT = {"heads": 4, "vdim": 24, "state": 8, "groups": 4, "conv": 2, "norm_groups": 1}
_B_MLP = {"kind": "moe", "router": {"experts": 3, "top": 3}, "expert": {"ff": 24, "limit": 0.75}}
_B_MLP2 = {"kind": "moe", "router": {"experts": 9, "top": 1}, "expert": {"ff": 16, "limit": 2.5},
           "shared": {"ff": 8, "limit": 0.5}}

TF_B = {
    "architecture": "Tafesun", "vocab": 130, "width": 100, "norm": {"eps": 1e-6}, "logit_scale": 3.0,
    "layers": [
        _layer(_B_LEFT, _B_RIGHT, 1.0, 1.0, _B_MLP2, weights_of=2),   # a later layer's tensors
        _layer(_B_LEFT, _B_RIGHT, 2.0, 0.25, _B_MLP),
        _layer(_B_LEFT, _B_RIGHT, 1.0, 1.0, _B_MLP2),
        _layer(_B_LEFT, _B_RIGHT, 1.0, 1.0, _B_MLP2, weights_of=0),   # through a layer that itself borrows
    ],
}

_C_LEFT = {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 40, "scale": 1.0, "rot": {"dims": 0, "base": 10000.0}}
_C_RIGHT = {"heads": 1, "vdim": 4, "state": 4, "groups": 1, "conv": 1, "norm_groups": 2}
_C_LEFT2 = {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 8, "scale": 0.25,
            "rot": {"dims": 24, "base": 300.0, "scaling": {"factor": 1.0}}}
_C_RIGHT2 = {"heads": 2, "vdim": 12, "state": 40, "groups": 2, "conv": 5, "norm_groups": 4}
_C_MLP = {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 12, "limit": 4.0},
          "shared": {"ff": 20, "limit": 1.0}}

TF_C = {
    "architecture": "Tafesun", "vocab": 97, "width": 44, "norm": {"eps": 1e-4}, "logit_scale": 1.0,
    "layers": [
        _layer(_C_LEFT, _C_RIGHT, 1.0, 2.0, None),
        _layer(_C_LEFT2, _C_RIGHT2, 0.5, 0.5, _C_MLP),
    ],
}

# Sizes at which the tensor-core forms of the kernels are the ones that run: head sizes of 64 and 128
# (a padded value size), head and state sizes the chunked scan takes, expert rows of whole 128-byte pieces
# (the tcgen05 grouped products in prompt steps, the mma.sync ones in decode steps).
_M_LEFT = {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09,
           "rot": {"dims": 64, "base": 100000.0, "scaling": {"factor": 2.0}}}
_M_RIGHT = {"heads": 8, "vdim": 64, "state": 64, "groups": 2, "conv": 4, "norm_groups": 4}
_M_MLP = {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": 128, "limit": 2.0},
          "shared": {"ff": 256, "limit": 4.0}}
_M_LEFT2 = {"heads": 4, "kv_heads": 4, "dim": 64, "vdim": 64, "scale": 0.125, "rot": {"dims": 32, "base": 10000.0}}
_M_RIGHT2 = {"heads": 4, "vdim": 32, "state": 128, "groups": 1, "conv": 3, "norm_groups": 1}

TF_M = {
    "architecture": "Tafesun", "vocab": 1000, "width": 384, "norm": {"eps": 1e-6}, "logit_scale": 1.5,
    "layers": [
        _layer(_M_LEFT, _M_RIGHT, 1.1, 0.7, _M_MLP),
        _layer(_M_LEFT2, _M_RIGHT2, 0.9, 1.2, None),
        _layer(_M_LEFT, _M_RIGHT, 1.1, 0.7, _M_MLP, weights_of=0),
    ],
}

CONFIGS = {"A": TF_A, "B": TF_B, "C": TF_C, "M": TF_M}


def config(which: str) -> dict:
    return copy.deepcopy(CONFIGS[which])


def owner(cfg: dict, i: int) -> int:
    """The layer whose tensors layer i uses."""
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """name -> float32 tensor of bfloat16-representable values, written from the names and shapes the
    architecture's tensors have (no package code): matrices N(0, gain / in), so that every branch of
    a layer carries weight in the logits; norms with weights around one, biases and alphas of order one."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    W: Dict[str, torch.Tensor] = {}

    def mat(name, out, inp, gain=1.0):
        W[name] = torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def vec(name, shape, std=1.0, mean=0.0):
        W[name] = torch.randn(shape, generator=g) * std + mean

    def norm(name, width):
        vec(name, (width,), 0.2, 1.0)
        vec(name + ".b", (width,), 0.2)
        W[name + ".alpha"] = torch.rand((), generator=g) * 0.6 + 0.3

    vec("embed", (V, D), 1.0)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p = f"l{i}."
        L, R = layer["mixer"]["left"], layer["mixer"]["right"]
        norm(p + "norm1", D)
        norm(p + "norm1b", D)
        H, G, d, dv = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
        for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            mat(p + "mix.left." + name, rows, D, 1.2)
            vec(p + f"mix.left.{name}.b", (rows,), 0.3)
        mat(p + "mix.left.g", H * dv, D, 1.2)
        mat(p + "mix.left.o", D, H * dv)
        Hr, P, N, Gr, taps = R["heads"], R["vdim"], R["state"], R["groups"], R["conv"]
        inner, gn = Hr * P, Gr * N
        mat(p + "mix.right.in", 2 * inner + 2 * gn + Hr, D, 1.0)
        vec(p + "mix.right.conv", (inner + 2 * gn, taps), 0.6)
        vec(p + "mix.right.conv.b", (inner + 2 * gn,), 0.2)
        vec(p + "mix.right.dt_bias", (Hr,), 1.0, -1.0)
        W[p + "mix.right.A_log"] = torch.log(torch.rand(Hr, generator=g) * 2.0 + 0.05)
        vec(p + "mix.right.D", (Hr,), 0.5, 1.0)
        vec(p + "mix.right.norm", (inner,), 0.2, 1.0)
        mat(p + "mix.right.o", D, inner)
        mlp = layer.get("mlp")
        if mlp is not None:
            norm(p + "norm2", D)
            norm(p + "norm2b", D)
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            mat(p + "mlp.router", E, D, 3.0)
            vec(p + "mlp.router.b", (E,), 0.5)
            for e in range(E):
                mat(p + f"mlp.e{e}.gate", F, D, 1.2)
                mat(p + f"mlp.e{e}.up", F, D, 1.2)
                mat(p + f"mlp.e{e}.down", D, F, 1.0)
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                mat(p + "mlp.shared.gate", Fs, D, 1.2)
                mat(p + "mlp.shared.up", Fs, D, 1.2)
                mat(p + "mlp.shared.down", D, Fs)
    norm("final.norm", D)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in W.items()}


def make_model_dir(which, out_dir: str, seed: int = 0, patch=None, edit=None) -> Tuple[str, dict, Dict[str, torch.Tensor]]:
    """(folder, config dict, float32 weights by name).  ``patch(cfg)`` changes the configuration before the
    weights are made, ``edit(weights)`` the weights before they are stored."""
    from poor_mans_mamba_b200.weights import save_file
    cfg = config(which) if isinstance(which, str) else copy.deepcopy(which)
    if patch:
        patch(cfg)
    weights = make_weights(cfg, seed)
    if edit:
        edit(weights)
        weights = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in weights.items()}
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()}, os.path.join(out_dir, "model.safetensors"))
    return out_dir, cfg, weights


def decisive_routers(weights: Dict[str, torch.Tensor]) -> None:
    """Routers whose choice no rounding can turn: the logits' spread over tokens becomes small beside gaps of one
    between the experts' biases (in an order of its own in every layer), so that every token of a layer takes the
    same experts, with weights that still depend on the token.  bfloat16 runs are compared with the plain
    implementation under such routers: with freely routed tokens a few per cent of them choose between two
    experts whose logits differ by less than bfloat16 rounding moves them, and either choice is right."""
    for name in sorted(weights):
        if name.endswith("mlp.router"):
            weights[name] = weights[name] * 0.02
            E = weights[name].shape[0]
            order = torch.randperm(E, generator=torch.Generator().manual_seed(len(name) + E))
            weights[name + ".b"] = order.to(torch.float32) * 1.0 + weights[name + ".b"] * 0.05


def sequences(cfg: dict, lengths, seed: int = 0) -> List[List[int]]:
    rng = random.Random(seed)
    return [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in lengths]
