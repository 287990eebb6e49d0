"""Tiny Boketar configurations of the test-suite and model folders with random weights for them.

The three differ in every size and option: lanes of the residual state (3, none, 1), layer order,
layers with and without a feed-forward, widths that are no power of two, head counts and groups
(equal, grouped, a single key/value head), key sizes smaller and larger than value sizes,
convolutions of 1 to 5 taps, windows shorter and longer than a cache page and of one token,
rotation of part of a head, of all of it and of none, and decays close to and far from one.
"""
from __future__ import annotations

import copy
import json
import math
import os
import random
from typing import Dict, List, Tuple

import torch

BK_A = {
    "architecture": "Boketar", "vocab": 200, "width": 64, "streams": 3,
    "embedding": {"scale": 4.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 96}, "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "conv": 2, "mask": {"size": 24},
                     "rot": {"dims": 8, "base": 1000.0}, "scale": 0.3},
            "right": {"heads": 2, "dim": 16, "vdim": 24, "decay": [0.9, 0.995]}}},
        {"type": "channel_delta", "mlp": None, "mixer": {
            "heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "conv": 3, "decay_rank": 8, "gate_rank": 12}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 80}, "mixer": {
            "heads": 2, "kv_heads": 2, "dim": 40, "vdim": 48, "conv": 5, "decay_rank": 4, "gate_rank": 4}},
    ],
}

BK_B = {
    "architecture": "Boketar", "vocab": 333, "width": 96,
    "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 160}, "mixer": {
            "heads": 3, "kv_heads": 1, "dim": 32, "vdim": 40, "conv": 4, "decay_rank": 16, "gate_rank": 8}},
        {"type": "parallel", "mlp": None, "mixer": {
            "left": {"heads": 3, "kv_heads": 1, "dim": 32, "vdim": 16, "conv": 4, "mask": {"size": 100},
                     "rot": {"dims": 32, "base": 250000.0}, "scale": 0.2},
            "right": {"heads": 3, "dim": 8, "vdim": 8, "decay": [0.5, 0.97, 0.9995]}}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 64}, "mixer": {
            "left": {"heads": 2, "kv_heads": 2, "dim": 48, "vdim": 48, "conv": 3, "mask": {"size": 17},
                     "rot": {"dims": 16, "base": 100.0}, "scale": 0.125},
            "right": {"heads": 1, "dim": 64, "vdim": 32, "decay": [0.98]}}},
    ],
}

BK_C = {
    "architecture": "Boketar", "vocab": 97, "width": 48, "streams": 1,
    "embedding": {"scale": 7.0}, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "parallel", "mlp": None, "mixer": {
            "left": {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 16, "conv": 1, "mask": {"size": 1},
                     "rot": {"dims": 0, "base": 10000.0}, "scale": 1.0},
            "right": {"heads": 4, "dim": 4, "vdim": 12, "decay": [1.0, 0.25, 0.8, 0.999]}}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 32}, "mixer": {
            "heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 1, "decay_rank": 2, "gate_rank": 3}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 40}, "mixer": {
            "left": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 24, "conv": 2, "mask": {"size": 64},
                     "rot": {"dims": 6, "base": 5000.0}, "scale": 0.5},
            "right": {"heads": 2, "dim": 12, "vdim": 4, "decay": [0.9, 0.95]}}},
    ],
}

# Sizes at which the tensor-core and vector forms of the kernels are the ones that run: head sizes of 64 and
# 128 (with a value size that is padded), key sizes the chunked recurrences take, rows of whole 16-byte groups.
BK_M = {
    "architecture": "Boketar", "vocab": 1000, "width": 384, "streams": 4,
    "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 512}, "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 96, "conv": 3, "mask": {"size": 300},
                     "rot": {"dims": 64, "base": 100000.0}, "scale": 0.1},
            "right": {"heads": 4, "dim": 64, "vdim": 64, "decay": [0.9, 0.99, 0.999, 0.9999]}}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 768}, "mixer": {
            "heads": 4, "kv_heads": 2, "dim": 128, "vdim": 64, "conv": 4, "decay_rank": 32, "gate_rank": 16}},
        {"type": "parallel", "mlp": None, "mixer": {
            "left": {"heads": 8, "kv_heads": 1, "dim": 64, "vdim": 64, "conv": 2, "mask": {"size": 64},
                     "rot": {"dims": 64, "base": 10000.0}, "scale": 0.125},
            "right": {"heads": 2, "dim": 128, "vdim": 128, "decay": [0.97, 1.0]}}},
        {"type": "channel_delta", "mlp": None, "mixer": {
            "heads": 6, "kv_heads": 6, "dim": 64, "vdim": 128, "conv": 2, "decay_rank": 8, "gate_rank": 8}},
    ],
}

CONFIGS = {"A": BK_A, "B": BK_B, "C": BK_C, "M": BK_M}


def config(which: str) -> dict:
    return copy.deepcopy(CONFIGS[which])


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """name -> float32 tensor of bfloat16-representable values, written from the names and shapes the
    architecture's tensors have (no package code): matrices N(0, 1/in), so that every branch of a
    layer carries weight in the logits, norm weights around zero, sinks and biases of order one."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    n = cfg.get("streams")
    W: Dict[str, torch.Tensor] = {}

    def mat(name, out, inp, gain=1.0):
        W[name] = torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def vec(name, shape, std=1.0, mean=0.0):
        W[name] = torch.randn(shape, generator=g) * std + mean

    vec("embed", (V, D), 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        subs = [1] + ([2] if layer["mlp"] is not None else [])
        for q in subs:
            vec(f"{p}norm{q}", (D,), 0.2)
            if n is not None:
                W[f"{p}hc{q}.in"] = torch.rand(n, generator=g) * 0.8 + 0.3
                W[f"{p}hc{q}.out"] = torch.rand(n, generator=g) * 0.8 + 0.4
                W[f"{p}hc{q}.mix"] = torch.eye(n) * 0.7 + torch.rand(n, n, generator=g) * 0.3
        if layer["type"] == "channel_delta":
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for name, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                mat(p + "mix." + name, rows, D, 2.0)
                vec(p + f"mix.{name}.conv", (rows, taps), 0.6)
            mat(p + "mix.b", H, D, 2.0)
            W[p + "mix.A_log"] = torch.log(torch.rand(H, generator=g) * 3.0 + 0.3)
            vec(p + "mix.norm", (dv,), 0.2, 1.0)
            mat(p + "mix.a1", m["decay_rank"], D)
            mat(p + "mix.a2", H * d, m["decay_rank"], 2.0)
            vec(p + "mix.dt_bias", (H * d,), 1.0, -2.0)
            mat(p + "mix.g1", m["gate_rank"], D)
            mat(p + "mix.g2", H * dv, m["gate_rank"], 2.0)
            mat(p + "mix.o", D, H * dv)
        else:
            L, R = m["left"], m["right"]
            H, G, d, dv, taps = L["heads"], L["kv_heads"], L["dim"], L["vdim"], L["conv"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                mat(p + "mix.left." + name, rows, D, 2.0)
                vec(p + f"mix.left.{name}.b", (rows,), 0.3)
                vec(p + f"mix.left.{name}.conv", (rows, taps), 0.6)
            vec(p + "mix.left.sink", (H,), 1.5)
            mat(p + "mix.left.o", D, H * dv)
            vec(p + "mix.left.o.b", (D,), 0.3)
            Hr, dr, dvr = R["heads"], R["dim"], R["vdim"]
            mat(p + "mix.right.q", Hr * dr, D)
            mat(p + "mix.right.k", Hr * dr, D)
            mat(p + "mix.right.v", Hr * dvr, D)
            mat(p + "mix.right.g", Hr * dvr, D)
            mat(p + "mix.right.o", D, Hr * dvr)
            vec(p + "mix.right.norm", (Hr * dvr,), 0.2, 1.0)
            vec(p + "mix.left.out", (D,), 0.2, 1.0)
            vec(p + "mix.right.out", (D,), 0.2, 1.0)
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            mat(p + "mlp.gate", F, D)
            mat(p + "mlp.up", F, D)
            mat(p + "mlp.down", D, F)
    vec("final.norm", (D,), 0.2)
    mat("head", V, D)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in W.items()}


def make_model_dir(which: str, out_dir: str, seed: int = 0, patch=None) -> Tuple[str, dict, Dict[str, torch.Tensor]]:
    """(folder, config dict, float32 weights by name).  The folder's config.json does not carry the
    low-rank sizes: the engine has to take them from the tensors' shapes."""
    from poor_mans_mamba_b200.weights import save_file
    cfg = config(which)
    if patch:
        patch(cfg)
    weights = make_weights(cfg, seed)
    stored = copy.deepcopy(cfg)
    for layer in stored["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(stored, fh)
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()}, os.path.join(out_dir, "model.safetensors"))
    return out_dir, cfg, weights


def sequences(cfg: dict, lengths, seed: int = 0) -> List[List[int]]:
    rng = random.Random(seed)
    return [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in lengths]
