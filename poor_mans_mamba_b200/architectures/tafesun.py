"""Tafesun: a decoder-only model of parallel layers with routed feed-forwards.

    x = embed[token]
    per layer:  x <- x + post(left_scale * attention(pre(x)) + right_scale * state_space(pre(x)))
                x <- x + post(routed_feed_forward(pre(x)))            (where the layer has one)
    logits = logit_scale * embed . norm(x)

Every norm is the statistic-free tanh norm (`parts.norm.TanhNorm`), before and after each sublayer.
Left: causal softmax attention with biased projections, rotation of the first rot.dims entries of a
head in the half layout with linearly scaled frequencies, a scale from the configuration and a
sigmoid output gate (`parts.gated_attention`).  Right: the Mamba-2 mixer with its gated norm in
norm_groups parts, the gate before the norm (`parts.mamba2`).  Feed-forward: a mixture of clamped
gated experts with a shared one (`parts.moe`).  A layer may use another layer's tensors
(``weights_of``) with a cache and state of its own: it is that layer run once more on another cache.

This module only describes the model: parts by name with their constants, tensor names and the
order of layers.  The parts themselves do not know this architecture.
"""
from __future__ import annotations

from ..config.tafesun import TafesunConfig, TafesunLayerConfig
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..parts.block import prenorm_layer

# constants of the design
ACT_ALPHA = 1.702     # the experts' activation: g * sigmoid(ACT_ALPHA * g) * (u + ACT_SHIFT)
ACT_SHIFT = 1.0

_SSM_TENSORS = {"in_proj.weight": "in", "conv1d.weight": "conv", "conv1d.bias": "conv.b", "out_proj.weight": "o",
                "norm.weight": "norm"}


def _norm(name: str) -> PartSpec:
    return PartSpec("tanh_norm", name, {"tensor": ""})


def _mixers(layer: TafesunLayerConfig, eps: float):
    left, right = layer.left, layer.right
    return (
        PartSpec("rotary_gated_attention", "mix.left", {
            "heads": left.heads, "kv_heads": left.kv_heads, "dim": left.dim, "vdim": left.vdim,
            "rot_dims": left.rot_dims, "rot_base": left.rot_base, "rot_factor": left.rot_factor,
            "rot_layout": "halves", "scale": left.scale, "bias": True, "gate": True,
            "out_multiplier": layer.left_scale}),
        PartSpec("mamba2", "mix.right", {
            "n_heads": right.heads, "d_head": right.vdim, "d_state": right.state, "d_conv": right.conv,
            "n_groups": right.groups, "conv_bias": True, "proj_bias": False, "gated_norm": True,
            "norm_before_gate": False, "norm_eps": eps, "norm_groups": right.norm_groups,
            "out_multiplier": layer.right_scale, "tensors": _SSM_TENSORS}),
    )


def model_spec(cfg: TafesunConfig) -> ModelSpec:
    layers, index_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        ffn = ffn_norm = ffn_post = None
        if layer.mlp is not None:
            m = layer.mlp
            ffn = PartSpec("routed_glu", "mlp", {
                "experts": m.experts, "top": m.top, "expert_ff": m.expert_ff, "expert_limit": m.expert_limit,
                "shared_ff": m.shared_ff, "shared_limit": m.shared_limit, "act_alpha": ACT_ALPHA,
                "act_shift": ACT_SHIFT, "router_bias": True})
            ffn_norm, ffn_post = _norm("norm2"), _norm("norm2b")
        index_of[i] = len(layers)
        layers.append(prenorm_layer(f"l{i}.", _norm("norm1"), _mixers(layer, cfg.norm_eps), ffn_norm, ffn,
                                    mixer_post_norm=_norm("norm1b"), ffn_post_norm=ffn_post))
    # a layer that uses another's tensors is that layer run on a cache of its own
    order = tuple(LayerCall(index_of[cfg.weights_layer(i)], i) for i in range(len(cfg.layers)))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding_name="embed",
        embedding_multiplier=1.0,
        layers=tuple(layers),
        order=order,
        final_norm=_norm("final.norm"),
        head_name=None,
        head_multiplier=cfg.logit_scale,
        eos_token_id=-1,
        bos_token_id=0,
    )
