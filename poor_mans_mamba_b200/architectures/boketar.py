"""Boketar: a decoder-only model whose layers alternate two kinds of mixer.

    x = embed[token] * embedding.scale
    per layer (pre-norm, norm weights stored around zero):
        "channel_delta": the gated delta rule with a decay per key channel
        "parallel":      sliding-window softmax attention with a sink beside linear attention with a
                         fixed decay per head; half the sum of their outputs, each RMS-normed
        then, where the layer has one, a dense SwiGLU feed-forward
    logits = head norm(x)

With ``streams`` in the configuration the residual state is that many lanes joined by
hyper-connections (`parts.hyper`), otherwise one stream with plain residual sums.  This module
only describes the model: parts by name with their constants, tensor-name prefixes (``l<i>.``,
``mix``, ``mlp``, ``norm1``/``norm2``, ``hc1``/``hc2``, ``embed``, ``final.norm``, ``head``) and the
order of layers.  The parts themselves do not know this architecture.
"""
from __future__ import annotations

from ..config.boketar import BoketarConfig, BoketarLayerConfig
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..parts.block import prenorm_layer
from ..parts.hyper import hyper_layer

# constants of the design
UNIT_EPS = 1e-6          # inside the root when q and k of the delta rule are scaled to unit length
BRANCH_SCALE = 0.5       # the parallel mixer is half the sum of its two normed branches


def _mixer(layer: BoketarLayerConfig, eps: float) -> PartSpec:
    if layer.type == "channel_delta":
        c = layer.delta
        return PartSpec("gated_delta", "mix", {
            "heads": c.heads, "kv_heads": c.kv_heads, "dim": c.dim, "vdim": c.vdim, "conv": c.conv,
            "decay_rank": c.decay_rank, "gate_rank": c.gate_rank, "norm_eps": eps, "unit_eps": UNIT_EPS})
    left, right = layer.left, layer.right
    return PartSpec("normed_parallel", "mix", {"eps": eps, "scale": BRANCH_SCALE, "branches": [
        {"name": "left", "kind": "window_sink_attention", "params": {
            "heads": left.heads, "kv_heads": left.kv_heads, "dim": left.dim, "vdim": left.vdim, "conv": left.conv,
            "window": left.window, "rot_dims": left.rot_dims, "rot_base": left.rot_base, "scale": left.scale}},
        {"name": "right", "kind": "decay_linear_attention", "params": {
            "heads": right.heads, "dim": right.dim, "vdim": right.vdim, "decay": tuple(right.decay), "norm_eps": eps}},
    ]})


def model_spec(cfg: BoketarConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", name, {"eps": cfg.norm_eps, "offset": 1.0, "tensor": ""})

    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer = _mixer(layer, cfg.norm_eps)
        ffn = ffn_norm = None
        if layer.ff is not None:
            ffn = PartSpec("swiglu", "mlp", {"intermediate_size": layer.ff, "tensors": ("gate", "up", "down")})
            ffn_norm = norm("norm2")
        if cfg.streams is None:
            layers.append(prenorm_layer(f"l{i}.", norm("norm1"), (mixer,), ffn_norm, ffn))
        else:
            layers.append(hyper_layer(f"l{i}.", cfg.streams, norm("norm1"), mixer, ffn_norm, ffn))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding_name="embed",
        embedding_multiplier=cfg.embedding_scale,
        layers=tuple(layers),
        order=tuple(LayerCall(i, i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head_name="head",
        head_multiplier=1.0,
        eos_token_id=-1,
        bos_token_id=0,
        residual_lanes=cfg.streams,
    )
