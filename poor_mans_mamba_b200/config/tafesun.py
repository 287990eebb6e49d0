"""Typed configuration of the Tafesun architecture, read from its own config.json keys.

    architecture: "Tafesun"; vocab, width; norm.eps; logit_scale;
    layers: [{type, mixer, mlp, weights_of?}], type "parallel";
      mixer: {left: {heads, kv_heads, dim, vdim, scale, rot: {dims, base, scaling: {factor}}},
              right: {heads, vdim, state, groups, conv, norm_groups}, left_scale, right_scale};
      mlp: null or {kind: "moe", router: {experts, top}, expert: {ff, limit}, shared: {ff, limit}};
      weights_of: j, the layer whose tensors this layer uses (its cache and state are its own).

Every size and constant comes from the file.  ``rot.scaling`` and ``mlp.shared`` may be absent (no
scaling of the rotation's frequencies, no shared expert).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader
from .boketar import _positive, _sub


@dataclass(frozen=True)
class GatedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_factor: float


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class RoutedConfig:
    experts: int
    top: int
    expert_ff: int
    expert_limit: float
    shared_ff: int          # 0: no shared expert
    shared_limit: float


@dataclass(frozen=True)
class TafesunLayerConfig:
    type: str
    left: GatedAttentionConfig
    right: StateSpaceConfig
    left_scale: float
    right_scale: float
    mlp: Optional[RoutedConfig]
    weights_of: Optional[int]   # None: the layer has tensors of its own


@dataclass(frozen=True)
class TafesunConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[TafesunLayerConfig, ...]

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself unless it names another)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config field 'layers[{i}].weights_of': the layers name each other in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    @staticmethod
    def from_dict(data: Dict[str, Any]) -> "TafesunConfig":
        top = KeyReader(data)
        vocab, width = _positive(top, "vocab", ""), _positive(top, "width", "")
        eps = KeyReader(_sub(data, "norm", "")).float("eps")
        logit_scale = top.float("logit_scale")
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config field 'layers': expected a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config field 'layers[{i}]': expected an object")
            kind = KeyReader(entry).str("type")
            if kind != "parallel":
                raise ConfigError(f"config field '{where}type': unknown layer type '{kind}' (known: parallel)")
            mixer = _sub(entry, "mixer", where)
            left = _gated_attention(_sub(mixer, "left", where + "mixer."), where + "mixer.left.")
            right = _state_space(_sub(mixer, "right", where + "mixer."), where + "mixer.right.")
            scales = KeyReader(mixer)
            try:
                left_scale, right_scale = scales.float("left_scale"), scales.float("right_scale")
            except ConfigError as exc:
                raise ConfigError(str(exc).replace("'left_scale'", f"'{where}mixer.left_scale'")
                                  .replace("'right_scale'", f"'{where}mixer.right_scale'")) from None
            mlp = _routed(_sub(entry, "mlp", where), where + "mlp.") if entry.get("mlp") is not None else None
            weights_of = KeyReader(entry).optional_int("weights_of")
            if weights_of is not None and not 0 <= weights_of < len(raw_layers):
                raise ConfigError(f"config field '{where}weights_of': names layer {weights_of}, which does not exist")
            layers.append(TafesunLayerConfig(kind, left, right, left_scale, right_scale, mlp, weights_of))
        cfg = TafesunConfig(vocab, width, eps, logit_scale, tuple(layers))
        for i, layer in enumerate(layers):
            j = cfg.weights_layer(i)
            own = layers[j]
            if (layer.left, layer.right, layer.left_scale, layer.right_scale, layer.mlp) != (
                    own.left, own.right, own.left_scale, own.right_scale, own.mlp):
                raise ConfigError(f"config field 'layers[{i}].weights_of': layer {i} differs from layer {j}, "
                                  "whose tensors it uses")
        return cfg


def _gated_attention(side: Dict[str, Any], where: str) -> GatedAttentionConfig:
    r = KeyReader(side)
    heads, kv = _positive(r, "heads", where), _positive(r, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config field '{where}heads': {heads} is no multiple of kv_heads {kv}")
    dim = _positive(r, "dim", where)
    rot = _sub(side, "rot", where)
    rot_dims = KeyReader(rot).int("dims")
    if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"config field '{where}rot.dims': an even number from 0 to dim = {dim}, got {rot_dims}")
    factor = 1.0
    if rot.get("scaling") is not None:
        factor = KeyReader(_sub(rot, "scaling", where + "rot.")).float("factor")
        if factor <= 0.0:
            raise ConfigError(f"config field '{where}rot.scaling.factor': must be positive, got {factor}")
    return GatedAttentionConfig(heads, kv, dim, _positive(r, "vdim", where), r.float("scale"), rot_dims,
                                KeyReader(rot).float("base"), factor)


def _state_space(side: Dict[str, Any], where: str) -> StateSpaceConfig:
    r = KeyReader(side)
    heads, groups = _positive(r, "heads", where), _positive(r, "groups", where)
    if heads % groups:
        raise ConfigError(f"config field '{where}heads': {heads} is no multiple of groups {groups}")
    vdim = _positive(r, "vdim", where)
    norm_groups = _positive(r, "norm_groups", where)
    if (heads * vdim) % norm_groups:
        raise ConfigError(f"config field '{where}norm_groups': {norm_groups} does not divide heads * vdim = {heads * vdim}")
    return StateSpaceConfig(heads, vdim, _positive(r, "state", where), groups, _positive(r, "conv", where), norm_groups)


def _routed(mlp: Dict[str, Any], where: str) -> RoutedConfig:
    kind = KeyReader(mlp).str("kind")
    if kind != "moe":
        raise ConfigError(f"config field '{where}kind': unknown feed-forward '{kind}' (known: moe)")
    router = KeyReader(_sub(mlp, "router", where))
    experts, top = _positive(router, "experts", where + "router."), _positive(router, "top", where + "router.")
    if top > experts:
        raise ConfigError(f"config field '{where}router.top': {top} is more than the {experts} experts")
    expert = KeyReader(_sub(mlp, "expert", where))
    shared_ff, shared_limit = 0, 0.0
    if mlp.get("shared") is not None:
        shared = KeyReader(_sub(mlp, "shared", where))
        shared_ff, shared_limit = _positive(shared, "ff", where + "shared."), shared.float("limit")
    return RoutedConfig(experts, top, _positive(expert, "ff", where + "expert."), expert.float("limit"),
                        shared_ff, shared_limit)
