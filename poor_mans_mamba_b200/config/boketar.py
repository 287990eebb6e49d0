"""Typed configuration of the Boketar architecture, read from its own config.json keys.

    architecture: "Boketar"; vocab, width; embedding.scale; norm.eps; streams (optional: the number
    of residual lanes of the hyper-connections; absent: one plain residual stream);
    layers: [{type, mixer, mlp}], type "channel_delta" or "parallel", mlp null or {kind: "dense", ff}.

Every size and constant comes from the file; nothing is defaulted except what the layout of a
layer makes optional.  Two sizes are in no key: the inner widths of the channel_delta mixer's two
low-rank projections (decay: ``a1``/``a2``, output gate: ``g1``/``g2``).  They are read from the
shapes of ``<layer>.mix.a1`` and ``<layer>.mix.g1`` in the model folder; a configuration without a
folder (the random-weights mode) names them ``decay_rank`` and ``gate_rank`` in the mixer's dict.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, KeyReader


def _sub(data: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    val = data.get(key)
    if not isinstance(val, dict):
        raise ConfigError(f"config field '{where}{key}': expected an object")
    return val


def _positive(reader: KeyReader, key: str, where: str) -> int:
    try:
        v = reader.int(key)
    except ConfigError as exc:
        raise ConfigError(str(exc).replace(f"'{key}'", f"'{where}{key}'")) from None
    if v <= 0:
        raise ConfigError(f"config field '{where}{key}': must be positive, got {v}")
    return v


@dataclass(frozen=True)
class ChannelDeltaConfig:
    """Gated delta rule with a decay per key channel."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int


@dataclass(frozen=True)
class WindowAttentionConfig:
    """The parallel mixer's left side: softmax attention over a sliding window with a sink."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    window: int
    rot_dims: int
    rot_base: float
    scale: float


@dataclass(frozen=True)
class DecayAttentionConfig:
    """The parallel mixer's right side: linear attention with one decay per head."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class BoketarLayerConfig:
    type: str
    delta: Optional[ChannelDeltaConfig] = None
    left: Optional[WindowAttentionConfig] = None
    right: Optional[DecayAttentionConfig] = None
    ff: Optional[int] = None   # None: the layer has no feed-forward


@dataclass(frozen=True)
class BoketarConfig:
    vocab_size: int
    hidden_size: int
    embedding_scale: float
    norm_eps: float
    streams: Optional[int]
    layers: Tuple[BoketarLayerConfig, ...]

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_dict(data: Dict[str, Any], shapes: Optional[Mapping[str, Tuple[int, ...]]] = None) -> "BoketarConfig":
        top = KeyReader(data)
        vocab, width = _positive(top, "vocab", ""), _positive(top, "width", "")
        scale = KeyReader(_sub(data, "embedding", "")).float("scale")
        eps = KeyReader(_sub(data, "norm", "")).float("eps")
        streams = top.optional_int("streams")
        if streams is not None and not 1 <= streams <= 8:
            raise ConfigError(f"config field 'streams': 1 to 8 residual lanes, got {streams}")
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config field 'layers': expected a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config field 'layers[{i}]': expected an object")
            kind = KeyReader(entry).str("type")
            mixer = _sub(entry, "mixer", where)
            ff = None
            if entry.get("mlp") is not None:
                mlp = _sub(entry, "mlp", where)
                mlp_kind = KeyReader(mlp).str("kind")
                if mlp_kind != "dense":
                    raise ConfigError(f"config field '{where}mlp.kind': unknown feed-forward '{mlp_kind}' (known: dense)")
                ff = _positive(KeyReader(mlp), "ff", where + "mlp.")
            if kind == "channel_delta":
                layers.append(BoketarLayerConfig(kind, delta=_channel_delta(mixer, where + "mixer.", i, width, shapes), ff=ff))
            elif kind == "parallel":
                left = _window_attention(_sub(mixer, "left", where + "mixer."), where + "mixer.left.")
                right = _decay_attention(_sub(mixer, "right", where + "mixer."), where + "mixer.right.")
                layers.append(BoketarLayerConfig(kind, left=left, right=right, ff=ff))
            else:
                raise ConfigError(f"config field '{where}type': unknown layer type '{kind}' "
                                  "(known: channel_delta, parallel)")
        return BoketarConfig(vocab, width, scale, eps, streams, tuple(layers))


def _heads(r: KeyReader, where: str) -> Tuple[int, int]:
    heads, kv = _positive(r, "heads", where), _positive(r, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config field '{where}heads': {heads} is no multiple of kv_heads {kv}")
    return heads, kv


def _rank(mixer: Dict[str, Any], key: str, tensor: str, width: int, where: str, shapes) -> int:
    if shapes is not None and tensor in shapes:
        shape = tuple(shapes[tensor])
        if len(shape) != 2 or shape[1] != width:
            raise ConfigError(f"tensor '{tensor}' has shape {list(shape)}; expected [rank, {width}]")
        return int(shape[0])
    if mixer.get(key) is None:
        raise ConfigError(f"config field '{where}{key}': missing, and the model folder has no tensor '{tensor}' "
                          "whose shape would give it")
    return _positive(KeyReader(mixer), key, where)


def _channel_delta(mixer: Dict[str, Any], where: str, layer: int, width: int, shapes) -> ChannelDeltaConfig:
    r = KeyReader(mixer)
    heads, kv = _heads(r, where)
    return ChannelDeltaConfig(heads, kv, _positive(r, "dim", where), _positive(r, "vdim", where),
                              _positive(r, "conv", where),
                              _rank(mixer, "decay_rank", f"l{layer}.mix.a1", width, where, shapes),
                              _rank(mixer, "gate_rank", f"l{layer}.mix.g1", width, where, shapes))


def _window_attention(side: Dict[str, Any], where: str) -> WindowAttentionConfig:
    r = KeyReader(side)
    heads, kv = _heads(r, where)
    dim = _positive(r, "dim", where)
    rot = _sub(side, "rot", where)
    rot_dims = KeyReader(rot).int("dims")
    if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"config field '{where}rot.dims': an even number from 0 to dim = {dim}, got {rot_dims}")
    return WindowAttentionConfig(heads, kv, dim, _positive(r, "vdim", where), _positive(r, "conv", where),
                                 _positive(KeyReader(_sub(side, "mask", where)), "size", where + "mask."),
                                 rot_dims, KeyReader(rot).float("base"), r.float("scale"))


def _decay_attention(side: Dict[str, Any], where: str) -> DecayAttentionConfig:
    r = KeyReader(side)
    heads = _positive(r, "heads", where)
    decay = r.float_list("decay", heads)
    return DecayAttentionConfig(heads, _positive(r, "dim", where), _positive(r, "vdim", where), decay)
