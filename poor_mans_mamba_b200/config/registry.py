"""One registry from an architecture's name to its configuration reader and model
description (reference src/runtime/model_registry.cpp:74-113: ``model_type`` -> parse +
create_runner, unknown types are refused by name)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Sequence, Tuple

from .base import ConfigError, load_config_json


@dataclass(frozen=True)
class Architecture:
    """``reads_tensor_shapes``: some sizes of the architecture are given by no configuration key but by
    a tensor's shape; ``parse_config`` then takes a second argument, the model folder's
    ``name -> shape`` table (None when there is no folder yet: the configuration must then say them)."""
    name: str
    parse_config: Callable[..., Any]
    model_spec: Callable[[Any], Any]
    reads_tensor_shapes: bool = False

    def parse(self, data: Dict[str, Any], shapes=None):
        return self.parse_config(data, shapes) if self.reads_tensor_shapes else self.parse_config(data)


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable[..., Any],
                          model_spec: Callable[[Any], Any], aliases: Sequence[str] = (),
                          reads_tensor_shapes: bool = False) -> None:
    arch = Architecture(name, parse_config, model_spec, reads_tensor_shapes)
    for key in (name, *aliases):
        _ARCHITECTURES[key] = arch


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted({a.name for a in _ARCHITECTURES.values()}))


def resolve_architecture(config: Dict[str, Any]) -> Architecture:
    """By ``model_type``, else by the first known entry of ``architectures``, else by
    ``architecture`` (a single name)."""
    mt = config.get("model_type")
    if isinstance(mt, str) and mt in _ARCHITECTURES:
        return _ARCHITECTURES[mt]
    for name in config.get("architectures") or []:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    one = config.get("architecture")
    if isinstance(one, str):
        if one in _ARCHITECTURES:
            return _ARCHITECTURES[one]
        mt = mt or one
    if mt is None:
        raise ConfigError("config field 'model_type': missing")
    raise ConfigError(f"unsupported model_type: {mt} (known: {', '.join(registered_architectures())})")


def open_model_dir(model_dir: str):
    """(architecture, typed config) of the model folder."""
    data = load_config_json(model_dir)
    arch = resolve_architecture(data)
    shapes = None
    if arch.reads_tensor_shapes:
        from ..weights.safetensors_io import ModelFiles, SafetensorsError
        try:
            files = ModelFiles(model_dir)
        except SafetensorsError:
            files = None
        if files is not None:
            try:
                shapes = {k: tuple(files.info(k)[1]) for k in files.keys()}
            finally:
                files.close()
    return arch, arch.parse(data, shapes)
