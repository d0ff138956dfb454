"""One registry from the architecture name in config.json to the model recipe."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

from ..config.errors import ConfigError, UnknownArchitectureError
from ..parts.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    """`config_from_dict` reads config.json's keys into a typed configuration (any object:
    only `build_spec` looks inside it); `build_spec` turns that configuration into a
    `ModelSpec`, the description of parts that everything else works from: loader, cache,
    step, generation, command line and replay read sizes, stop tokens and the longest
    sequence from the `ModelSpec` alone.  `sizes_from_shapes` (optional) is for a design whose config.json
    leaves a size to the shape of a stored tensor: given config.json's content and the folder's tensor shapes
    (name -> shape) it returns the content with those sizes filled in; it runs before `config_from_dict`
    wherever a model folder is opened (`complete_config`)."""
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]
    sizes_from_shapes: Optional[Callable[[Mapping[str, Any], Mapping[str, Tuple[int, ...]]], Mapping[str, Any]]] = None


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    ARCHITECTURES[arch.name] = arch
    return arch


def architecture_for(config_dict: Mapping[str, Any]) -> Architecture:
    """Look the model up by config.json["architectures"][0], or by config.json["architecture"] (one name)."""
    archs = config_dict.get("architectures")
    if archs is None and isinstance(config_dict.get("architecture"), str):
        archs = [config_dict["architecture"]]
    if not archs or not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names (or 'architecture' one "
                          f"name); known architectures: {sorted(ARCHITECTURES)}")
    name = archs[0]
    if name not in ARCHITECTURES:
        raise UnknownArchitectureError(
            f"config.json names architecture '{name}', which is not registered; "
            f"known architectures: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[name]


def complete_config(config_dict: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Mapping[str, Any]:
    """config.json's content with the sizes that only tensor shapes give filled in (see `Architecture`)."""
    arch = architecture_for(config_dict)
    if arch.sizes_from_shapes is None:
        return config_dict
    return arch.sizes_from_shapes(config_dict, shapes)
