"""One registry from an architecture's name to its configuration class and
its model builder (the reference: ``Arch.detect`` string table,
src/arch.zig:18-51, and the ``ModelStorage`` union, src/models/model.zig:492-532).

``config.json`` chooses the entry through ``architectures[0]`` or, failing
that, ``model_type``; an unknown name is an error that lists what is known.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from .base import ConfigError


@dataclass
class ArchitectureEntry:
    name: str
    config_class: Any                  # has from_dict(dict) and to_model_spec()
    weight_names: Callable[[Any], Dict[str, Any]]   # config -> WeightPlan (see models/)
    model_types: tuple = ()


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_class, weight_names, model_types=()) -> None:
    """Add an architecture; a second registration under one name replaces the first."""
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_class, weight_names, tuple(model_types))
    for mt in model_types:
        _MODEL_TYPES[mt] = name


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw_config: Dict[str, Any]) -> ArchitectureEntry:
    """The entry that a parsed config.json names."""
    names = raw_config.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    candidates = [raw_config.get("model_type")]
    tc = raw_config.get("text_config")
    if isinstance(tc, dict):
        candidates.append(tc.get("model_type"))
    for mt in candidates:
        if mt in _MODEL_TYPES:
            return _ARCHITECTURES[_MODEL_TYPES[mt]]
    raise ConfigError(
        f"unsupported architecture {names or raw_config.get('model_type')!r}; "
        f"registered: {', '.join(registered_architectures()) or '(none)'}")


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")
    with open(path, "r") as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None


def _shape_lookup(folder: str):
    """suffix -> shape of the folder's tensor whose name ends with it (the
    shortest such name), reading only the files' headers; None without files."""
    from ..weights.safetensors_io import SafetensorsError, SafetensorsFolder
    try:
        files = SafetensorsFolder(folder)
    except (SafetensorsError, OSError):
        return None

    def shapes(suffix: str):
        hits = [n for n in files.names() if n == suffix or n.endswith("." + suffix)]
        if not hits:
            return None
        return tuple(files.tensors[min(hits, key=len)].shape)
    return shapes


def load_config(folder: str):
    """(entry, typed config) of a model folder.  A configuration class whose
    ``from_dict`` takes ``shapes`` may read sizes that config.json omits from
    the checkpoint's tensor shapes."""
    import inspect
    raw = read_config_json(folder)
    entry = resolve_architecture(raw)
    from_dict = entry.config_class.from_dict
    if "shapes" in inspect.signature(from_dict).parameters:
        return entry, from_dict(raw, shapes=_shape_lookup(folder))
    return entry, from_dict(raw)
