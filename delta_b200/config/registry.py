"""One registry from the architecture name in config.json to its configuration
class and to the function that turns a configuration into a model.

The reference picks sizes by matching the checkpoint's directory name against a
table (DELTA/Engine/DELTA/model.py:57-69) and always builds its one
``Transformer``; here the name in ``architectures`` decides, and an unknown name
is an error that lists the known ones.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, Optional

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable  # dict of config.json -> typed configuration
    build_spec: Callable        # (configuration, EngineConfig) -> ModelSpec
    sizes_from_shapes: Optional[Callable] = None   # (dict of config.json, {tensor name: shape}) -> dict with the sizes filled in that
                                                   # config.json leaves to the tensors' shapes (None: config.json says everything)


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict: Callable, build_spec: Callable, sizes_from_shapes: Optional[Callable] = None) -> None:
    ARCHITECTURES[name] = Architecture(name, config_from_dict, build_spec, sizes_from_shapes)


def unregister_architecture(name: str) -> None:
    ARCHITECTURES.pop(name, None)


def architecture_of(config_json: dict) -> Architecture:
    archs = config_json.get("architectures") or []
    if not archs and isinstance(config_json.get("architecture"), str):
        archs = [config_json["architecture"]]      # some designs name themselves in the singular
    if not archs:
        raise ConfigError("config.json has no 'architectures' (nor 'architecture')")
    name = archs[0]
    if name not in ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; known: {', '.join(sorted(ARCHITECTURES))}")
    return ARCHITECTURES[name]


def read_config(folder):
    """(architecture, typed configuration) of a model folder."""
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {folder}")
    raw = json.loads(path.read_text())
    arch = architecture_of(raw)
    if arch.sizes_from_shapes is not None:
        from ..weights.safetensors_io import open_model_files
        shapes = {}
        for f in open_model_files(folder):
            for n in f.names():
                shapes[n] = tuple(f.info(n)[0])
            f.close()
        raw = arch.sizes_from_shapes(raw, shapes)
    return arch, arch.config_from_dict(raw)
