"""One registry from an architecture's name (config.json ``architectures[0]``) to its model.

7QiC/ccInfer routes every name containing "Qwen" to its one model
(src/model/config.h:44-53, src/model/registry.cpp:30-34); here the name must
match exactly and an unknown one is ModelUnsupportedArch.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Callable, Dict

from ..errors import ModelConfigInvalid, ModelLoadFailed, ModelUnsupportedArch


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], object]   # config.json dict -> typed configuration
    build_plan: Callable[[object], object]   # typed configuration -> ModelPlan


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_plan, replace: bool = False) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _REGISTRY[name] = Architecture(name, parse_config, build_plan)


def registered_architectures():
    _builtin()
    return sorted(_REGISTRY)


def _builtin():
    if "Qwen3ForCausalLM" not in _REGISTRY:
        from ..architectures import qwen3
        from .qwen3 import Qwen3Config
        register_architecture("Qwen3ForCausalLM", Qwen3Config.from_json, qwen3.build_plan)


def architecture_of(config_json: dict) -> Architecture:
    _builtin()
    archs = config_json.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ModelUnsupportedArch("config.json: 'architectures' must be a list that starts with a name")
    arch = _REGISTRY.get(archs[0])
    if arch is None:
        raise ModelUnsupportedArch(f"architecture '{archs[0]}' is not registered (known: {sorted(_REGISTRY)})")
    return arch


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path) as f:
            j = json.load(f)
    except OSError as e:
        raise ModelLoadFailed(f"cannot read {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise ModelConfigInvalid(f"{path} is not valid JSON: {e}") from e
    if not isinstance(j, dict):
        raise ModelConfigInvalid(f"{path} does not hold a JSON object")
    return j


def load_config(model_dir: str):
    """(architecture, typed configuration) of a model folder."""
    j = read_config_json(model_dir)
    arch = architecture_of(j)
    return arch, arch.parse_config(j)
