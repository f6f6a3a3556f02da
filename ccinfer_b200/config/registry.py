"""One registry from an architecture's name (config.json ``architectures[0]``) to its model.

7QiC/ccInfer routes every name containing "Qwen" to its one model
(src/model/config.h:44-53, src/model/registry.cpp:30-34); here the name must
match exactly and an unknown one is ModelUnsupportedArch.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Callable, Dict, Optional

from ..errors import ModelConfigInvalid, ModelLoadFailed, ModelUnsupportedArch


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], object]   # config.json dict -> typed configuration
    build_plan: Callable[[object], object]   # typed configuration -> ModelPlan
    # (typed configuration, {tensor name: shape} of a checkpoint) -> typed configuration, for sizes that the
    # file of an architecture leaves to its tensors' shapes; None where config.json says everything
    complete_config: Optional[Callable[[object, dict], object]] = None


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_plan, replace: bool = False, complete_config=None) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _REGISTRY[name] = Architecture(name, parse_config, build_plan, complete_config)


def registered_architectures():
    _builtin()
    return sorted(_REGISTRY)


def _builtin():
    if "Qwen3ForCausalLM" not in _REGISTRY:
        from ..architectures import qwen3
        from .qwen3 import Qwen3Config
        register_architecture("Qwen3ForCausalLM", Qwen3Config.from_json, qwen3.build_plan)
    if "Tugelorn" not in _REGISTRY:
        from ..architectures import tugelorn
        from .tugelorn import TugelornConfig
        register_architecture("Tugelorn", TugelornConfig.from_json, tugelorn.build_plan,
                              complete_config=lambda cfg, shapes: cfg.with_shapes(shapes))
    if "Burolorn" not in _REGISTRY:
        from ..architectures import burolorn
        from .burolorn import BurolornConfig
        register_architecture("Burolorn", BurolornConfig.from_json, burolorn.build_plan)
    if "Gevovik" not in _REGISTRY:
        from ..architectures import gevovik
        from .gevovik import GevovikConfig
        register_architecture("Gevovik", GevovikConfig.from_json, gevovik.build_plan,
                              complete_config=lambda cfg, shapes: cfg.with_shapes(shapes))
    if "Dufizen" not in _REGISTRY:
        from ..architectures import dufizen
        from .dufizen import DufizenConfig
        register_architecture("Dufizen", DufizenConfig.from_json, dufizen.build_plan,
                              complete_config=lambda cfg, shapes: cfg.with_shapes(shapes))


def architecture_of(config_json: dict) -> Architecture:
    _builtin()
    archs = config_json.get("architectures")
    if archs is None and isinstance(config_json.get("architecture"), str):
        archs = [config_json["architecture"]]   # files that name their one architecture as a plain string
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ModelUnsupportedArch("config.json: 'architectures' must be a list that starts with a name "
                                   "(or 'architecture' a name)")
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
    cfg = arch.parse_config(j)
    if arch.complete_config is not None:
        from ..weights.loader import open_checkpoint
        f, _ = open_checkpoint(model_dir)
        try:
            cfg = arch.complete_config(cfg, {name: tuple(e[1]) for name, e in f.entries.items()})
        finally:
            f.close()
    return arch, cfg
