"""Model folder -> configuration object.  A folder holds `config.json` and `model.safetensors`; the
architecture name in config.json ("architecture", or the first entry of "architectures") selects
both the configuration class here and the model class in models/registry.py — the role of the
reference's ModelConfig (python/sglang/srt/configs/model_config.py)."""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict

_CONFIG_CLASSES: Dict[str, Callable[[dict], Any]] = {}


def register_config(architecture: str):
    def deco(fn):
        _CONFIG_CLASSES[architecture] = fn
        return fn
    return deco


def architecture_of(raw: dict) -> str:
    if "architecture" in raw:
        return str(raw["architecture"])
    archs = raw.get("architectures")
    if archs:
        return str(archs[0])
    raise ValueError("config.json names no architecture")


class ModelConfig:
    def __init__(self, model_path: str):
        self.model_path = model_path
        with open(os.path.join(model_path, "config.json")) as f:
            self.raw = json.load(f)
        self.architecture = architecture_of(self.raw)
        from . import desirax, dozetar, kisilix, kulesun  # noqa: F401  (register their configuration classes)

        if self.architecture not in _CONFIG_CLASSES:
            raise ValueError(f"no configuration class for architecture {self.architecture!r}; known: "
                             f"{sorted(_CONFIG_CLASSES)}")
        self.hf_config = _CONFIG_CLASSES[self.architecture](self.raw)

    @property
    def weights_path(self) -> str:
        return os.path.join(self.model_path, "model.safetensors")
