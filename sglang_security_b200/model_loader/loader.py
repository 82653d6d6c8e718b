"""Build a registered model from a model folder: configuration -> model class -> parameters on the
device -> weights streamed from the safetensors file (model_loader/loader.py DefaultModelLoader of
the reference, without the download and quantisation branches)."""
from __future__ import annotations

import torch

from ..configs.model_config import ModelConfig
from ..models.registry import resolve_model_cls
from .safetensors_reader import SafetensorsFile


def load_model(model_config: ModelConfig, device: str, dtype: torch.dtype):
    cls = resolve_model_cls(model_config.architecture)
    f = SafetensorsFile(model_config.weights_path)
    if hasattr(model_config.hf_config, "resolve_shapes"):
        # sizes that config.json leaves to the tensors' shapes
        model_config.hf_config.resolve_shapes({name: f.shape(name) for name in f.keys()})
    with torch.device(device):
        model = cls(model_config.hf_config, params_dtype=dtype)
    model = model.to(device)
    try:
        model.load_weights((name, t.to(device)) for name, t in f.items())
    finally:
        f.close()
    return model.eval()
