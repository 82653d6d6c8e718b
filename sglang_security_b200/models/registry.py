"""Architecture name -> model class (the reference's ModelRegistry,
python/sglang/srt/models/registry.py).  A model class provides:

    __init__(config, params_dtype)          modules with empty parameters
    cache_spec() -> CacheSpec               what the runner must allocate (token pool rows, state rows)
    load_weights(iterable of (name, tensor))
    forward(input_ids, forward_batch) -> hidden [T, width]
    compute_logits(hidden_rows) -> [n, vocab]
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Type

_MODELS: Dict[str, Type] = {}


@dataclass
class CacheSpec:
    kind: str                                   # "latent" / "rows": one row per token and owning layer
    row_dims: Dict[int, int] = field(default_factory=dict)     # owning layer -> row width (layers
                                                               # without an entry cache nothing per token)
    source_of: Dict[int, int] = field(default_factory=dict)    # layer -> layer whose rows it reads
    state_widths: Dict[int, int] = field(default_factory=dict)  # layer -> fp32 carry width per sequence
    block_summaries: Dict[int, int] = field(default_factory=dict)  # layer -> tokens per summarised block


def register_model(architecture: str):
    def deco(cls):
        _MODELS[architecture] = cls
        return cls
    return deco


def resolve_model_cls(architecture: str):
    from . import desirax, dozetar, kisilix, kulesun  # noqa: F401  (register themselves)

    if architecture not in _MODELS:
        raise ValueError(f"architecture {architecture!r} is not supported; known: {sorted(_MODELS)}")
    return _MODELS[architecture]


def supported_architectures():
    from . import desirax, dozetar, kisilix, kulesun  # noqa: F401

    return sorted(_MODELS)
