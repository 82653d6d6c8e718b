"""Configuration of the Kulesun design: a decoder-only model over a 32-bit residual with an RMS norm
(weight stored around zero, applied as 1 + w) before AND after every sublayer,

    x += norm_b(mixer(norm_a(x)));   x += norm_d(ff(norm_c(x)))

whose mixers are, layer by layer, either grouped-query attention without rotation (query temperature
by position, unit-RMS values mixed with the first such layer's values, capped scores, a unit sink in
the softmax, heads' weights mixed after the softmax, one output gate per head) or latent attention
(one cached latent and one rotated key part for all heads, scaled rotation in the half pairing,
element-wise output gate).  The feed-forward is a silu-gated MLP or absent; the output head is the
embedding table.  Every size, the layer order and the constants a model may choose are read from
config.json."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Union

from .model_config import register_config


@dataclass
class TalkingAttentionSpec:
    heads: int
    kv_heads: int
    dim: int                     # query/key size per head
    vdim: int                    # value size per head
    scale: float
    softcap: float               # 0 = scores are not capped
    temp_coef: float             # query temperature 1 + coef * ln(floor((p + 1) / every) + 1)
    temp_every: int              # 0 = no temperature
    v_mix: bool                  # values mixed with those of the first layer that says so


@dataclass
class RotationSpec:
    dims: int
    base: float
    factor: Optional[float] = None      # scaled rotation: stretch of the long wavelengths (None: unscaled)
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0


@dataclass
class GatedLatentSpec:
    heads: int
    dim: int                     # unrotated query/key coordinates per head
    rot_dim: int                 # rotated coordinates per head (one key part shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotationSpec


@dataclass
class DenseSpec:
    ff: int


@dataclass
class KulesunLayerSpec:
    type: str                                    # "attention" | "latent_attention"
    mixer: Union[TalkingAttentionSpec, GatedLatentSpec]
    mlp: Optional[DenseSpec]


@dataclass
class KulesunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: List[KulesunLayerSpec] = field(default_factory=list)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @property
    def first_v_mix_layer(self) -> Optional[int]:
        for i, L in enumerate(self.layers):
            if L.type == "attention" and L.mixer.v_mix:
                return i
        return None


def _attention(m: dict) -> TalkingAttentionSpec:
    heads, kv_heads = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
    if heads % kv_heads:
        raise ValueError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    temp = m.get("q_temp") or {}
    every = temp.get("every", 0) or 0
    if every != int(every) or every < 0:
        raise ValueError(f"query temperature step {every!r} must be a whole number of positions")
    return TalkingAttentionSpec(heads=heads, kv_heads=kv_heads, dim=int(m["dim"]), vdim=int(m["vdim"]),
                                scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                                temp_coef=float(temp.get("coef", 0.0)) if every else 0.0,
                                temp_every=int(every), v_mix=bool(m.get("v_mix", False)))


def _rotation(rot: dict, rot_dim: int) -> RotationSpec:
    dims = int(rot.get("dims", rot_dim))
    if dims % 2 or dims > rot_dim:
        raise ValueError(f"rotated coordinates {dims} must be even and at most {rot_dim}")
    spec = RotationSpec(dims=dims, base=float(rot.get("base", 10000.0)))
    sc = rot.get("scaling")
    if sc:
        spec.factor, spec.original = float(sc["factor"]), float(sc["original"])
        spec.fast, spec.slow = float(sc["fast"]), float(sc["slow"])
    return spec


def _latent(m: dict) -> GatedLatentSpec:
    rot_dim = int(m["rot_dim"])
    return GatedLatentSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=rot_dim, vdim=int(m["vdim"]),
                           kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                           rot=_rotation(m.get("rot") or {}, rot_dim))


def _mlp(f: Optional[dict]) -> Optional[DenseSpec]:
    if not f:
        return None
    if f.get("kind") != "dense":
        raise ValueError(f"unknown feed-forward kind {f.get('kind')!r}")
    return DenseSpec(ff=int(f["ff"]))


@register_config("Kulesun")
def kulesun_config(raw: dict) -> KulesunConfig:
    layers = []
    for i, L in enumerate(raw["layers"]):
        if L["type"] == "attention":
            mixer = _attention(L["mixer"])
        elif L["type"] == "latent_attention":
            mixer = _latent(L["mixer"])
        else:
            raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        layers.append(KulesunLayerSpec(type=L["type"], mixer=mixer, mlp=_mlp(L.get("mlp"))))
    cfg = KulesunConfig(vocab=int(raw["vocab"]), width=int(raw["width"]), eps=float(raw["norm"]["eps"]),
                        embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                        logit_scale=float(raw.get("logit_scale", 1.0)), layers=layers)
    first = cfg.first_v_mix_layer
    if first is not None:
        a = layers[first].mixer
        for i, L in enumerate(layers):
            if L.type == "attention" and L.mixer.v_mix and (L.mixer.kv_heads, L.mixer.vdim) != (a.kv_heads, a.vdim):
                raise ValueError(f"layer {i}: mixed values need the value heads and size of layer {first}")
    return cfg
