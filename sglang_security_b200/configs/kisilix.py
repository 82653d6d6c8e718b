"""Configuration of the Kisilix design: a decoder-only model over a 32-bit residual with learned
positions and a layer norm (weight and bias) AFTER every residual sum, x <- LN(alpha x + sublayer(x)).
A layer's mixer is a gated delta rule with a decay per key channel ("channel_delta"), a state-space
recurrence with a scalar decay per head ("mamba2"), or grouped-query attention over a sliding window
plus pooled blocks of older tokens ("attention"); its feed-forward is a clamped gated MLP, a mixture of
silu-gated experts with a shared expert, or absent.  Every size, the layer order and the constants a
model may choose are read from config.json."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Union

from .model_config import register_config


@dataclass
class ChannelDeltaSpec:
    heads: int
    kv_heads: int       # query/key heads; value head h reads query/key head h // (heads / kv_heads)
    dim: int            # query/key size per head = rows of the memory
    vdim: int           # value size per head = columns of the memory
    conv: int           # taps of the short convolution on q, k and v
    decay_rank: int = 0  # inner sizes of the two low-rank projections (decay, output gate): config.json
    gate_rank: int = 0   # does not carry them, the checkpoint's tensor shapes do (resolve_shapes)


@dataclass
class StateSpaceSpec:
    heads: int
    vdim: int           # channels per head
    state: int          # rows of the memory (N)
    groups: int         # B / C groups; head h reads group h // (heads / groups)
    norm_groups: int    # equal parts of the gated output that are normed on their own
    conv: int


@dataclass
class PooledAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]       # tokens a position sees, itself included; None = all before
    pool: int                   # tokens per pooled block before the window (0 = no blocks)
    rope_base: float
    rope_dims: int              # rotated leading coordinates of a query / key head (0 = no rotation at all)


@dataclass
class ClampedMLPSpec:
    ff: int
    limit: float


@dataclass
class GroupedExpertsSpec:
    experts: int
    top: int
    ff: int
    groups: int                 # equal groups of neighbouring experts (1 = no group limit)
    keep: int                   # groups that take part in the choice
    shared_ff: int              # 0 = no shared expert


@dataclass
class KisilixLayerSpec:
    type: str                                    # "channel_delta" | "mamba2" | "attention"
    mixer: Union[ChannelDeltaSpec, StateSpaceSpec, PooledAttentionSpec]
    mlp: Union[ClampedMLPSpec, GroupedExpertsSpec, None]


@dataclass
class KisilixConfig:
    vocab: int
    width: int
    eps: float
    alpha: float                                 # multiplier of the residual inside every sum
    max_positions: int
    layers: List[KisilixLayerSpec] = field(default_factory=list)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def resolve_shapes(self, shapes) -> None:
        """Sizes that only the checkpoint knows: shapes = {tensor name: shape}."""
        for i, L in enumerate(self.layers):
            if L.type == "channel_delta":
                for attr, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    if name not in shapes:
                        raise ValueError(f"checkpoint lacks {name}")
                    setattr(L.mixer, attr, int(shapes[name][0]))
            # the taps of a convolution are its tensor's second size
            conv = {"channel_delta": f"l{i}.mix.q.conv", "mamba2": f"l{i}.mix.conv"}.get(L.type)
            if conv in shapes and len(shapes[conv]) == 2:
                L.mixer.conv = int(shapes[conv][1])


def _heads(m: dict, key: str = "kv_heads"):
    heads = int(m["heads"])
    sub = int(m.get(key, heads))
    if sub < 1 or heads % sub:
        raise ValueError(f"{heads} heads cannot share {sub} {key}")
    return heads, sub


def _mixer(kind: str, m: dict):
    if kind == "channel_delta":
        heads, kv = _heads(m)
        return ChannelDeltaSpec(heads=heads, kv_heads=kv, dim=int(m["dim"]), vdim=int(m["vdim"]),
                                conv=int(m.get("conv", 1)))
    if kind == "mamba2":
        heads, groups = _heads(m, "groups")
        parts = int(m.get("norm_groups", 1))
        if parts < 1 or (heads * int(m["vdim"])) % parts:
            raise ValueError(f"{parts} norm groups do not divide {heads * int(m['vdim'])} channels")
        return StateSpaceSpec(heads=heads, vdim=int(m["vdim"]), state=int(m["state"]), groups=groups,
                              norm_groups=parts, conv=int(m.get("conv", 1)))
    if kind == "attention":
        heads, kv = _heads(m)
        mask, rot = m.get("mask") or {}, m.get("rot") or {}
        dims = int(rot.get("dims", 0))
        if dims % 2 or dims > int(m["dim"]):
            raise ValueError(f"rotated coordinates {dims} must be even and at most the head size {m['dim']}")
        if dims and int(m["vdim"]) % 2:
            raise ValueError(f"rotated values need an even value size, not {m['vdim']}")
        window = int(mask["size"]) if mask.get("size") else None
        pool = int(mask.get("pool") or 0)
        if pool and not window:
            raise ValueError("pooled blocks need a window")
        return PooledAttentionSpec(heads=heads, kv_heads=kv, dim=int(m["dim"]), vdim=int(m["vdim"]),
                                   scale=float(m["scale"]), window=window, pool=pool,
                                   rope_base=float(rot.get("base", 10000.0)), rope_dims=dims)
    raise ValueError(f"unknown mixer type {kind!r}")


def _mlp(f: Optional[dict]):
    if not f:
        return None
    if f.get("kind") == "dense":
        return ClampedMLPSpec(ff=int(f["ff"]), limit=float(f["limit"]))
    if f.get("kind") == "moe":
        r, grp = f["router"], f["router"].get("groups") or {}
        spec = GroupedExpertsSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(f["expert"]["ff"]),
                                  groups=int(grp.get("count", 1)), keep=int(grp.get("keep", grp.get("count", 1))),
                                  shared_ff=int((f.get("shared") or {}).get("ff", 0)))
        if not 0 < spec.top <= spec.experts:
            raise ValueError(f"top {spec.top} of {spec.experts} experts")
        if spec.groups < 1 or spec.experts % spec.groups or not 0 < spec.keep <= spec.groups:
            raise ValueError(f"{spec.experts} experts in {spec.groups} groups, {spec.keep} kept")
        if spec.keep * (spec.experts // spec.groups) < spec.top:
            raise ValueError(f"{spec.keep} groups of {spec.experts // spec.groups} experts cannot give {spec.top}")
        return spec
    raise ValueError(f"unknown feed-forward kind {f.get('kind')!r}")


@register_config("Kisilix")
def kisilix_config(raw: dict) -> KisilixConfig:
    layers = []
    for i, L in enumerate(raw["layers"]):
        try:
            layers.append(KisilixLayerSpec(type=L["type"], mixer=_mixer(L["type"], L["mixer"]),
                                           mlp=_mlp(L.get("mlp"))))
        except ValueError as e:
            raise ValueError(f"layer {i}: {e}") from None
    return KisilixConfig(vocab=int(raw["vocab"]), width=int(raw["width"]), eps=float(raw["norm"]["eps"]),
                         alpha=float(raw.get("postln_alpha", 1.0)),
                         max_positions=int(raw["max_positions"]), layers=layers)
