"""Kulesun: decoder-only model over a 32-bit residual stream with an RMS norm on both sides of every
sublayer (weights stored around zero and applied as 1 + w):

    x = embed[token] * embedding_scale
    per layer:  x += norm_1b(mixer(norm_1(x)))
                x += norm_2b(ff(norm_2(x)))                  (layers with a feed-forward)
    logits = logit_scale * embed @ norm_f(x)                  (the head is the embedding table, unscaled)

A layer's mixer is grouped-query attention without rotation (query temperature, unit-RMS values mixed
with the first such layer's values, capped scores, unit sink, heads' weights mixed after the softmax,
a gate per head) or latent attention (scaled rotation in the half pairing, element-wise output gate);
the feed-forward is a silu-gated MLP.  Norms, temperature, angles, attention scores and weights and
the residual are fp32; the matrix products run in the model dtype.  Built from the shared layers
AddNormed / ResidualRMSNorm, TalkingHeadsAttention, LatentAttention with PairedRotary, GatedMLP.

Launches per layer: fused input GEMM, one prep launch that writes the token's pool row, attention,
head mix / gate, output GEMM, then ONE launch per sublayer boundary that norms the sublayer's output,
adds it to the residual and emits the next sublayer's pre-norm."""
from __future__ import annotations

import re
from typing import Iterable, Optional, Tuple

import torch
import torch.nn as nn

from ..configs.kulesun import KulesunConfig, KulesunLayerSpec
from ..layers.attention.latent_attention import LatentAttention
from ..layers.attention.talking_heads_attention import TalkingHeadsAttention
from ..layers.gated_mlp import GatedMLP
from ..layers.residual_norm import AddNormed, ResidualRMSNorm
from ..layers.rotary_embedding import PairedRotary, ramp_scaled_frequencies
from .registry import CacheSpec, register_model


def _rotary(rot) -> PairedRotary:
    freqs, amplitude = None, 1.0
    if rot.factor is not None:
        freqs, amplitude = ramp_scaled_frequencies(rot.dims, rot.base, rot.factor, rot.original, rot.fast,
                                                   rot.slow)
    return PairedRotary(rot.dims, rot.base, pairing="half", frequencies=freqs, amplitude=amplitude)


class KulesunLayer(nn.Module):
    def __init__(self, cfg: KulesunConfig, spec: KulesunLayerSpec, layer_id: int, params_dtype):
        super().__init__()
        self.layer_id, self.type, self.params_dtype = layer_id, spec.type, params_dtype
        m, W = spec.mixer, cfg.width
        if spec.type == "attention":
            first = cfg.first_v_mix_layer
            self.mix = TalkingHeadsAttention(
                W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, layer_id, cfg.eps, softcap=m.softcap,
                temp_coef=m.temp_coef, temp_every=m.temp_every, value_norm=True, unit_sink=True,
                head_gate=True, bias=True,
                v_first_layer=first if (m.v_mix and first is not None and first != layer_id) else None,
                params_dtype=params_dtype)
        else:
            self.mix = LatentAttention(W, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, None, m.scale,
                                       layer_id, cfg.eps, params_dtype=params_dtype, rotary=_rotary(m.rot),
                                       gate=True)
        self.norm1 = ResidualRMSNorm(W, cfg.eps)          # used by the first layer only: every other
        self.norm1b = AddNormed(W, cfg.eps)               # pre-norm is emitted by the launch before it
        self.mlp = GatedMLP(W, spec.mlp.ff, "silu", params_dtype) if spec.mlp is not None else None
        self.norm2 = ResidualRMSNorm(W, cfg.eps) if spec.mlp is not None else None
        self.norm2b = AddNormed(W, cfg.eps) if spec.mlp is not None else None

    def forward(self, x: torch.Tensor, h: torch.Tensor, fb, next_weight: Optional[torch.Tensor]):
        """x: the fp32 residual [T, width], updated in place; h = norm_1(x) in the model dtype.
        -> the next layer's norm_1(x) (None after the last layer)."""
        dt = self.params_dtype
        y = self.mix(h, fb)
        if self.mlp is None:
            return self.norm1b(x, a=y, out_dtype=dt if next_weight is not None else None,
                               next_weight=next_weight)
        h2 = self.norm1b(x, a=y, out_dtype=dt, next_weight=self.norm2.weight)
        return self.norm2b(x, a=self.mlp(h2), out_dtype=dt if next_weight is not None else None,
                           next_weight=next_weight)


@register_model("Kulesun")
class KulesunForCausalLM(nn.Module):
    def __init__(self, config: KulesunConfig, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.config, self.params_dtype = config, params_dtype
        self.embed = nn.Parameter(torch.empty(config.vocab, config.width, dtype=params_dtype),
                                  requires_grad=False)
        self.layers = nn.ModuleList(KulesunLayer(config, s, i, params_dtype)
                                    for i, s in enumerate(config.layers))
        self.final_norm = ResidualRMSNorm(config.width, config.eps)

    # ---- what the runner allocates -------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        spec = CacheSpec(kind="rows")
        for i, (layer, L) in enumerate(zip(self.layers, self.config.layers)):
            spec.row_dims[i] = (layer.mix.row_width if L.type == "attention"
                                else L.mixer.kv_rank + L.mixer.rot_dim)
        return spec

    # ---- forward -------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, forward_batch) -> torch.Tensor:
        x = self.embed[input_ids].float() * self.config.embedding_scale
        hook = forward_batch.extra.get("layer_hook") if forward_batch.extra else None
        if not len(self.layers):
            return x
        h = self.layers[0].norm1(x, self.params_dtype)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].norm1.weight if i + 1 < len(self.layers) else None
            h = layer(x, h, forward_batch, nxt)
            if hook is not None:
                hook(layer.layer_id, x)
        return x

    def compute_logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """-> fp32 [rows, vocab]: the product accumulates and is stored in fp32, then scaled."""
        h = self.final_norm(hidden_rows.contiguous(), self.params_dtype)
        if h.dtype == torch.float32:
            z = torch.mm(h, self.embed.t())
        else:
            z = torch.mm(h, self.embed.t(), out_dtype=torch.float32)
        return z * self.config.logit_scale

    # ---- weights -------------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> None:
        seen, pending = set(), {}
        for name, w in weights:
            seen.add(name)
            if name == "embed":
                self.embed.data.copy_(w)
            elif name == "final.norm":
                self.final_norm.weight.data.copy_(1.0 + w.float())
            else:
                m = re.match(r"^l(\d+)\.(.+)$", name)
                if not m or int(m.group(1)) >= len(self.layers):
                    raise ValueError(f"unexpected tensor {name!r}")
                self._load_layer_tensor(self.layers[int(m.group(1))], m.group(2), w, pending)
        missing = self.expected_tensor_names() - seen
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {sorted(missing)[:4]}")
        for (lid, what), parts in pending.items():      # fused projections wait for all their parts
            layer = self.layers[lid]
            if what == "mlp":
                layer.mlp.load(parts["gate"], parts["up"], parts["down"])
            else:
                layer.mix.load_direct(parts["q"], parts["dkv"], parts["g"])

    def _load_layer_tensor(self, layer: KulesunLayer, key: str, w: torch.Tensor, pending) -> None:
        lid = layer.layer_id
        bad = ValueError(f"unexpected tensor l{lid}.{key}")
        norms = {"norm1": layer.norm1, "norm1b": layer.norm1b, "norm2": layer.norm2, "norm2b": layer.norm2b}
        if key in norms:
            if norms[key] is None:
                raise bad
            norms[key].weight.data.copy_(1.0 + w.float())          # stored around zero
        elif key in ("mlp.gate", "mlp.up", "mlp.down") and layer.mlp is not None:
            pending.setdefault((lid, "mlp"), {})[key[4:]] = w
        elif key.startswith("mix.") and layer.type == "attention":
            k, att = key[4:], layer.mix
            if k in ("q", "k", "v", "g"):
                att.load_part(k, w)
            elif k in ("q.b", "k.b", "v.b"):
                att.load_part(k[0], w, is_bias=True)
            elif k == "talk":
                att.head_mix.data.copy_(w.float())
            elif k == "vmix":
                att.v_mix.data.copy_(w.float().reshape(()))
            elif k == "o":
                att.o_proj.weight_loader(att.o_proj.weight, w)
            elif k == "o.b":
                att.o_proj.bias.data.copy_(w)
            else:
                raise bad
        elif key.startswith("mix.") and layer.type == "latent_attention":
            k, att = key[4:], layer.mix
            if k in ("q", "dkv", "g"):
                pending.setdefault((lid, "mix"), {})[k] = w
            elif k == "dkv.norm":
                att.kv_norm_weight.data.copy_(w.float())
            elif k == "uk":
                att.load_uk(w)
            elif k == "uv":
                att.load_uv(w)
            elif k == "o":
                att.o_proj.weight_loader(att.o_proj.weight, w)
            else:
                raise bad
        else:
            raise bad

    def expected_tensor_names(self):
        names = {"embed", "final.norm"}
        for i, L in enumerate(self.config.layers):
            p = f"l{i}."
            names |= {p + "norm1", p + "norm1b"}
            if L.type == "attention":
                names |= {p + "mix." + k for k in ("q", "q.b", "k", "k.b", "v", "v.b", "talk", "g", "o", "o.b")}
                if self.layers[i].mix.v_first_layer is not None:
                    names.add(p + "mix.vmix")             # elsewhere the tensor, if present, is unused
            else:
                names |= {p + "mix." + k for k in ("q", "dkv", "dkv.norm", "uk", "uv", "g", "o")}
            if L.mlp is not None:
                names |= {p + "norm2", p + "norm2b"} | {p + "mlp." + k for k in ("gate", "up", "down")}
        return names
