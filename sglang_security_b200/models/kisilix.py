"""Kisilix: decoder-only model over a 32-bit residual stream with learned positions and a layer norm
(weight and bias) AFTER every residual sum; the sublayers read the residual itself:

    x = embed[token] + pos[position]
    per layer:  x <- LN_1(alpha x + mixer(x))
                x <- LN_2(alpha x + ff(x))                 (layers with a feed-forward)
    logits = head(LN_f(x))

A layer's mixer is a gated delta rule with a decay per key channel behind short convolutions
("channel_delta"), a state-space recurrence with a scalar decay per head ("mamba2"), or grouped-query
attention over a sliding window plus pooled blocks, with rotated values and a multiplier per head
("attention").  The feed-forward is a clamped gated MLP or a mixture of silu-gated experts (softmax
scores, a correction that only steers the choice, groups of experts) plus a shared expert.  Norms,
recurrent state, decays and step sizes, attention scores, routers and the residual are fp32; the matrix
products run in the model dtype.  Built from the shared layers PostSumLayerNorm, ChannelDeltaMixer /
StateSpaceMixer, PooledWindowAttention, GatedMLP, GroupedSoftmaxRouter / FusedExperts."""
from __future__ import annotations

import re
from typing import Iterable, Tuple

import torch
import torch.nn as nn

from ..configs.kisilix import (ClampedMLPSpec, GroupedExpertsSpec, KisilixConfig, KisilixLayerSpec)
from ..layers.attention.pooled_window_attention import PooledWindowAttention
from ..layers.gated_mlp import GatedMLP
from ..layers.linear import ColumnParallelLinear
from ..layers.moe.fused_moe import FusedExperts, GroupedSoftmaxRouter
from ..layers.recurrent.delta_recurrence import ChannelDeltaMixer, StateSpaceMixer
from ..layers.residual_norm import PostSumLayerNorm
from .registry import CacheSpec, register_model


class KisilixExperts(nn.Module):
    def __init__(self, width: int, spec: GroupedExpertsSpec, params_dtype):
        super().__init__()
        self.router = GroupedSoftmaxRouter(width, spec.experts, spec.top, spec.groups, spec.keep, correction=True)
        self.experts = FusedExperts(width, spec.ff, spec.experts, "silu", params_dtype)
        self.shared = GatedMLP(width, spec.shared_ff, "silu", params_dtype) if spec.shared_ff else None


class KisilixLayer(nn.Module):
    def __init__(self, cfg: KisilixConfig, spec: KisilixLayerSpec, layer_id: int, params_dtype):
        super().__init__()
        self.layer_id, self.type, self.params_dtype = layer_id, spec.type, params_dtype
        m, W = spec.mixer, cfg.width
        if spec.type == "channel_delta":
            self.mix = ChannelDeltaMixer(W, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, m.decay_rank, m.gate_rank,
                                         layer_id, cfg.eps, params_dtype)
        elif spec.type == "mamba2":
            self.mix = StateSpaceMixer(W, m.heads, m.vdim, m.state, m.groups, m.norm_groups, m.conv, layer_id,
                                       cfg.eps, params_dtype)
        else:
            self.mix = PooledWindowAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, layer_id, cfg.eps,
                                             window=m.window, pool=m.pool, rope_base=m.rope_base,
                                             rope_dims=m.rope_dims, pairing="half", rotate_values=True,
                                             params_dtype=params_dtype)
        self.norm1 = PostSumLayerNorm(W, cfg.eps, cfg.alpha)
        self.dense = self.moe = self.norm2 = None
        if isinstance(spec.mlp, ClampedMLPSpec):
            self.dense = GatedMLP(W, spec.mlp.ff, "clamped", params_dtype, limit=spec.mlp.limit)
        elif isinstance(spec.mlp, GroupedExpertsSpec):
            self.moe = KisilixExperts(W, spec.mlp, params_dtype)
        if spec.mlp is not None:
            self.norm2 = PostSumLayerNorm(W, cfg.eps, cfg.alpha)

    def forward(self, x: torch.Tensor, h: torch.Tensor, fb) -> torch.Tensor:
        """x: the fp32 residual [T, width], replaced in place; h: x in the model dtype.  -> the new h."""
        h = self.norm1(x, a=self.mix(h, fb), out_dtype=self.params_dtype)
        if self.dense is not None:
            h = self.norm2(x, a=self.dense(h), out_dtype=self.params_dtype)
        elif self.moe is not None:
            ids, wts = self.moe.router(x)                    # logits from the fp32 residual
            rows = self.moe.experts(h, ids)
            shared = self.moe.shared(h) if self.moe.shared is not None else None
            h = self.norm2(x, b=shared, rows=rows, row_weights=wts, out_dtype=self.params_dtype)
        return h


@register_model("Kisilix")
class KisilixForCausalLM(nn.Module):
    def __init__(self, config: KisilixConfig, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.config, self.params_dtype = config, params_dtype
        self.max_positions = config.max_positions
        self.embed = nn.Parameter(torch.empty(config.vocab, config.width, dtype=params_dtype), requires_grad=False)
        self.pos = nn.Parameter(torch.empty(config.max_positions, config.width, dtype=params_dtype),
                                requires_grad=False)
        self.layers = nn.ModuleList(KisilixLayer(config, s, i, params_dtype) for i, s in enumerate(config.layers))
        self.final_norm = PostSumLayerNorm(config.width, config.eps)
        self.head = ColumnParallelLinear(config.width, config.vocab, bias=False, params_dtype=params_dtype,
                                         tp_rank=0, tp_size=1)

    # ---- what the runner allocates -------------------------------------------------------------
    def cache_spec(self) -> CacheSpec:
        spec = CacheSpec(kind="rows")
        for i, layer in enumerate(self.layers):
            if isinstance(layer.mix, PooledWindowAttention):
                spec.row_dims[i] = layer.mix.row_width
                if layer.mix.pool:
                    spec.block_summaries[i] = layer.mix.pool
            else:
                spec.state_widths[i] = layer.mix.state_width()
        return spec

    # ---- forward -------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, forward_batch) -> torch.Tensor:
        x = self.embed[input_ids].float() + self.pos[forward_batch.positions].float()
        h = x if self.params_dtype == torch.float32 else x.to(self.params_dtype)
        hook = forward_batch.extra.get("layer_hook") if forward_batch.extra else None
        for layer in self.layers:
            h = layer(x, h, forward_batch)
            if hook is not None:
                hook(layer.layer_id, x)
        return x

    def compute_logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """-> fp32 [rows, vocab]: the product accumulates and is stored in fp32."""
        h = self.final_norm(hidden_rows.contiguous(), out_dtype=self.params_dtype, in_place=False)
        if h.dtype == torch.float32:
            return torch.mm(h, self.head.weight.t())
        return torch.mm(h, self.head.weight.t(), out_dtype=torch.float32)

    # ---- weights -------------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> None:
        seen = set()
        top = {"embed": lambda w: self.embed.data.copy_(w), "pos": lambda w: self.pos.data.copy_(w),
               "head": lambda w: self.head.weight_loader(self.head.weight, w),
               "final.norm": lambda w: self.final_norm.weight.data.copy_(w.float()),
               "final.norm.b": lambda w: self.final_norm.bias.data.copy_(w.float())}
        for name, w in weights:
            seen.add(name)
            if name in top:
                top[name](w)
                continue
            m = re.match(r"^l(\d+)\.(.+)$", name)
            if not m or int(m.group(1)) >= len(self.layers):
                raise ValueError(f"unexpected tensor {name!r}")
            self._load_layer_tensor(self.layers[int(m.group(1))], m.group(2), w)
        missing = self.expected_tensor_names() - seen
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {sorted(missing)[:4]}")

    def _load_layer_tensor(self, layer: KisilixLayer, key: str, w: torch.Tensor) -> None:
        bad = ValueError(f"unexpected tensor l{layer.layer_id}.{key}")
        norms = {"norm1": layer.norm1, "norm2": layer.norm2}
        if key in norms or (key.endswith(".b") and key[:-2] in norms):
            norm = norms[key[:5]]
            if norm is None:
                raise bad
            (norm.bias if key.endswith(".b") else norm.weight).data.copy_(w.float())
        elif key.startswith("mlp."):
            self._load_mlp_tensor(layer, key[4:], w, bad)
        elif key.startswith("mix."):
            k, mix = key[4:], layer.mix
            if k == "o":
                mix.o_proj.weight_loader(mix.o_proj.weight, w)
            elif layer.type == "channel_delta":
                if k in ("q", "k", "v", "b", "a1", "g1"):
                    mix.load_part(k, w)
                elif k in ("q.conv", "k.conv", "v.conv"):
                    mix.load_conv(k[0], w)
                elif k == "a2":
                    mix.decay_up.weight_loader(mix.decay_up.weight, w)
                elif k == "g2":
                    mix.gate_up.weight_loader(mix.gate_up.weight, w)
                elif k == "A_log":
                    mix.a_log.data.copy_(w.float())
                elif k == "dt_bias":
                    mix.dt_bias.data.copy_(w.float())
                elif k == "norm":
                    mix.norm_weight.data.copy_(w.float().repeat(mix.heads))
                else:
                    raise bad
            elif layer.type == "mamba2":
                dst = {"conv": mix.conv_weight, "conv.b": mix.conv_bias, "dt_bias": mix.dt_bias, "A_log": mix.a_log,
                       "D": mix.skip, "norm": mix.norm_weight}
                if k == "in":
                    mix.in_proj.weight_loader(mix.in_proj.weight, w)
                elif k in dst:
                    dst[k].data.copy_(w.float())
                else:
                    raise bad
            else:
                dst = {"q.norm": mix.q_norm_weight, "k.norm": mix.k_norm_weight, "temp": mix.head_scale}
                if k in ("q", "k", "v"):
                    mix.load_part(k, w)
                elif k in ("q.b", "k.b", "v.b"):
                    mix.load_part(k[0], w, is_bias=True)
                elif k in dst:
                    dst[k].data.copy_(w.float())
                else:
                    raise bad
        else:
            raise bad

    def _load_mlp_tensor(self, layer: KisilixLayer, k: str, w: torch.Tensor, bad: Exception) -> None:
        if layer.dense is not None:
            if k not in ("gate", "up", "down"):
                raise bad
            mlp = layer.dense
        elif layer.moe is not None and k.startswith("shared.") and layer.moe.shared is not None:
            mlp, k = layer.moe.shared, k[7:]
        elif layer.moe is not None:
            m = re.match(r"^e(\d+)\.(gate|up|down)$", k)
            ex = layer.moe.experts
            if k == "router":
                layer.moe.router.weight.data.copy_(w.float())
            elif k == "correction":
                layer.moe.router.correction.data.copy_(w.float())
            elif m and int(m.group(1)) < ex.experts:
                e, ff = int(m.group(1)), ex.ff
                if m.group(2) == "down":
                    ex.w_down.data[e].copy_(w)
                else:
                    lo = 0 if m.group(2) == "gate" else ff
                    ex.w_gate_up.data[e, lo:lo + ff].copy_(w)
            else:
                raise bad
            return
        else:
            raise bad
        if k == "gate":
            mlp.gate_up_proj.weight_loader(mlp.gate_up_proj.weight, w, 0)
        elif k == "up":
            mlp.gate_up_proj.weight_loader(mlp.gate_up_proj.weight, w, 1)
        elif k == "down":
            mlp.down_proj.weight_loader(mlp.down_proj.weight, w)
        else:
            raise bad

    def expected_tensor_names(self):
        names = {"embed", "pos", "head", "final.norm", "final.norm.b"}
        for i, L in enumerate(self.config.layers):
            p = f"l{i}."
            names |= {p + "norm1", p + "norm1.b"}
            if L.type == "channel_delta":
                keys = ("q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "A_log", "norm", "a1", "a2", "dt_bias",
                        "g1", "g2", "o")
            elif L.type == "mamba2":
                keys = ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")
            else:
                keys = ("q", "q.b", "k", "k.b", "v", "v.b", "q.norm", "k.norm", "temp", "o")
            names |= {p + "mix." + k for k in keys}
            if L.mlp is not None:
                names |= {p + "norm2", p + "norm2.b"}
            if isinstance(L.mlp, ClampedMLPSpec):
                names |= {p + "mlp." + k for k in ("gate", "up", "down")}
            elif isinstance(L.mlp, GroupedExpertsSpec):
                names |= {p + "mlp.router", p + "mlp.correction"}
                for e in range(L.mlp.experts):
                    names |= {p + f"mlp.e{e}." + k for k in ("gate", "up", "down")}
                if L.mlp.shared_ff:
                    names |= {p + "mlp.shared." + k for k in ("gate", "up", "down")}
        return names
