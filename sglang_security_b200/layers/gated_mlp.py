"""Gated feed-forward W_down (act(W_gate h) * (W_up h)) with a fused [gate; up] projection, for the
designs whose activations may be fp32 as well as 16-bit (the decoder layer of the Llama family keeps
its own FP8-aware chain in model_executor/decoder_layer.py)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .activation import ClampedGluAndMul, GatedActAndMul
from .linear import MergedColumnParallelLinear, RowParallelLinear


class GatedMLP(nn.Module):
    def __init__(self, width: int, ff: int, act: str, params_dtype: torch.dtype = torch.bfloat16,
                 limit: float = 0.0):
        """act: "silu" / "gelu_tanh", or "clamped" = g sigmoid(1.702 g) (u + 1) on the gate clamped from
        above and the up-projection clamped on both sides at `limit`."""
        super().__init__()
        kw = dict(bias=False, params_dtype=params_dtype, tp_rank=0, tp_size=1)
        self.ff = ff
        self.gate_up_proj = MergedColumnParallelLinear(width, [ff, ff], **kw)
        self.down_proj = RowParallelLinear(ff, width, **kw)
        self.act_fn = ClampedGluAndMul(limit) if act == "clamped" else GatedActAndMul(act)

    def load(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> None:
        self.gate_up_proj.weight_loader(self.gate_up_proj.weight, gate, 0)
        self.gate_up_proj.weight_loader(self.gate_up_proj.weight, up, 1)
        self.down_proj.weight_loader(self.down_proj.weight, down)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        gu, _ = self.gate_up_proj(h)
        out, _ = self.down_proj(self.act_fn(gu))
        return out
