"""Mixture-of-experts feed-forward on the kernels of csrc/moe.cu.

    TopKRouter   : z = W_r h + b in fp32; the `top` largest logits; weights = softmax over the chosen
                   logits only, or (score="sigmoid") the sigmoid of each chosen logit, not
                   renormalised.  Optionally the scalar gate sigmoid(w_sg . h) of a shared expert.
    GroupedSoftmaxRouter : z = W_r h in fp32; scores s = softmax(z) over ALL experts; the choice is made
                   on s + correction, among the experts of the `keep` groups (of `groups` equal groups
                   of neighbours) whose best choice score is largest; weights = the chosen experts' s,
                   divided by their sum (+ 1e-20).
    FusedExperts : all experts' gated feed-forwards W_down (act(W_gate h) * (W_up h)) as two grouped
                   GEMMs over the (token, choice) rows sorted by expert; nothing is read back to the
                   host, so the step stays capturable.  Returns one row per (token, choice); the
                   weighted sum is taken in fp32 together with the residual add
                   (layers/scalar_norm.py residual_combine).
    ScaledInputExperts : experts without a gate, W_down act(W_up (s h)), whose router weight s
                   multiplies the expert's INPUT.  Same sort and grouped GEMMs; s is applied to the
                   fp32 accumulator of the up-projection (W (s h) = s (W h)) before the activation.
                   Returns one row per (token, choice), already weighted: the caller only sums them.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from ... import _lib
from ..activation import GatedActAndMul


class TopKRouter(nn.Module):
    SCORES = {"softmax_chosen": 0, "sigmoid": 1}

    def __init__(self, width: int, experts: int, top: int, bias: bool = True, shared_gate: bool = False,
                 score: str = "softmax_chosen"):
        super().__init__()
        if score not in self.SCORES:
            raise ValueError(f"unknown router score {score!r}")
        self.experts, self.top, self.score = experts, top, self.SCORES[score]
        self.weight = nn.Parameter(torch.zeros(experts, width, dtype=torch.float32), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(experts, dtype=torch.float32), requires_grad=False) if bias else None
        self.shared_gate = (nn.Parameter(torch.zeros(width, dtype=torch.float32), requires_grad=False)
                            if shared_gate else None)

    def forward(self, h: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
        """-> (ids int32 [T, top], weights fp32 [T, top], gate fp32 [T] or None)."""
        if not h.is_cuda:
            raise _lib.B200Error("TopKRouter: tensor must live on a CUDA device (no CPU path)")
        t, w = h.shape
        ids = torch.empty((t, self.top), dtype=torch.int32, device=h.device)
        wts = torch.empty((t, self.top), dtype=torch.float32, device=h.device)
        gate = torch.empty((t,), dtype=torch.float32, device=h.device) if self.shared_gate is not None else None
        rc = _lib.load().b200_moe_route_scored(
            h.data_ptr(), h.stride(0), self.weight.data_ptr(), _lib.ptr(self.bias), self.experts, w,
            self.top, _lib.ptr(self.shared_gate), ids.data_ptr(), wts.data_ptr(), _lib.ptr(gate), t,
            self.score, _lib.dtype_code(h.dtype), _lib.current_stream())
        _lib.check(rc, "b200_moe_route")
        return ids, wts, gate


class GroupedSoftmaxRouter(nn.Module):
    def __init__(self, width: int, experts: int, top: int, groups: int = 1, keep: int = 1,
                 correction: bool = True):
        super().__init__()
        if experts % groups or not 0 < keep <= groups or keep * (experts // groups) < top:
            raise ValueError(f"{experts} experts in {groups} groups, {keep} kept, top {top}")
        self.experts, self.top, self.groups, self.keep = experts, top, groups, keep
        self.weight = nn.Parameter(torch.zeros(experts, width, dtype=torch.float32), requires_grad=False)
        self.correction = (nn.Parameter(torch.zeros(experts, dtype=torch.float32), requires_grad=False)
                           if correction else None)

    def forward(self, h: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """h [T, width] (fp32 or the model dtype) -> (ids int32 [T, top], weights fp32 [T, top])."""
        if not h.is_cuda:
            raise _lib.B200Error("GroupedSoftmaxRouter: tensor must live on a CUDA device (no CPU path)")
        t, w = h.shape
        ids = torch.empty((t, self.top), dtype=torch.int32, device=h.device)
        wts = torch.empty((t, self.top), dtype=torch.float32, device=h.device)
        rc = _lib.load().b200_moe_route_grouped(
            h.data_ptr(), h.stride(0), self.weight.data_ptr(), _lib.ptr(self.correction), self.experts, w,
            self.top, self.groups, self.keep, ids.data_ptr(), wts.data_ptr(), t, _lib.dtype_code(h.dtype),
            _lib.current_stream())
        _lib.check(rc, "b200_moe_route_grouped")
        return ids, wts


class FusedExperts(nn.Module):
    def __init__(self, width: int, ff: int, experts: int, act: str = "silu",
                 params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.width, self.ff, self.experts = width, ff, experts
        self.act_kind = GatedActAndMul.KINDS[act]
        self.w_gate_up = nn.Parameter(torch.empty(experts, 2 * ff, width, dtype=params_dtype), requires_grad=False)
        self.w_down = nn.Parameter(torch.empty(experts, width, ff, dtype=params_dtype), requires_grad=False)

    def load_expert(self, e: int, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> None:
        self.w_gate_up.data[e, :self.ff].copy_(gate)
        self.w_gate_up.data[e, self.ff:].copy_(up)
        self.w_down.data[e].copy_(down)

    def forward(self, h: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """h [T, width], ids [T, top] -> expert outputs [T * top, width] (row t * top + k)."""
        t, top = ids.shape
        n = t * top
        lib, st, code = _lib.load(), _lib.current_stream(), _lib.dtype_code(h.dtype)
        dev = h.device
        offsets = torch.empty(self.experts + 1, dtype=torch.int32, device=dev)
        sorted_rows = torch.empty(n, dtype=torch.int32, device=dev)
        rc = lib.b200_moe_align(ids.data_ptr(), n, self.experts, offsets.data_ptr(),
                                sorted_rows.data_ptr(), st)
        _lib.check(rc, "b200_moe_align")
        inter = torch.empty((n, self.ff), dtype=h.dtype, device=dev)
        rc = lib.b200_moe_grouped_gemm(
            h.data_ptr(), h.stride(0), self.w_gate_up.data_ptr(), self.w_gate_up.stride(1),
            self.w_gate_up.stride(0), offsets.data_ptr(), sorted_rows.data_ptr(), self.experts, top, n,
            self.ff, self.width, inter.data_ptr(), inter.stride(0), 1, self.act_kind, code, st)
        _lib.check(rc, "b200_moe_grouped_gemm")
        out = torch.empty((n, self.width), dtype=h.dtype, device=dev)
        rc = lib.b200_moe_grouped_gemm(
            inter.data_ptr(), inter.stride(0), self.w_down.data_ptr(), self.w_down.stride(1),
            self.w_down.stride(0), offsets.data_ptr(), sorted_rows.data_ptr(), self.experts, top, n,
            self.width, self.ff, out.data_ptr(), out.stride(0), 0, self.act_kind, code, st)
        _lib.check(rc, "b200_moe_grouped_gemm")
        return out


class ScaledInputExperts(nn.Module):
    ACTS = {"silu": 0, "gelu_tanh": 1, "relu2": 2}

    def __init__(self, width: int, ff: int, experts: int, act: str = "relu2",
                 params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if act not in self.ACTS:
            raise ValueError(f"unknown activation {act!r}")
        self.width, self.ff, self.experts, self.act_kind = width, ff, experts, self.ACTS[act]
        self.w_up = nn.Parameter(torch.empty(experts, ff, width, dtype=params_dtype), requires_grad=False)
        self.w_down = nn.Parameter(torch.empty(experts, width, ff, dtype=params_dtype), requires_grad=False)

    def forward(self, h: torch.Tensor, ids: torch.Tensor, weights: Optional[torch.Tensor]) -> torch.Tensor:
        """h [T, width], ids int32 [T, top], weights fp32 [T, top] (None: unweighted) ->
        [T * top, width], row t * top + k = expert ids[t, k] applied to weights[t, k] * h[t]."""
        t, top = ids.shape
        n = t * top
        lib, st, code = _lib.load(), _lib.current_stream(), _lib.dtype_code(h.dtype)
        dev = h.device
        offsets = torch.empty(self.experts + 1, dtype=torch.int32, device=dev)
        sorted_rows = torch.empty(n, dtype=torch.int32, device=dev)
        rc = lib.b200_moe_align(ids.data_ptr(), n, self.experts, offsets.data_ptr(),
                                sorted_rows.data_ptr(), st)
        _lib.check(rc, "b200_moe_align")
        inter = torch.empty((n, self.ff), dtype=h.dtype, device=dev)
        rc = lib.b200_moe_grouped_gemm_mode(
            h.data_ptr(), h.stride(0), self.w_up.data_ptr(), self.w_up.stride(1), self.w_up.stride(0),
            offsets.data_ptr(), sorted_rows.data_ptr(), self.experts, top, n, self.ff, self.width,
            inter.data_ptr(), inter.stride(0), 2, self.act_kind, _lib.ptr(weights), code, st)
        _lib.check(rc, "b200_moe_grouped_gemm_mode")
        out = torch.empty((n, self.width), dtype=h.dtype, device=dev)
        rc = lib.b200_moe_grouped_gemm_mode(
            inter.data_ptr(), inter.stride(0), self.w_down.data_ptr(), self.w_down.stride(1),
            self.w_down.stride(0), offsets.data_ptr(), sorted_rows.data_ptr(), self.experts, top, n,
            self.width, self.ff, out.data_ptr(), out.stride(0), 0, self.act_kind, None, code, st)
        _lib.check(rc, "b200_moe_grouped_gemm_mode")
        return out
