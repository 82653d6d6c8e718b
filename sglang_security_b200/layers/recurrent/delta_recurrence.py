"""Mixers whose matrix memory decays by an amount computed from the token, fed through a short causal
convolution (csrc/delta_recurrence.cu):

    ChannelDeltaMixer   gated delta rule with one decay per head and KEY CHANNEL:
                          q, k, v = silu(conv(W h));  q, k unit vectors per head, q / sqrt(dim)
                          g = exp(-exp(A_h) softplus(W_a2 W_a1 h + dt_bias))      [heads, dim]
                          S <- diag(g) S;  u = sigmoid(w_b . h) (v - S^T k);  S += k u^T;  o = S^T q
                          o / rms(o) * weight * sigmoid(W_g2 W_g1 h), W_o
    StateSpaceMixer     state-space recurrence with a scalar decay per head:
                          [z | x | B | C | dt] = W_in h;  x, B, C = silu(conv(.) + bias)
                          dt = softplus(dt + dt_bias);  S <- exp(-exp(A_h) dt) S + B (dt x)^T
                          y = S^T C + D_h x;  (y silu(z)) normed in equal parts * weight, W_o

Both keep, per sequence and layer, one fp32 row of a SeqStatePool: the convolution's last taps-1
inputs followed by the memory of every head.  Prompt portions and single decoded tokens are the same
kernels; a portion that starts at position 0 ignores what the row holds."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import _lib
from ..linear import ColumnParallelLinear, RowParallelLinear
from .linear_recurrence import gated_group_rmsnorm


def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                     fb) -> torch.Tensor:
    """x [T, C] (a row-strided view is fine), weight fp32 [C, taps] (last column = the current token),
    state fp32 [slots, >= (taps-1) * C] (a column slice of the layer's state rows) -> silu(conv) [T, C]
    in x.dtype; the state rows of the step's sequences are advanced."""
    if not x.is_cuda:
        raise _lib.B200Error("causal_conv_silu: tensors must live on a CUDA device (no CPU path)")
    if x.stride(-1) != 1 or weight.dtype != torch.float32 or not weight.is_contiguous():
        raise _lib.B200Error("causal_conv_silu: contiguous input rows and fp32 taps [C, taps] are expected")
    T, C = x.shape
    taps = weight.shape[1]
    out = torch.empty((T, C), dtype=x.dtype, device=x.device)
    rc = _lib.load().b200_causal_conv_silu(
        x.data_ptr(), x.stride(0), weight.data_ptr(), _lib.ptr(bias), state.data_ptr(), state.stride(0),
        fb.req_pool_indices.data_ptr(), fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), fb.ext_start.data_ptr(),
        fb.ext_len.data_ptr(), out.data_ptr(), out.stride(0), T, int(fb.batch_size), C, taps,
        _lib.dtype_code(x.dtype), _lib.current_stream())
    _lib.check(rc, "b200_causal_conv_silu")
    return out


def delta_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay_raw: torch.Tensor,
                     decay_bias: torch.Tensor, a_log: torch.Tensor, heads: int, groups: int, dim: int,
                     vdim: int, state: torch.Tensor, fb, beta_raw: Optional[torch.Tensor] = None,
                     skip: Optional[torch.Tensor] = None, q_scale: float = 1.0, unit_eps: float = 1e-6
                     ) -> torch.Tensor:
    """q, k [T, groups * dim], v [T, heads * vdim], row-strided views of one dtype -> fp32 [T, heads * vdim].
    With `beta_raw` [T, heads] the delta rule with a decay per key channel (decay_raw [T, heads * dim]);
    without it the state-space form with a scalar decay and step size per head (decay_raw [T, heads]).
    decay_bias, a_log, skip are fp32.  state: fp32 [slots, >= heads * dim * vdim]."""
    if not q.is_cuda:
        raise _lib.B200Error("delta_recurrence: tensors must live on a CUDA device (no CPU path)")
    for t in (q, k, v, decay_raw) + ((beta_raw,) if beta_raw is not None else ()):
        if t.stride(-1) != 1 or t.dtype != q.dtype:
            raise _lib.B200Error("delta_recurrence: inputs need contiguous rows of one dtype")
    T = q.shape[0]
    out = torch.empty((T, heads * vdim), dtype=torch.float32, device=q.device)
    mode = 0 if beta_raw is not None else 1
    lib = _lib.load()
    work = torch.empty(T * int(lib.b200_delta_recurrence_work_width(heads, groups, dim, mode)),
                       dtype=torch.float32, device=q.device)
    rc = lib.b200_delta_recurrence(
        q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
        decay_raw.data_ptr(), decay_raw.stride(0), decay_bias.data_ptr(), a_log.data_ptr(),
        _lib.ptr(beta_raw), beta_raw.stride(0) if beta_raw is not None else 0, _lib.ptr(skip),
        float(q_scale), float(unit_eps), mode, state.data_ptr(), state.stride(0),
        fb.req_pool_indices.data_ptr(), fb.tok_pos.data_ptr(), fb.ext_start.data_ptr(), fb.ext_len.data_ptr(),
        out.data_ptr(), out.stride(0), work.data_ptr(), T, int(fb.batch_size), heads, groups, dim, vdim,
        _lib.dtype_code(q.dtype), _lib.current_stream())
    _lib.check(rc, "b200_delta_recurrence")
    return out


class _ConvRecurrentMixer(nn.Module):
    """Shared plumbing: the convolution's taps and the split of the per-sequence state row."""

    def _init_conv(self, channels: int, taps: int, bias: bool) -> None:
        self.conv_channels, self.taps = channels, int(taps)
        self.conv_weight = nn.Parameter(torch.zeros(channels, self.taps, dtype=torch.float32), requires_grad=False)
        self.conv_bias = nn.Parameter(torch.zeros(channels, dtype=torch.float32), requires_grad=False) if bias else None

    @property
    def conv_state_width(self) -> int:
        return (self.taps - 1) * self.conv_channels

    def _states(self, fb):
        row = fb.state_pool.get(self.layer_id)
        cw = self.conv_state_width
        return row[:, :max(cw, 1)], row[:, cw:]


class ChannelDeltaMixer(_ConvRecurrentMixer):
    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, decay_rank: int,
                 gate_rank: int, layer_id: int, eps: float, params_dtype: torch.dtype = torch.bfloat16,
                 unit_eps: float = 1e-6):
        super().__init__()
        if heads % kv_heads:
            raise ValueError("value heads must be a multiple of query/key heads")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.layer_id, self.eps, self.unit_eps, self.params_dtype = layer_id, float(eps), float(unit_eps), params_dtype
        kw = dict(bias=False, params_dtype=params_dtype, tp_rank=0, tp_size=1)
        # one input GEMM: [q ; k ; v ; a1 ; g1 ; b] (the low-rank halves and the write strength ride along)
        self.parts = {"q": kv_heads * dim, "k": kv_heads * dim, "v": heads * vdim, "a1": decay_rank,
                      "g1": gate_rank, "b": heads}
        self.in_proj = ColumnParallelLinear(width, sum(self.parts.values()), **kw)
        self.decay_up = ColumnParallelLinear(decay_rank, heads * dim, **kw)      # W_a2
        self.gate_up = ColumnParallelLinear(gate_rank, heads * vdim, **kw)       # W_g2
        self.o_proj = RowParallelLinear(heads * vdim, width, **kw)
        self._init_conv(2 * kv_heads * dim + heads * vdim, conv, bias=False)
        f32 = dict(dtype=torch.float32)
        self.a_log = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(heads * dim, **f32), requires_grad=False)
        # the output norm's weight [vdim] is shared by the heads: stored once per head
        self.norm_weight = nn.Parameter(torch.ones(heads * vdim, **f32), requires_grad=False)

    def state_width(self) -> int:
        n = int(_lib.load().b200_delta_recurrence_state_width(self.heads, self.dim, self.vdim))
        return self.conv_state_width + n

    def _offset(self, which: str) -> int:
        names = list(self.parts)
        return sum(self.parts[n] for n in names[:names.index(which)])

    def load_part(self, which: str, w: torch.Tensor) -> None:
        lo = self._offset(which)
        self.in_proj.weight.data[lo:lo + self.parts[which]].copy_(w)

    def load_conv(self, which: str, w: torch.Tensor) -> None:
        lo = self._offset(which)
        self.conv_weight.data[lo:lo + self.parts[which]].copy_(w.float())

    def forward(self, h: torch.Tensor, fb) -> torch.Tensor:
        y, _ = self.in_proj(h)
        p, nqkv = self.parts, self.conv_channels
        o_a1 = nqkv
        o_g1, o_b = o_a1 + p["a1"], o_a1 + p["a1"] + p["g1"]
        conv_state, mem = self._states(fb)
        c = causal_conv_silu(y[:, :nqkv], self.conv_weight, None, conv_state, fb)
        q, k, v = c[:, :p["q"]], c[:, p["q"]:p["q"] + p["k"]], c[:, p["q"] + p["k"]:]
        decay_raw, _ = self.decay_up(y[:, o_a1:o_g1])
        gate_raw, _ = self.gate_up(y[:, o_g1:o_b])
        o = delta_recurrence(q, k, v, decay_raw, self.dt_bias, self.a_log, self.heads, self.kv_heads, self.dim,
                             self.vdim, mem, fb, beta_raw=y[:, o_b:], q_scale=self.dim ** -0.5,
                             unit_eps=self.unit_eps)
        z = gated_group_rmsnorm(o, self.norm_weight, gate_raw, self.vdim, self.eps, self.params_dtype)
        out, _ = self.o_proj(z)
        return out


class StateSpaceMixer(_ConvRecurrentMixer):
    def __init__(self, width: int, heads: int, vdim: int, state: int, groups: int, norm_groups: int, conv: int,
                 layer_id: int, eps: float, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if heads % groups or (heads * vdim) % norm_groups:
            raise ValueError("heads must be a multiple of the groups, the channels of the norm groups")
        self.width, self.heads, self.vdim, self.state, self.groups = width, heads, vdim, state, groups
        self.norm_groups, self.layer_id, self.eps, self.params_dtype = norm_groups, layer_id, float(eps), params_dtype
        self.inner = heads * vdim
        kw = dict(bias=False, params_dtype=params_dtype, tp_rank=0, tp_size=1)
        # [z | x | B | C | dt] in one GEMM, the checkpoint's own layout
        self.in_proj = ColumnParallelLinear(width, 2 * self.inner + 2 * groups * state + heads, **kw)
        self.o_proj = RowParallelLinear(self.inner, width, **kw)
        self._init_conv(self.inner + 2 * groups * state, conv, bias=True)
        f32 = dict(dtype=torch.float32)
        self.a_log = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False)
        self.skip = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(self.inner, **f32), requires_grad=False)

    def state_width(self) -> int:
        n = int(_lib.load().b200_delta_recurrence_state_width(self.heads, self.state, self.vdim))
        return self.conv_state_width + n

    def forward(self, h: torch.Tensor, fb) -> torch.Tensor:
        y, _ = self.in_proj(h)
        inner, gn = self.inner, self.groups * self.state
        conv_state, mem = self._states(fb)
        c = causal_conv_silu(y[:, inner:2 * inner + 2 * gn], self.conv_weight, self.conv_bias, conv_state, fb)
        x, B, C = c[:, :inner], c[:, inner:inner + gn], c[:, inner + gn:]
        o = delta_recurrence(C, B, x, y[:, 2 * inner + 2 * gn:], self.dt_bias, self.a_log, self.heads, self.groups,
                             self.state, self.vdim, mem, fb, skip=self.skip)
        z = gated_group_rmsnorm(o, self.norm_weight, y[:, :inner], inner // self.norm_groups, self.eps,
                                self.params_dtype, gate="silu_before")
        out, _ = self.o_proj(z)
        return out
