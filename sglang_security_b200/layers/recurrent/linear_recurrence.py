"""Mixers whose memory is a matrix per head, carried from token to token in fp32
(csrc/linear_recurrence.cu):

    S_t = a_t S_(t-1) + b_t k_t v_t^T ,   o_t = S_t^T q_t  (/ den_t)

`linear_recurrence` is the kernel call; it walks every batch entry's new tokens in order from the
entry's row of a SeqStatePool (zero at position 0) and leaves the new state there, so prompt
portions and single decoded tokens are the same code and a position's output does not depend on how
the sequence was cut.  Two mixers are built on it:

    MLSTMMixer              exponential input / forget gates in log space with a running stabiliser and
                            a normaliser vector (xLSTM's matrix memory); per-head RMS of the output,
                            a weight over all heads, an output gate sigmoid(W_g h), W_o
    DecayedLinearAttention  constant decay per head, silu on q, k and v, RMS norm over all heads
                            together with a weight, an output gate, W_o
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import _lib
from ..linear import ColumnParallelLinear, RowParallelLinear


def state_width(heads: int, dim: int, vdim: int, gated: bool) -> int:
    """fp32 values one sequence keeps for one such layer."""
    n = int(_lib.load().b200_linear_recurrence_state_width(heads, dim, vdim, 1 if gated else 0))
    if n < 0:
        raise _lib.B200Error(f"linear_recurrence: heads {heads}, key size {dim}, value size {vdim} unsupported")
    return n


def linear_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, dim: int, vdim: int,
                      state: torch.Tensor, fb, gates: Optional[torch.Tensor] = None,
                      decay: Optional[torch.Tensor] = None, cap: float = 0.0, q_scale: float = 1.0,
                      silu: bool = False):
    """q, k [T, heads * dim], v [T, heads * vdim] (row-strided views are fine) -> fp32 [T, heads * vdim].
    `decay` fp32 [heads] selects the constant form.  `gates` fp32 [T, 2 * heads] (input then forget
    pre-activations) selects the gated form, which returns (o, aux): o un-normalised and aux fp32
    [T, 2 * heads] = (n . q, m) per head, for the division by max(|n . q|, exp(-m)) + den_eps that
    `gated_group_rmsnorm` performs.  `fb` carries tok_pos / ext_start / ext_len / req_pool_indices."""
    if not q.is_cuda:
        raise _lib.B200Error("linear_recurrence: tensors must live on a CUDA device (no CPU path)")
    for t in (q, k, v):
        if t.stride(-1) != 1 or t.dtype != q.dtype:
            raise _lib.B200Error("linear_recurrence: q, k, v need contiguous rows of one dtype")
    T = q.shape[0]
    out = torch.empty((T, heads * vdim), dtype=torch.float32, device=q.device)
    aux = torch.empty((T, 2 * heads), dtype=torch.float32, device=q.device) if gates is not None else None
    if gates is not None and (gates.dtype != torch.float32 or gates.stride(-1) != 1):
        raise _lib.B200Error("linear_recurrence: gate pre-activations must be fp32 rows")
    rc = _lib.load().b200_linear_recurrence(
        q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
        _lib.ptr(gates), gates.stride(0) if gates is not None else 0, _lib.ptr(decay), float(cap),
        float(q_scale), 1 if silu else 0, state.data_ptr(), state.stride(0),
        fb.req_pool_indices.data_ptr(), fb.tok_pos.data_ptr(), fb.ext_start.data_ptr(),
        fb.ext_len.data_ptr(), out.data_ptr(), out.stride(0), _lib.ptr(aux), 2 * heads,
        int(fb.batch_size), heads, dim, vdim, _lib.dtype_code(q.dtype), _lib.current_stream())
    _lib.check(rc, "b200_linear_recurrence")
    return out if aux is None else (out, aux)


def gated_group_rmsnorm(o: torch.Tensor, weight: Optional[torch.Tensor], z: Optional[torch.Tensor],
                        group: int, eps: float, out_dtype: torch.dtype, aux: Optional[torch.Tensor] = None,
                        heads: int = 0, den_eps: float = 1e-6, gate: str = "sigmoid") -> torch.Tensor:
    """o fp32 [T, N] -> o / rms over groups of `group` coordinates * weight * sigmoid(z), in out_dtype.
    gate="silu_before": o is multiplied by silu(z) BEFORE the norm instead (the norm sees the gated values).
    With `aux` (the gated recurrence's (n . q, m), fp32 [T, 2 * heads]) each head of o is first divided
    by max(|n . q|, exp(-m)) + den_eps."""
    T, N = o.shape
    if z is not None and (z.dtype != out_dtype or z.stride(-1) != 1):
        raise _lib.B200Error("gated_group_rmsnorm: the gate must have the output dtype and contiguous rows")
    out = torch.empty((T, N), dtype=out_dtype, device=o.device)
    if gate not in ("sigmoid", "silu_before"):
        raise ValueError(f"unknown gate form {gate!r}")
    rc = _lib.load().b200_gated_group_rmsnorm_mode(
        o.data_ptr(), o.stride(0), _lib.ptr(weight), _lib.ptr(z), z.stride(0) if z is not None else 0,
        out.data_ptr(), out.stride(0), T, N, int(group), float(eps), _lib.ptr(aux),
        aux.stride(0) if aux is not None else 0, int(heads), float(den_eps),
        1 if gate == "silu_before" else 0, _lib.dtype_code(out_dtype), _lib.current_stream())
    _lib.check(rc, "b200_gated_group_rmsnorm")
    return out


class _MatrixMemoryMixer(nn.Module):
    """Shared plumbing: one fused projection [q ; k ; v ; g], the output norm weight and W_o."""

    gated = False

    def __init__(self, width: int, heads: int, dim: int, vdim: int, layer_id: int, eps: float,
                 params_dtype: torch.dtype):
        super().__init__()
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.layer_id, self.eps, self.params_dtype = layer_id, float(eps), params_dtype
        kw = dict(bias=False, params_dtype=params_dtype, tp_rank=0, tp_size=1)
        self.sizes = [heads * dim, heads * dim, heads * vdim, heads * vdim]
        self.qkvg_proj = ColumnParallelLinear(width, sum(self.sizes), **kw)
        self.o_proj = RowParallelLinear(heads * vdim, width, **kw)
        self.norm_weight = nn.Parameter(torch.ones(heads * vdim, dtype=torch.float32), requires_grad=False)

    def state_width(self) -> int:
        return state_width(self.heads, self.dim, self.vdim, self.gated)

    def load_part(self, which: str, w: torch.Tensor) -> None:
        i = "qkvg".index(which)
        lo = sum(self.sizes[:i])
        self.qkvg_proj.weight.data[lo:lo + self.sizes[i]].copy_(w)

    def _split(self, h: torch.Tensor):
        y, _ = self.qkvg_proj(h)
        a = self.sizes
        return (y[:, :a[0]], y[:, a[0]:a[0] + a[1]], y[:, a[0] + a[1]:a[0] + a[1] + a[2]],
                y[:, a[0] + a[1] + a[2]:])


class MLSTMMixer(_MatrixMemoryMixer):
    gated = True

    def __init__(self, width: int, heads: int, dim: int, vdim: int, gate_cap: float, layer_id: int,
                 eps: float, params_dtype: torch.dtype = torch.bfloat16, den_eps: float = 1e-6):
        super().__init__(width, heads, dim, vdim, layer_id, eps, params_dtype)
        self.gate_cap, self.den_eps = float(gate_cap), float(den_eps)
        # input and forget gates enter the recurrence: fp32 weights applied to the fp32 residual
        self.gate_weight = nn.Parameter(torch.zeros(2 * heads, width, dtype=torch.float32), requires_grad=False)
        self.gate_bias = nn.Parameter(torch.zeros(2 * heads, dtype=torch.float32), requires_grad=False)

    def forward(self, h: torch.Tensor, x32: torch.Tensor, fb) -> torch.Tensor:
        q, k, v, g = self._split(h)
        gates = F.linear(x32, self.gate_weight, self.gate_bias)
        o, aux = linear_recurrence(q, k, v, self.heads, self.dim, self.vdim, fb.state_pool.get(self.layer_id),
                                   fb, gates=gates, cap=self.gate_cap, q_scale=self.dim ** -0.5)
        y = gated_group_rmsnorm(o, self.norm_weight, g, self.vdim, self.eps, self.params_dtype, aux=aux,
                                heads=self.heads, den_eps=self.den_eps)
        out, _ = self.o_proj(y)
        return out


class DecayedLinearAttention(_MatrixMemoryMixer):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, decay: Sequence[float], layer_id: int,
                 eps: float, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__(width, heads, dim, vdim, layer_id, eps, params_dtype)
        if len(decay) != heads:
            raise ValueError("one decay constant per head")
        self.register_buffer("decay", torch.tensor([float(d) for d in decay], dtype=torch.float64)
                             .to(torch.float32), persistent=False)

    def forward(self, h: torch.Tensor, x32: torch.Tensor, fb) -> torch.Tensor:
        q, k, v, g = self._split(h)
        o = linear_recurrence(q, k, v, self.heads, self.dim, self.vdim, fb.state_pool.get(self.layer_id), fb,
                              decay=self.decay, silu=True)
        y = gated_group_rmsnorm(o, self.norm_weight, g, self.heads * self.vdim, self.eps, self.params_dtype)
        out, _ = self.o_proj(y)
        return out
