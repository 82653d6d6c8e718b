"""Norm on a sublayer's OUTPUT followed by the residual add, for designs whose sublayers read the
32-bit residual itself (csrc/norm_shift.cu add_normed):

    y = sa * a + sb * b + sum_k rows[t * top + k]        (fp32 sum of the terms given)
    x += mult * y / sqrt(mean(y^2) + eps) * weight

`AddNormed` owns the weight; one launch does the sum, the norm, the add and, on request, the copy of
the new residual in the model dtype that the next sublayer's matrix products read.  For designs with a
norm BEFORE every sublayer as well, that copy is the next sublayer's pre-norm
x / sqrt(mean(x^2) + eps) * next_weight instead (still the one launch).  `ResidualRMSNorm`
is the plain RMS norm of the fp32 residual with a per-coordinate weight (a model's final norm), its
output in the model dtype.  `PostSumLayerNorm` is for designs whose norm follows the residual SUM:
x <- LN(alpha * x + terms) with weight and bias (csrc/norm_shift.cu scaled_add_layernorm), the expert
rows weighted inside the same fp32 sum; without terms it is a plain layer norm of the residual.  `softcap` is the logit cap cap * tanh(z / cap) with a fp32 result."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _lib


class AddNormed(nn.Module):
    def __init__(self, width: int, eps: float, mult: float = 1.0):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, dtype=torch.float32), requires_grad=False)
        self.eps, self.mult = float(eps), float(mult)

    def forward(self, x: torch.Tensor, a: Optional[torch.Tensor] = None, sa: float = 1.0,
                b: Optional[torch.Tensor] = None, sb: float = 1.0, rows: Optional[torch.Tensor] = None,
                top: int = 0, out_dtype: Optional[torch.dtype] = None,
                next_weight: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """x: fp32 residual [T, W], updated in place.  -> the new x in `out_dtype` (None: not asked), or
        with `next_weight` (fp32 [W]) its RMS norm times that weight."""
        if not x.is_cuda:
            raise _lib.B200Error("AddNormed: tensor must live on a CUDA device (no CPU path)")
        if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
            raise _lib.B200Error("AddNormed: the residual must be a 2-D fp32 tensor with contiguous rows")
        terms = [v for v in (a, b, rows) if v is not None]
        if not terms:
            raise _lib.B200Error("AddNormed: nothing to add")
        dt = terms[0].dtype
        for v in terms:
            if v.dtype != dt or v.stride(-1) != 1:
                raise _lib.B200Error("AddNormed: terms must share a dtype and have contiguous rows")
        t, w = x.shape
        out = None
        if out_dtype is not None and (out_dtype != torch.float32 or next_weight is not None):
            if out_dtype != dt:
                raise _lib.B200Error("AddNormed: the copy of the residual has the terms' dtype")
            out = torch.empty((t, w), dtype=out_dtype, device=x.device)
        ld = lambda v: v.stride(0) if v is not None else 0
        rc = _lib.load().b200_add_normed_next(
            x.data_ptr(), x.stride(0), _lib.ptr(a), ld(a), float(sa), _lib.ptr(b), ld(b), float(sb),
            _lib.ptr(rows), ld(rows), int(top), self.weight.data_ptr(), self.eps, self.mult,
            _lib.ptr(out), ld(out), _lib.ptr(next_weight) if out is not None else None, t, w,
            _lib.dtype_code(dt), _lib.current_stream())
        _lib.check(rc, "b200_add_normed")
        return out if out is not None else (x if out_dtype == torch.float32 else None)


class PostSumLayerNorm(nn.Module):
    def __init__(self, width: int, eps: float, alpha: float = 1.0):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, dtype=torch.float32), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(width, dtype=torch.float32), requires_grad=False)
        self.eps, self.alpha = float(eps), float(alpha)

    def forward(self, x: torch.Tensor, a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, row_weights: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, in_place: bool = True) -> Optional[torch.Tensor]:
        """x: fp32 residual [T, W].  in_place: x <- LN(alpha x + a + b + sum_k row_weights[t, k] *
        rows[t * top + k]) and -> its copy in `out_dtype` (None: no copy; fp32: x itself).  Not in place
        (a final norm): x is only read, alpha counts as 1 and the result is returned in `out_dtype`."""
        if not x.is_cuda:
            raise _lib.B200Error("PostSumLayerNorm: tensor must live on a CUDA device (no CPU path)")
        if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
            raise _lib.B200Error("PostSumLayerNorm: the residual must be a 2-D fp32 tensor with contiguous rows")
        terms = [v for v in (a, b, rows) if v is not None]
        dt = terms[0].dtype if terms else (out_dtype or torch.float32)
        for v in terms:
            if v.dtype != dt or v.stride(-1) != 1:
                raise _lib.B200Error("PostSumLayerNorm: terms must share a dtype and have contiguous rows")
        t, w = x.shape
        top = 0
        if rows is not None:
            top = rows.shape[0] // max(t, 1)
            if rows.shape[0] != t * top or (row_weights is not None and (
                    row_weights.dtype != torch.float32 or tuple(row_weights.shape) != (t, top)
                    or not row_weights.is_contiguous())):
                raise _lib.B200Error("PostSumLayerNorm: expert rows [T * top, W] with fp32 weights [T, top]")
        out = None
        if out_dtype is not None and (out_dtype != torch.float32 or not in_place):
            out = torch.empty((t, w), dtype=out_dtype, device=x.device)
        ld = lambda v: v.stride(0) if v is not None else 0
        rc = _lib.load().b200_scaled_add_layernorm(
            x.data_ptr(), x.stride(0), self.alpha if in_place else 1.0, _lib.ptr(a), ld(a), _lib.ptr(b), ld(b),
            _lib.ptr(rows), ld(rows), _lib.ptr(row_weights), int(top), self.weight.data_ptr(),
            self.bias.data_ptr(), self.eps, _lib.ptr(out), ld(out), 1 if in_place else 0, t, w,
            _lib.dtype_code(dt), _lib.dtype_code(out.dtype if out is not None else dt), _lib.current_stream())
        _lib.check(rc, "b200_scaled_add_layernorm")
        return out if out is not None else (x if out_dtype == torch.float32 else None)


class ResidualRMSNorm(nn.Module):
    def __init__(self, width: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, dtype=torch.float32), requires_grad=False)
        self.eps = float(eps)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """x fp32 [T, W] -> x / sqrt(mean(x^2) + eps) * weight in out_dtype (csrc/norm_shift.cu)."""
        if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
            raise _lib.B200Error("ResidualRMSNorm: a 2-D fp32 CUDA tensor with contiguous rows is expected")
        t, w = x.shape
        out = torch.empty((t, w), dtype=out_dtype, device=x.device)
        rc = _lib.load().b200_scalar_rmsnorm_shift(
            x.data_ptr(), x.stride(0), None, self.weight.data_ptr(), self.eps, None, None, 0, None, None, None,
            None, None, out.data_ptr(), out.stride(0), None, 0, t, w, _lib.dtype_code(out_dtype),
            _lib.current_stream())
        _lib.check(rc, "b200_scalar_rmsnorm_shift")
        return out


def softcap(z: torch.Tensor, cap: float) -> torch.Tensor:
    """-> fp32 cap * tanh(z / cap) (cap <= 0: a fp32 copy)."""
    if not z.is_cuda or z.dim() != 2 or z.stride(1) != 1:
        raise _lib.B200Error("softcap: a 2-D CUDA tensor with contiguous rows is expected")
    out = torch.empty(z.shape, dtype=torch.float32, device=z.device)
    rc = _lib.load().b200_softcap_rows(z.data_ptr(), z.stride(0), out.data_ptr(), out.stride(0),
                                       z.shape[0], z.shape[1], float(cap), _lib.dtype_code(z.dtype),
                                       _lib.current_stream())
    _lib.check(rc, "b200_softcap_rows")
    return out
