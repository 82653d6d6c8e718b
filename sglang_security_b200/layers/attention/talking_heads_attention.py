"""Grouped-query attention without rotation whose heads exchange their softmax weights (talking heads
after the softmax: Shazeer et al., "Talking-Heads Attention"), over a token pool whose row holds
[keys | values] of all key/value heads.  Per token at position p with mixer input h:

    [q ; k ; v ; z] = W h + b                   one fused GEMM (z: one gate pre-activation per head, no bias)
    q *= 1 + coef * ln(floor((p + 1) / every) + 1)                         query temperature
    v  = v / rms(v) per head;  v = (1 - lam) v + lam v_first               unit-RMS values, mixed with the
                                                  values another layer cached for the same token -> pool
    s_g(i, j) = cap * tanh(scale * q_g(i) . k_c(g)(j) / cap)               j <= i
    w_g(i, j) = exp(s_g) / (1 + sum_j exp(s_g))                            a sink of score 0 without a value
    w'_h      = sum_g M[h, g] w_g                                          heads' weights mixed
    out_h(i)  = sigmoid(z_h) * sum_j w'_h(i, j) v_c(h)(j);  result = W_o concat_h(out_h) + b_o

The mixed output is linear in the weights: out_h = sum_g M[h, g] A[c(h)][g] with A[c][g](i) = sum_j
w_g(i, j) v_c(j), so the attention kernels run their usual one-pass softmax once per VALUE head (every
query head's weights on that head's values) and csrc/head_mix.cu combines the planes per token and
applies the gate.  Prompt portions of at least `tensor_core_min_tokens` tokens run on the tcgen05 extend
kernel (16-bit operands, fp32 scores, maxima and sums; key and value size equal, 64 or 128; two value
heads per launch share one pass of scores and softmax, each with its own accumulator), decoded
tokens and short portions on the CUDA-core kernel (fp32 throughout; the only path of a 32-bit engine).
Both read the pool only, so a position's result does not depend on how the prompt was cut or batched
beyond rounding.  Every option is a parameter; without temperature, cap, mix and gate this is plain
grouped-query attention."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import _lib
from ..linear import ColumnParallelLinear, RowParallelLinear
from .sink_attention import SinkAttention


class TalkingHeadsAttention(nn.Module):
    # prompt portions at least this long go to the tensor-core kernel (0 = never); tests lower it
    tensor_core_min_tokens = 128

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 layer_id: int, eps: float, softcap: float = 0.0, temp_coef: float = 0.0,
                 temp_every: int = 0, value_norm: bool = True, unit_sink: bool = True,
                 head_gate: bool = True, bias: bool = True, v_first_layer: Optional[int] = None,
                 params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.layer_id, self.eps = float(scale), layer_id, float(eps)
        self.softcap, self.temp_coef, self.temp_every = float(softcap), float(temp_coef), int(temp_every)
        self.value_norm, self.head_gate = bool(value_norm), bool(head_gate)
        self.v_first_layer = v_first_layer          # layer whose cached values are mixed in (None: none)
        self.params_dtype = params_dtype
        kw = dict(params_dtype=params_dtype, tp_rank=0, tp_size=1)
        # [q ; k ; v ; gate], rows padded to a multiple of 8 (16-byte rows for the GEMM's output tiles)
        self.sizes = [heads * dim, kv_heads * dim, kv_heads * vdim, heads if head_gate else 0]
        total = (sum(self.sizes) + 7) // 8 * 8
        self.in_proj = ColumnParallelLinear(width, total, bias=bias, **kw)
        self.in_proj.weight.data.zero_()
        self.o_proj = RowParallelLinear(heads * vdim, width, bias=bias, **kw)
        f32 = dict(dtype=torch.float32)
        self.head_mix = nn.Parameter(torch.eye(heads, **f32), requires_grad=False)
        self.v_mix = nn.Parameter(torch.zeros((), **f32), requires_grad=False)
        self.register_buffer("sink", torch.zeros(heads, **f32) if unit_sink else None, persistent=False)

    @property
    def row_width(self) -> int:
        """Pool row of one token: keys of all key/value heads, then their values."""
        return self.kv_heads * (self.dim + self.vdim)

    def load_part(self, which: str, w: torch.Tensor, is_bias: bool = False) -> None:
        """which: "q", "k", "v" or "g" (the gate rows)."""
        i = "qkvg".index(which)
        lo = sum(self.sizes[:i])
        dst = self.in_proj.bias if is_bias else self.in_proj.weight
        if tuple(w.shape[:1]) != (self.sizes[i],):
            raise ValueError(f"projection {which!r}: {tuple(w.shape)} rows for {self.sizes[i]}")
        dst.data[lo:lo + self.sizes[i]].copy_(w)

    def _tensor_core_ok(self, h: torch.Tensor) -> bool:
        return (h.dtype in (torch.bfloat16, torch.float16) and self.dim == self.vdim and self.dim in (64, 128)
                and self.tensor_core_min_tokens > 0 and self.row_width % 8 == 0)

    def forward(self, h: torch.Tensor, fb) -> torch.Tensor:
        if not h.is_cuda:
            raise _lib.B200Error("TalkingHeadsAttention: tensors must live on a CUDA device (no CPU path)")
        T = h.shape[0]
        H, G, D, E = self.heads, self.kv_heads, self.dim, self.vdim
        y, _ = self.in_proj(h)
        a = self.sizes
        q, k, v = y[:, :a[0]], y[:, a[0]:a[0] + a[1]], y[:, a[0] + a[1]:a[0] + a[1] + a[2]]
        z = y[:, a[0] + a[1] + a[2]:] if self.head_gate else None
        pool = fb.token_to_kv_pool.get_kv_buffer(self.layer_id)
        if pool.dtype != h.dtype or pool.shape[1] != self.row_width:
            raise _lib.B200Error("TalkingHeadsAttention: the token pool does not fit this layer")
        first = None
        if self.v_first_layer is not None:
            first = fb.token_to_kv_pool.get_kv_buffer(self.v_first_layer)
            if first.dtype != pool.dtype or first.shape[1] < G * E:
                raise _lib.B200Error("TalkingHeadsAttention: the first layer's rows do not hold these values")
        lib, st, code = _lib.load(), _lib.current_stream(), _lib.dtype_code(h.dtype)
        plan = SinkAttention._plan(fb, self.tensor_core_min_tokens) if self._tensor_core_ok(h) else None
        n_core = T if plan is None else plan["n_rest"]           # tokens of the CUDA-core kernel
        q32 = torch.empty((T, H * D), dtype=torch.float32, device=h.device) if n_core else None
        q16 = torch.empty((T, H * D), dtype=h.dtype, device=h.device) if plan is not None else None
        rc = lib.b200_qkv_prep_write(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), None, None, 0, 0,
            self.eps, None, None, 0, fb.tok_pos.data_ptr(), fb.out_cache_loc.data_ptr(), pool.data_ptr(),
            pool.stride(0), 0, G * D, _lib.ptr(q32), H * D, _lib.ptr(q16), H * D, T, H, G, D, E,
            self.temp_coef, self.temp_every, 1 if self.value_norm else 0,
            self.v_mix.data_ptr() if first is not None else None, _lib.ptr(first),
            first.stride(0) if first is not None else 0,
            first.shape[1] - G * E if first is not None else 0, code, st)
        _lib.check(rc, "b200_qkv_prep_write")
        r2t = fb.req_to_token_pool.req_to_token
        out = torch.empty((T, H * E), dtype=h.dtype, device=h.device)
        if n_core:
            planes = torch.empty((G, T, H * E), dtype=torch.float32, device=h.device)
            rc = lib.b200_sink_attn_heads(
                q32.data_ptr(), q32.stride(0), pool.data_ptr(), pool.stride(0), 0, G * D, r2t.data_ptr(),
                r2t.stride(0), fb.req_pool_indices.data_ptr(), fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(),
                _lib.ptr(self.sink), self.scale, self.softcap, 0, 0, planes.data_ptr(), planes.stride(1), 1,
                planes.stride(0), n_core, H, G, D, E, _lib.ptr(plan["rest"]) if plan is not None else None,
                fb.max_seq_len, code, st)
            _lib.check(rc, "b200_sink_attn_heads")
            for start, n in ([(0, T)] if plan is None else plan["rest_ranges"]):
                self._mix(planes, z, out, start, n, code, st)
        if plan is not None:
            planes16 = torch.empty((G, T, H * E), dtype=h.dtype, device=h.device)
            for gv in range(0, G, 2):           # two value heads per launch: scores and softmax once
                pair = 2 if gv + 1 < G else 1
                rc = lib.b200_attn_extend_heads(
                    q16.data_ptr(), q16.stride(0), pool.data_ptr(), pool[:, G * D:].data_ptr(), pool.stride(0),
                    planes16[gv].data_ptr(), planes16.stride(1), r2t.data_ptr(), r2t.stride(0),
                    plan["req"].data_ptr(), plan["seq"].data_ptr(), plan["prefix"].data_ptr(),
                    plan["ext"].data_ptr(), plan["start"].data_ptr(), plan["bs"], plan["max_ext"], H, G, D, E,
                    self.scale, self.softcap, 1.0, 1, 0, 0, _lib.ptr(self.sink), gv if G > 1 else -1, pair,
                    planes16.stride(0), code, st)
                _lib.check(rc, "b200_attn_extend_heads")
            for start, n in plan["ranges"]:
                self._mix(planes16, z, out, start, n, code, st)
        res, _ = self.o_proj(out)
        return res

    def _mix(self, planes: torch.Tensor, z: Optional[torch.Tensor], out: torch.Tensor, start: int, n: int,
             code: int, st) -> None:
        """Rows start .. start + n of `out` from the same rows of the value-head planes."""
        rc = _lib.load().b200_head_mix_gate(
            planes[0, start:].data_ptr(), planes.stride(1), planes.stride(0), _lib.dtype_code(planes.dtype),
            self.head_mix.data_ptr(), z[start:].data_ptr() if z is not None else None,
            z.stride(0) if z is not None else 0, out[start:].data_ptr(), out.stride(0), n, self.heads,
            self.kv_heads, self.vdim, code, st)
        _lib.check(rc, "b200_head_mix_gate")
