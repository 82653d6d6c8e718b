"""Grouped-query softmax attention with the options of csrc/sink_attn.cu, over a token pool whose
row holds [keys | values] of all key/value heads (mem_cache/latent_pool.py's one-row-per-token pool):

  * biases on the projections; RMS norm of the whole query and of the whole key projection (all heads
    at once) with learned weights, before rotation;
  * interleaved rotary positions on the first `rope_dims` coordinates of each head;
  * a causal sliding window that keeps the first `keep_first` tokens of the sequence visible;
  * a learned sink per query head in the softmax denominator;
  * key size and value size that differ.
Per step: one fused GEMM [q ; k ; v] (with bias), one launch that norms, rotates and writes the pool
row, the attention over req_to_token, W_o.  The attention of a step is divided by batch entry: prompt
portions of at least `tensor_core_min_tokens` tokens run on the tcgen05 extend kernel
(csrc/attn_extend.cu: 16-bit operands, fp32 scores, maxima and sums; key and value size equal, 64 or
128), decoded tokens and short portions on the CUDA-core kernel, which keeps the weights in fp32 too and
is the only path of a 32-bit engine.  Both read the pool only, so a position's result does not depend
on the cut of the prompt or on the batch beyond rounding."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import _lib
from ..linear import ColumnParallelLinear, RowParallelLinear


class SinkAttention(nn.Module):
    # prompt portions at least this long go to the tensor-core kernel (0 = never); tests lower it
    tensor_core_min_tokens = 128

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 layer_id: int, eps: float, window: Optional[int] = None, keep_first: int = 0,
                 rope_base: float = 10000.0, rope_dims: int = 0, qk_norm: str = "whole",
                 sink: bool = True, bias: bool = True, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if qk_norm not in ("whole", "head", "none"):
            raise ValueError(f"unknown query/key norm {qk_norm!r}")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.layer_id, self.eps = float(scale), layer_id, float(eps)
        self.window, self.keep_first = int(window) if window else 0, int(keep_first)
        self.rope_dims = int(rope_dims)
        self.params_dtype = params_dtype
        kw = dict(params_dtype=params_dtype, tp_rank=0, tp_size=1)
        self.sizes = [heads * dim, kv_heads * dim, kv_heads * vdim]
        self.qkv_proj = ColumnParallelLinear(width, sum(self.sizes), bias=bias, **kw)
        self.o_proj = RowParallelLinear(heads * vdim, width, bias=bias, **kw)
        self.q_group = {"whole": heads * dim, "head": dim, "none": 0}[qk_norm]
        self.k_group = {"whole": kv_heads * dim, "head": dim, "none": 0}[qk_norm]
        f32 = dict(dtype=torch.float32)
        self.q_norm_weight = nn.Parameter(torch.ones(heads * dim, **f32), requires_grad=False) if self.q_group else None
        self.k_norm_weight = nn.Parameter(torch.ones(kv_heads * dim, **f32), requires_grad=False) if self.k_group else None
        self.sink = nn.Parameter(torch.zeros(heads, **f32), requires_grad=False) if sink else None
        # frequency base^(-2i / dims) as a sum of two floats: the angle position * frequency keeps
        # fp64-like accuracy at large positions although every operation on it is a 32-bit one
        f = torch.tensor([float(rope_base) ** (-2.0 * i / self.rope_dims) for i in range(self.rope_dims // 2)],
                         dtype=torch.float64)
        hi = f.to(torch.float32)
        self.register_buffer("freq_hi", hi, persistent=False)
        self.register_buffer("freq_lo", (f - hi.double()).to(torch.float32), persistent=False)

    @property
    def row_width(self) -> int:
        """Pool row of one token: keys of all key/value heads, then their values."""
        return self.kv_heads * (self.dim + self.vdim)

    def load_part(self, which: str, w: torch.Tensor, is_bias: bool = False) -> None:
        i = "qkv".index(which)
        lo = sum(self.sizes[:i])
        dst = self.qkv_proj.bias if is_bias else self.qkv_proj.weight
        dst.data[lo:lo + self.sizes[i]].copy_(w)

    def _tensor_core_ok(self, h: torch.Tensor) -> bool:
        return (h.dtype in (torch.bfloat16, torch.float16) and self.dim == self.vdim and self.dim in (64, 128)
                and self.tensor_core_min_tokens > 0)

    @staticmethod
    def _merged(ranges):
        """(first row, rows) ranges in row order, neighbours joined."""
        out = []
        for start, n in ranges:
            if out and out[-1][0] + out[-1][1] == start:
                out[-1] = (out[-1][0], out[-1][1] + n)
            else:
                out.append((start, n))
        return out

    @staticmethod
    def _plan(fb, min_tokens: int):
        """Which batch entries take the tensor-core kernel: their sub-tables (one host-to-device copy),
        and the rows of all other tokens.  Shared by the layers of a step."""
        key = ("sink_attn_plan", min_tokens)
        if key in fb.extra:
            return fb.extra[key]
        ext, pre = fb.extend_seq_lens_cpu, fb.extend_prefix_lens_cpu
        long = [b for b, n in enumerate(ext) if n >= min_tokens]
        plan = None
        if long:
            starts, at = [], 0
            for n in ext:
                starts.append(at)
                at += n
            rest = [t for b, n in enumerate(ext) if n < min_tokens for t in range(starts[b], starts[b] + n)]
            host = torch.tensor([long, [pre[b] for b in long], [ext[b] for b in long],
                                 [starts[b] for b in long], [pre[b] + ext[b] for b in long]], dtype=torch.int64)
            dev = host.to(fb.req_pool_indices.device, non_blocking=True)
            plan = {"bs": len(long), "max_ext": max(ext[b] for b in long),
                    "req": fb.req_pool_indices[dev[0]], "prefix": dev[1].to(torch.int32),
                    "ext": dev[2].to(torch.int32), "start": dev[3].to(torch.int32), "seq": dev[4].contiguous(),
                    "rest": (torch.tensor(rest, dtype=torch.int32).to(fb.req_pool_indices.device, non_blocking=True)
                             if rest else None), "n_rest": len(rest),
                    # (first row, rows) of the entries of either kind, for per-row steps that follow
                    "ranges": SinkAttention._merged([(starts[b], ext[b]) for b in long]),
                    "rest_ranges": SinkAttention._merged([(starts[b], n) for b, n in enumerate(ext)
                                                          if n < min_tokens])}
        fb.extra[key] = plan
        return plan

    def forward(self, h: torch.Tensor, fb) -> torch.Tensor:
        if not h.is_cuda:
            raise _lib.B200Error("SinkAttention: tensors must live on a CUDA device (no CPU path)")
        T = h.shape[0]
        H, G, D, E = self.heads, self.kv_heads, self.dim, self.vdim
        y, _ = self.qkv_proj(h)
        a = self.sizes
        q, k, v = y[:, :a[0]], y[:, a[0]:a[0] + a[1]], y[:, a[0] + a[1]:]
        pool = fb.token_to_kv_pool.get_kv_buffer(self.layer_id)
        if pool.dtype != h.dtype or pool.shape[1] != self.row_width:
            raise _lib.B200Error("SinkAttention: the token pool does not fit this layer")
        lib, st, code = _lib.load(), _lib.current_stream(), _lib.dtype_code(h.dtype)
        plan = self._plan(fb, self.tensor_core_min_tokens) if self._tensor_core_ok(h) else None
        n_core = T if plan is None else plan["n_rest"]           # tokens of the CUDA-core kernel
        q32 = torch.empty((T, H * D), dtype=torch.float32, device=h.device) if n_core else None
        q16 = torch.empty((T, H * D), dtype=h.dtype, device=h.device) if plan is not None else None
        rot = self.rope_dims > 0
        rc = lib.b200_qk_norm_rope_write(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
            _lib.ptr(self.q_norm_weight), _lib.ptr(self.k_norm_weight), self.q_group, self.k_group,
            self.eps, self.freq_hi.data_ptr() if rot else None, self.freq_lo.data_ptr() if rot else None,
            self.rope_dims, fb.tok_pos.data_ptr(), fb.out_cache_loc.data_ptr(), pool.data_ptr(),
            pool.stride(0), 0, G * D, _lib.ptr(q32), H * D, _lib.ptr(q16), H * D, T, H, G, D, E, code, st)
        _lib.check(rc, "b200_qk_norm_rope_write")
        r2t = fb.req_to_token_pool.req_to_token
        out = torch.empty((T, H * E), dtype=h.dtype, device=h.device)
        if plan is not None:
            rc = lib.b200_attn_extend_sink(
                q16.data_ptr(), q16.stride(0), pool.data_ptr(), pool[:, G * D:].data_ptr(), pool.stride(0),
                out.data_ptr(), out.stride(0), r2t.data_ptr(), r2t.stride(0), plan["req"].data_ptr(),
                plan["seq"].data_ptr(), plan["prefix"].data_ptr(), plan["ext"].data_ptr(),
                plan["start"].data_ptr(), plan["bs"], plan["max_ext"], H, G, D, E, self.scale, 0.0, 1.0, 1,
                self.window, self.keep_first, _lib.ptr(self.sink), code, st)
            _lib.check(rc, "b200_attn_extend_sink")
        if n_core:
            rc = lib.b200_sink_attn(
                q32.data_ptr(), q32.stride(0), pool.data_ptr(), pool.stride(0), 0, G * D, r2t.data_ptr(),
                r2t.stride(0), fb.req_pool_indices.data_ptr(), fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(),
                _lib.ptr(self.sink), self.scale, self.window, self.keep_first, out.data_ptr(), out.stride(0),
                n_core, H, G, D, E, _lib.ptr(plan["rest"]) if plan is not None else None,
                min(fb.max_seq_len, self.window + self.keep_first) if self.window else fb.max_seq_len, code, st)
            _lib.check(rc, "b200_sink_attn")
        res, _ = self.o_proj(out)
        return res
