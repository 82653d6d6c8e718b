"""Grouped-query softmax attention over a sliding window plus pooled blocks of the tokens before it
(csrc/pooled_attn.cu), over the one-row-per-token pool ([keys | values] of all key/value heads) and its
block-summary buffer:

  * biases on q, k, v; RMS norm of every query and key head with one weight [dim] shared by the heads,
    before rotation;
  * rotary positions on the first `rope_dims` coordinates of a head, pairing "half" (i with i + dims/2)
    or "neighbour" (2i with 2i + 1);
  * values rotated by their own position over the whole head before they are cached, the attention's
    output turned back by the query's position (`rotate_values`);
  * a learned multiplier per query head on the scores, besides the fixed scale;
  * position p sees the tokens j with 0 <= p - j < window and one pooled key / value (the mean of the
    cached rows) for each block of `pool` tokens that ends at or before p - window; one softmax.
Per step: one fused GEMM [q ; k ; v] with bias, one launch that norms, rotates and writes the pool row,
one that forms the means of the blocks completed in this step (from the pool, so the cut of the prompt
does not matter), the attention over req_to_token, W_o."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import _lib
from ..linear import ColumnParallelLinear, RowParallelLinear


def _split_frequencies(base: float, dims: int):
    """base^(-2i / dims), i < dims / 2, as a sum of two fp32 tables: position * frequency keeps
    fp64-like accuracy at large positions although every device operation on it is a 32-bit one."""
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    hi = f.to(torch.float32)
    return hi, (f - hi.double()).to(torch.float32)


class PooledWindowAttention(nn.Module):
    PAIRINGS = {"neighbour": 0, "half": 1}

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, layer_id: int,
                 eps: float, window: Optional[int] = None, pool: int = 0, rope_base: float = 10000.0,
                 rope_dims: int = 0, pairing: str = "half", rotate_values: bool = True, qk_norm: bool = True,
                 head_scale: bool = True, bias: bool = True, params_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if pairing not in self.PAIRINGS:
            raise ValueError(f"unknown pairing {pairing!r}")
        if pool and not window:
            raise ValueError("pooled blocks need a window")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.layer_id, self.eps = float(scale), layer_id, float(eps)
        self.window, self.pool = int(window) if window else 0, int(pool)
        self.rope_dims, self.pairing = int(rope_dims), self.PAIRINGS[pairing]
        self.rotate_values = bool(rotate_values) and self.rope_dims > 0
        self.params_dtype = params_dtype
        kw = dict(params_dtype=params_dtype, tp_rank=0, tp_size=1)
        self.sizes = [heads * dim, kv_heads * dim, kv_heads * vdim]
        self.qkv_proj = ColumnParallelLinear(width, sum(self.sizes), bias=bias, **kw)
        self.o_proj = RowParallelLinear(heads * vdim, width, bias=False, **kw)
        f32 = dict(dtype=torch.float32)
        self.q_norm_weight = nn.Parameter(torch.ones(dim, **f32), requires_grad=False) if qk_norm else None
        self.k_norm_weight = nn.Parameter(torch.ones(dim, **f32), requires_grad=False) if qk_norm else None
        self.head_scale = nn.Parameter(torch.ones(heads, **f32), requires_grad=False) if head_scale else None
        if self.rope_dims:
            hi, lo = _split_frequencies(rope_base, self.rope_dims)
            self.register_buffer("freq_hi", hi, persistent=False)
            self.register_buffer("freq_lo", lo, persistent=False)
        if self.rotate_values:
            hi, lo = _split_frequencies(rope_base, vdim)
            self.register_buffer("vfreq_hi", hi, persistent=False)
            self.register_buffer("vfreq_lo", lo, persistent=False)

    @property
    def row_width(self) -> int:
        """Pool row of one token: keys of all key/value heads, then their values."""
        return self.kv_heads * (self.dim + self.vdim)

    def load_part(self, which: str, w: torch.Tensor, is_bias: bool = False) -> None:
        i = "qkv".index(which)
        lo = sum(self.sizes[:i])
        dst = self.qkv_proj.bias if is_bias else self.qkv_proj.weight
        dst.data[lo:lo + self.sizes[i]].copy_(w)

    def forward(self, h: torch.Tensor, fb) -> torch.Tensor:
        if not h.is_cuda:
            raise _lib.B200Error("PooledWindowAttention: tensors must live on a CUDA device (no CPU path)")
        T = h.shape[0]
        H, G, D, E = self.heads, self.kv_heads, self.dim, self.vdim
        y, _ = self.qkv_proj(h)
        a = self.sizes
        q, k, v = y[:, :a[0]], y[:, a[0]:a[0] + a[1]], y[:, a[0] + a[1]:]
        kvp = fb.token_to_kv_pool
        pool = kvp.get_kv_buffer(self.layer_id)
        if pool.dtype != h.dtype or pool.shape[1] != self.row_width:
            raise _lib.B200Error("PooledWindowAttention: the token pool does not fit this layer")
        lib, st, code = _lib.load(), _lib.current_stream(), _lib.dtype_code(h.dtype)
        rot, vrot = self.rope_dims > 0, self.rotate_values
        q32 = torch.empty((T, H * D), dtype=torch.float32, device=h.device)
        rc = lib.b200_headnorm_rot_write(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
            _lib.ptr(self.q_norm_weight), _lib.ptr(self.k_norm_weight), self.eps,
            self.freq_hi.data_ptr() if rot else None, self.freq_lo.data_ptr() if rot else None, self.rope_dims,
            self.vfreq_hi.data_ptr() if vrot else None, self.vfreq_lo.data_ptr() if vrot else None,
            self.pairing, _lib.ptr(self.head_scale), fb.tok_pos.data_ptr(), fb.out_cache_loc.data_ptr(),
            pool.data_ptr(), pool.stride(0), 0, G * D, q32.data_ptr(), q32.stride(0), T, H, G, D, E, code, st)
        _lib.check(rc, "b200_headnorm_rot_write")
        r2t = fb.req_to_token_pool.req_to_token
        summary, pdiv = None, 1
        if self.pool:
            summary, pdiv = kvp.get_block_summary(self.layer_id)
            if summary.shape[1] != self.row_width:
                raise _lib.B200Error("PooledWindowAttention: the block-summary buffer does not fit this layer")
            rc = lib.b200_pool_block_means(
                pool.data_ptr(), pool.stride(0), self.row_width, summary.data_ptr(), summary.stride(0),
                self.pool, pdiv, r2t.data_ptr(), r2t.stride(0), fb.req_pool_indices.data_ptr(),
                fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), T, code, st)
            _lib.check(rc, "b200_pool_block_means")
        out = torch.empty((T, H * E), dtype=h.dtype, device=h.device)
        if self.window:
            max_keys = min(fb.max_seq_len, self.window) + (fb.max_seq_len // self.pool if self.pool else 0)
        else:
            max_keys = fb.max_seq_len
        rc = lib.b200_pooled_window_attn(
            q32.data_ptr(), q32.stride(0), pool.data_ptr(), pool.stride(0), 0, G * D, _lib.ptr(summary),
            summary.stride(0) if summary is not None else 0, self.pool, pdiv, r2t.data_ptr(), r2t.stride(0),
            fb.req_pool_indices.data_ptr(), fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), self.scale, self.window,
            self.vfreq_hi.data_ptr() if vrot else None, self.vfreq_lo.data_ptr() if vrot else None, self.pairing,
            out.data_ptr(), out.stride(0), T, H, G, D, E, None, max_keys, code, st)
        _lib.check(rc, "b200_pooled_window_attn")
        res, _ = self.o_proj(out)
        return res
