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
does not matter), the attention over req_to_token, W_o.  The attention of a step is divided by batch
entry: prompt portions of at least `tensor_core_min_tokens` tokens take the tcgen05 extend kernel for
the window (16-bit operands, fp32 scores and sums; key size = value size, 64 or 128) with the log-sum of
every row, the CUDA-core kernel for the few pooled blocks alone, and one launch that joins the two parts
as one softmax and turns the result back; decoded tokens, short portions and every step of a 32-bit
engine take the CUDA-core kernel for everything.  Both read the pool only."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import _lib
from ..linear import ColumnParallelLinear, RowParallelLinear
from .sink_attention import SinkAttention


def _split_frequencies(base: float, dims: int):
    """base^(-2i / dims), i < dims / 2, as a sum of two fp32 tables: position * frequency keeps
    fp64-like accuracy at large positions although every device operation on it is a 32-bit one."""
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    hi = f.to(torch.float32)
    return hi, (f - hi.double()).to(torch.float32)


class PooledWindowAttention(nn.Module):
    PAIRINGS = {"neighbour": 0, "half": 1}
    # prompt portions at least this long go to the tensor-core kernel (0 = never); tests lower it
    tensor_core_min_tokens = 128

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

    def _tensor_core_ok(self, h: torch.Tensor) -> bool:
        return (h.dtype in (torch.bfloat16, torch.float16) and self.dim == self.vdim and self.dim in (64, 128)
                and self.tensor_core_min_tokens > 0)

    @staticmethod
    def _long_rows(fb, plan):
        """Token rows of the entries that take the tensor-core kernel, as a device list (shared by the layers)."""
        key = ("pooled_attn_long_rows", plan["bs"], plan["max_ext"])
        if key not in fb.extra:
            rows = [t for start, n in plan["ranges"] for t in range(start, start + n)]
            fb.extra[key] = torch.tensor(rows, dtype=torch.int32).to(fb.req_pool_indices.device, non_blocking=True)
        return fb.extra[key]

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
        plan = SinkAttention._plan(fb, self.tensor_core_min_tokens) if self._tensor_core_ok(h) else None
        q32 = torch.empty((T, H * D), dtype=torch.float32, device=h.device)
        q16 = torch.empty((T, H * D), dtype=h.dtype, device=h.device) if plan is not None else None
        rc = lib.b200_headnorm_rot_write(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
            _lib.ptr(self.q_norm_weight), _lib.ptr(self.k_norm_weight), self.eps,
            self.freq_hi.data_ptr() if rot else None, self.freq_lo.data_ptr() if rot else None, self.rope_dims,
            self.vfreq_hi.data_ptr() if vrot else None, self.vfreq_lo.data_ptr() if vrot else None,
            self.pairing, _lib.ptr(self.head_scale), fb.tok_pos.data_ptr(), fb.out_cache_loc.data_ptr(),
            pool.data_ptr(), pool.stride(0), 0, G * D, q32.data_ptr(), q32.stride(0), _lib.ptr(q16), H * D,
            T, H, G, D, E, code, st)
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
        ld_sum = summary.stride(0) if summary is not None else 0
        vhi = self.vfreq_hi.data_ptr() if vrot else None
        vlo = self.vfreq_lo.data_ptr() if vrot else None
        n_core = T if plan is None else plan["n_rest"]           # tokens of the CUDA-core kernel
        if plan is not None:
            # long portions: the window on the tensor cores, the blocks beside it, joined as one softmax
            n_long = T - n_core
            long_rows = self._long_rows(fb, plan)
            lse1 = torch.empty((T, H), dtype=torch.float32, device=h.device)
            rc = lib.b200_attn_extend_lse(
                q16.data_ptr(), q16.stride(0), pool.data_ptr(), pool[:, G * D:].data_ptr(), pool.stride(0),
                out.data_ptr(), out.stride(0), r2t.data_ptr(), r2t.stride(0), plan["req"].data_ptr(),
                plan["seq"].data_ptr(), plan["prefix"].data_ptr(), plan["ext"].data_ptr(),
                plan["start"].data_ptr(), plan["bs"], plan["max_ext"], H, G, D, E, self.scale, self.window,
                lse1.data_ptr(), lse1.stride(0), code, st)
            _lib.check(rc, "b200_attn_extend_lse")
            part = lse2 = None
            if self.pool:
                part = torch.empty((T, H * E), dtype=torch.float32, device=h.device)
                lse2 = torch.empty((T, H), dtype=torch.float32, device=h.device)
                rc = lib.b200_pooled_blocks_attn_part(
                    q32.data_ptr(), q32.stride(0), pool.data_ptr(), pool.stride(0), 0, G * D, summary.data_ptr(),
                    ld_sum, self.pool, pdiv, r2t.data_ptr(), r2t.stride(0), fb.req_pool_indices.data_ptr(),
                    fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), self.scale, self.window, part.data_ptr(),
                    part.stride(0), lse2.data_ptr(), lse2.stride(0), n_long, H, G, D, E, long_rows.data_ptr(),
                    fb.max_seq_len // self.pool, code, st)
                _lib.check(rc, "b200_pooled_blocks_attn_part")
            if part is not None or vrot:
                rc = lib.b200_pooled_merge_unrotate(
                    out.data_ptr(), out.stride(0), lse1.data_ptr(), lse1.stride(0), _lib.ptr(part),
                    part.stride(0) if part is not None else 0, _lib.ptr(lse2),
                    lse2.stride(0) if lse2 is not None else 0, vhi, vlo, self.pairing, fb.tok_pos.data_ptr(),
                    long_rows.data_ptr(), n_long, H, E, code, st)
                _lib.check(rc, "b200_pooled_merge_unrotate")
        if n_core:
            rc = lib.b200_pooled_window_attn(
                q32.data_ptr(), q32.stride(0), pool.data_ptr(), pool.stride(0), 0, G * D, _lib.ptr(summary),
                ld_sum, self.pool, pdiv, r2t.data_ptr(), r2t.stride(0), fb.req_pool_indices.data_ptr(),
                fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), self.scale, self.window, vhi, vlo, self.pairing,
                out.data_ptr(), out.stride(0), n_core, H, G, D, E,
                _lib.ptr(plan["rest"]) if plan is not None else None, max_keys, code, st)
            _lib.check(rc, "b200_pooled_window_attn")
        res, _ = self.o_proj(out)
        return res
