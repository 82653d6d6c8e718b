"""Latent attention layer (queries and keys/values through low-rank latents, one rotated key part
shared by all heads, optional causal sliding window, optional reuse of another layer's latent) over
LatentTokenToKVPool, on the kernels of csrc/latent_attn.cu.

Per token with mixer input h (dims: H heads, `dim` unrotated + `rot_dim` rotated query/key
coordinates, value size `vdim`, latent size R):
    [cq_raw | ckv_raw] = W_down h                    (one fused GEMM; layers that borrow a latent: W_dq only)
    cq = RMSnorm(cq_raw) * w_q ;  c = RMSnorm(ckv_raw[:R]) * w_kv ;  kr = rotary(ckv_raw[R:])  -> pool
    q  = W_uq cq                                      [H, dim + rot_dim]
    q_lat[h] = W_uk[h]^T q[h, :dim]                   (absorbed key up-projection, fp32 result)
    p  = softmax_j((q_lat[h] . c_j + rotary(q[h, dim:]) . kr_j) * scale)   over the visible keys
    out = W_o concat_h(W_uv[h] sum_j p_j c_j)
Only c and kr are cached.  Two forms of the same sum run on them:
  * absorbed (above): every query attends to the latent rows themselves, head size R + rot_dim.
    It needs nothing per key but the cached row, so it serves decoded tokens and short portions
    (and every step of a 32-bit engine).
  * expanded: for a step whose new tokens outweigh the keys they see, K_j[h] = [W_uk[h] c_j | kr_j]
    and V_j[h] = W_uv[h] c_j are formed once per visible key by one GEMM and the step runs as
    ordinary causal windowed multi-head attention of head size max(dim + rot_dim, vdim) (padded to
    64 or 128) on the tcgen05 extend kernel: (dim + rot_dim + vdim) instead of (2 R + rot_dim)
    multiply-adds per score.  16-bit engines only; chosen per step by a cost estimate.
Both read the cache only, so a position's result does not depend on how the sequence was cut into
steps or batched, beyond rounding.

Variants, all parameters: `q_rank=None` projects the queries straight from h (no query latent and no
norm of it): one fused GEMM [W_q ; W_dkv ; W_g]; `gate=True` multiplies the concatenated heads element
by element with sigmoid(W_g h) before W_o; `rotary` replaces the default rotation by one with its own
frequency table, pairing and sine/cosine multiplier (layers/rotary_embedding.py PairedRotary: a
checkpoint in the half pairing has its rotated rows reordered as it is loaded, and the squared
multiplier goes onto the cached key part)."""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn as nn

from ... import _lib
from ..linear import ColumnParallelLinear, RowParallelLinear
from ..rotary_embedding import InterleavedRotary, PairedRotary


_SM_COUNT = 148      # B200
# relative speed of the kernels in the cost estimate that picks the form of a step: the library GEMM
# and the tcgen05 extend kernel against the mma.sync latent kernel, and the most scratch the expanded
# keys and values may take
_GEMM_SPEEDUP, _EXTEND_SPEEDUP, _EXPAND_MAX_BYTES = 10.0, 4.0, 1 << 30
# what the expanded form's extra launches and tables cost per layer, in multiply-adds of the latent
# kernel (about 0.15 ms): below this saving a step stays absorbed (measured: a 512-token portion beside
# 32 decoded tokens is faster absorbed, a 2048-token prompt 2 to 4 times faster expanded)
_EXPAND_FIXED = 6e9


def _visible_pairs(prefix: int, new: int, window: int) -> int:
    """Number of (query, key) pairs of `new` tokens after `prefix` cached ones under a causal window."""
    a = prefix + 1
    if not window:
        return new * a + new * (new - 1) // 2
    k = min(max(window - a, 0), new)
    return k * a + k * (k - 1) // 2 + (new - k) * window


def _bmm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched product with a fp32 result (16-bit operands keep their tensor-core path)."""
    if a.dtype == torch.float32:
        return torch.bmm(a, b)
    try:
        return torch.bmm(a, b, out_dtype=torch.float32)
    except (TypeError, RuntimeError):
        return torch.bmm(a.float(), b.float())


class LatentAttention(nn.Module):
    # None: the cost estimate picks the form of every step; "absorbed" / "expanded" pin it, "split"
    # divides every step by the per-entry estimate alone, without the fixed cost (A/B measurements and
    # tests at small sizes; where the expanded form does not exist the step stays absorbed)
    force_form: Optional[str] = None

    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 q_rank: Optional[int], scale: float, layer_id: int, eps: float, window: Optional[int] = None,
                 rope_base: float = 10000.0, rope_dims: Optional[int] = None,
                 kv_layer_id: Optional[int] = None, params_dtype: torch.dtype = torch.bfloat16,
                 rotary: Optional[PairedRotary] = None, gate: bool = False):
        super().__init__()
        self.width, self.heads, self.dim, self.rot_dim, self.vdim = width, heads, dim, rot_dim, vdim
        self.kv_rank, self.q_rank, self.scale, self.eps = kv_rank, q_rank, float(scale), eps
        self.layer_id = layer_id
        self.kv_layer_id = layer_id if kv_layer_id is None else kv_layer_id
        self.owns_kv = self.kv_layer_id == layer_id
        self.window = int(window) if window else 0
        kw = dict(bias=False, params_dtype=params_dtype, tp_rank=0, tp_size=1)
        self.gate = bool(gate)
        q_out = heads * (dim + rot_dim)
        # rows of the first GEMM: the query part (its latent, or the queries themselves), the KV latent
        # and key part of a layer that owns them, the gate; padded to a multiple of 8
        self.q_part = q_rank if q_rank is not None else q_out
        self.kv_part = kv_rank + rot_dim if self.owns_kv else 0
        self.gate_part = heads * vdim if gate else 0
        down_out = self.q_part + self.kv_part + self.gate_part
        if q_rank is None:
            down_out = (down_out + 7) // 8 * 8
        self.down_proj = ColumnParallelLinear(width, down_out, **kw)     # [W_dq or W_q ; W_dkv ; W_g]
        if down_out != self.q_part + self.kv_part + self.gate_part:
            self.down_proj.weight.data.zero_()
        self.q_up_proj = ColumnParallelLinear(q_rank, q_out, **kw) if q_rank is not None else None
        self.o_proj = RowParallelLinear(heads * vdim, width, **kw)
        self.w_uk = nn.Parameter(torch.empty(heads, dim, kv_rank, dtype=params_dtype), requires_grad=False)
        self.w_uv_t = nn.Parameter(torch.empty(heads, kv_rank, vdim, dtype=params_dtype), requires_grad=False)
        self.q_norm_weight = (nn.Parameter(torch.ones(q_rank, dtype=torch.float32), requires_grad=False)
                              if q_rank is not None else None)
        self.kv_norm_weight = nn.Parameter(torch.ones(kv_rank, dtype=torch.float32), requires_grad=False)
        self.rotary = rotary if rotary is not None else InterleavedRotary(
            rot_dim if rope_dims is None else rope_dims, rope_base)
        # sine and cosine multiplied by m on the query and the key side: m^2 on the cached key part
        self.rot_scale = float(getattr(self.rotary, "amplitude", 1.0)) ** 2
        if self.rotary.dims > rot_dim:
            raise ValueError("rotary dims exceed the rotated part of a head")
        need = max(dim + rot_dim, vdim)
        self.expand_dim = 64 if need <= 64 else (128 if need <= 128 else 0)   # 0: no expanded form
        self._w_expand = None

    # ---- checkpoint tensors ([out, in]) -> the layouts above ------------------------------------
    def load_down(self, w_dq: torch.Tensor, w_dkv: Optional[torch.Tensor]) -> None:
        w = w_dq if w_dkv is None else torch.cat([w_dq, w_dkv], 0)
        self.down_proj.weight.data.copy_(w)

    def load_direct(self, w_q: torch.Tensor, w_dkv: torch.Tensor, w_g: Optional[torch.Tensor]) -> None:
        """Checkpoint tensors of the variant without a query latent: W_q [H * (dim + rot_dim), width],
        W_dkv [kv_rank + rot_dim, width], W_g [H * vdim, width].  The rotated rows of every query head and
        of the key part are taken in the rotation's row order (half pairing -> neighbours)."""
        if self.q_up_proj is not None or not self.owns_kv:
            raise ValueError("load_direct is for a layer that projects its queries directly and owns its latent")
        H, dq = self.heads, self.dim + self.rot_dim
        order = getattr(self.rotary, "row_order", lambda n: torch.arange(n))(self.rot_dim).to(w_q.device)
        wq = w_q.view(H, dq, -1)
        wq = torch.cat([wq[:, :self.dim], wq[:, self.dim:][:, order]], 1).reshape(H * dq, -1)
        wkv = torch.cat([w_dkv[:self.kv_rank], w_dkv[self.kv_rank:][order]], 0)
        dst = self.down_proj.weight.data
        dst[:self.q_part].copy_(wq)
        dst[self.q_part:self.q_part + self.kv_part].copy_(wkv)
        if self.gate:
            dst[self.q_part + self.kv_part:self.q_part + self.kv_part + self.gate_part].copy_(w_g)

    def load_uk(self, w: torch.Tensor) -> None:      # [H * dim, R]
        self.w_uk.data.copy_(w.view(self.heads, self.dim, self.kv_rank))
        self._w_expand = None

    def load_uv(self, w: torch.Tensor) -> None:      # [H * vdim, R] -> [H, R, vdim]
        self.w_uv_t.data.copy_(w.view(self.heads, self.vdim, self.kv_rank).transpose(1, 2))
        self._w_expand = None

    # ---- expanded form ---------------------------------------------------------------------------
    def _expand_weight(self) -> torch.Tensor:
        """[2 * H * D, R]: rows (h, d < dim) = W_uk[h], rows H*D + (h, d < vdim) = W_uv[h], zero
        elsewhere, so one GEMM writes keys and values in the head-major layout the kernel reads."""
        if self._w_expand is None:
            H, D = self.heads, self.expand_dim
            w = torch.zeros((2, H, D, self.kv_rank), dtype=self.w_uk.dtype, device=self.w_uk.device)
            w[0, :, :self.dim] = self.w_uk
            w[1, :, :self.vdim] = self.w_uv_t.transpose(1, 2)
            self._w_expand = w.view(2 * H * D, self.kv_rank)
        return self._w_expand

    def _expand_plan(self, fb):
        """The step's gather tables for the expanded form, or False when the absorbed form is the
        cheaper one.  Shared by the layers of equal window through fb.extra."""
        key = ("latent_expand", self.window, self.heads, self.kv_rank, self.rot_dim, self.expand_dim)
        if key in fb.extra:
            return fb.extra[key]
        plan = fb.extra[key] = self._make_expand_plan(fb)
        return plan

    def _absorbed_takes_subsets(self, fb) -> bool:
        """Whether the absorbed kernel that would run walks the batch entry by entry (the tiled 16-bit
        instance does; the CUDA-core one walks all tokens), i.e. whether a step may be divided."""
        cache = fb.token_to_kv_pool.get_kv_buffer(self.layer_id) if fb.token_to_kv_pool is not None else None
        return (cache is not None and cache.dtype in (torch.bfloat16, torch.float16)
                and self.kv_rank % 8 == 0 and self.rot_dim % 8 == 0 and self.kv_rank <= 512
                and cache.stride(0) % 8 == 0 and os.environ.get("B200_LATENT_ATTN_MMA", "1")[:1] != "0")

    def _make_expand_plan(self, fb):
        pre, ext = fb.extend_prefix_lens_cpu, fb.extend_seq_lens_cpu
        forced = self.force_form
        if not self.expand_dim or pre is None or ext is None or forced == "absorbed":
            return False
        if forced is None and max(ext) < 16:
            return False
        H, D, R, W = self.heads, self.expand_dim, self.kv_rank, self.window
        bs = len(ext)
        lo = [max(0, p - W + 1) if W else 0 for p in pre]
        n = [p + e - l for p, e, l in zip(pre, ext, lo)]
        # cost of every entry in either form (multiply-adds weighted by the speed of their kernel)
        absorbed = [_visible_pairs(p, e, W) * H * (2 * R + self.rot_dim) for p, e in zip(pre, ext)]
        expanded = [k * 2 * H * D * R / _GEMM_SPEEDUP
                    + ((e + 127) // 128 * 128) * ((min(k, (W or k) + 128) + 63) // 64 * 64) * H * 2 * D
                    / _EXTEND_SPEEDUP for e, k in zip(ext, n)]          # 128 x 64 tiles touched
        if forced == "expanded":
            take = [True] * bs
        else:
            take = [e >= 16 and x < a for e, x, a in zip(ext, expanded, absorbed)]
            if any(take) and not all(take) and not self._absorbed_takes_subsets(fb):
                take = [sum(expanded) < sum(absorbed)] * bs              # undivided step: one form for all
            saved = sum(a - x for a, x, t in zip(absorbed, expanded, take) if t)
            if forced != "split" and saved < _EXPAND_FIXED:
                return False
        B = [b for b in range(bs) if take[b]]
        if not B:
            return False
        N = sum(n[b] for b in B)
        if N * 2 * H * D * 2 > _EXPAND_MAX_BYTES and forced != "expanded":
            return False
        dev = fb.req_pool_indices.device
        off, at = [], 0
        for b in B:
            off.append(at)
            at += n[b]
        key_b = torch.repeat_interleave(torch.tensor(B), torch.tensor([n[b] for b in B]))
        key_pos = torch.cat([torch.arange(lo[b], lo[b] + n[b]) for b in B])
        host = torch.tensor([off, [pre[b] - lo[b] for b in B], [n[b] for b in B], B], dtype=torch.int64)
        tab = host.to(dev, non_blocking=True)
        kb, kp = key_b.to(dev, non_blocking=True), key_pos.to(dev, non_blocking=True)
        r2t = fb.req_to_token_pool.req_to_token
        slots = r2t[fb.req_pool_indices[kb], kp].to(torch.int64)
        max_n = max(n[b] for b in B)
        rtt = (tab[0][:, None] + torch.arange(max_n, device=dev)[None, :]).to(torch.int32).contiguous()
        plan = dict(N=N, slots=slots, rtt=rtt, prefix=tab[1].to(torch.int32), seq=tab[2].contiguous(),
                    rows=torch.arange(len(B), dtype=torch.int64, device=dev), bs=len(B),
                    max_ext=max(ext[b] for b in B), rest=None)
        if len(B) == bs:
            plan["ext_len"], plan["ext_start"] = fb.ext_len, fb.ext_start
            return plan
        # a divided step: the entries in B run expanded, the others absorbed, each on its own rows
        A = [b for b in range(bs) if not take[b]]
        idx_a = torch.tensor(A, dtype=torch.int64).to(dev, non_blocking=True)
        plan["ext_len"], plan["ext_start"] = fb.ext_len[tab[3]].contiguous(), fb.ext_start[tab[3]].contiguous()
        in_b = torch.zeros(bs, dtype=torch.bool, device=dev)
        in_b[tab[3]] = True
        plan["tok_mask"] = in_b[fb.tok_b.long()]
        plan["rest"] = dict(bs=len(A), tokens=sum(ext[b] for b in A), max_seq=max(pre[b] + ext[b] for b in A),
                            ext_len=fb.ext_len[idx_a].contiguous(), ext_start=fb.ext_start[idx_a].contiguous(),
                            req_pool=fb.req_pool_indices[idx_a].contiguous())
        return plan

    def _forward_expanded(self, q3: torch.Tensor, cache: torch.Tensor, plan, fb) -> torch.Tensor:
        lib = _lib.load()
        t, H, D, R, N = q3.shape[0], self.heads, self.expand_dim, self.kv_rank, plan["N"]
        code = _lib.dtype_code(q3.dtype)
        c_g = torch.empty((N, R), dtype=q3.dtype, device=q3.device)
        q_x = torch.empty((t, H, D), dtype=q3.dtype, device=q3.device)
        rc = lib.b200_latent_expand_gather(
            cache.data_ptr(), cache.stride(0), plan["slots"].data_ptr(), N, R, c_g.data_ptr(), c_g.stride(0),
            q3.data_ptr(), q3.stride(0), q3.stride(1), H, self.dim, self.rot_dim, self.rotary.dims,
            _lib.ptr(self.rotary.inv_freq), fb.tok_pos.data_ptr(), q_x.data_ptr(), D, t, code,
            _lib.current_stream())
        _lib.check(rc, "b200_latent_expand_gather")
        kv = torch.matmul(c_g, self._expand_weight().t())                          # [N, 2 * H * D]
        rc = lib.b200_latent_expand_rotkeys(
            cache.data_ptr(), cache.stride(0), plan["slots"].data_ptr(), N, R, self.rot_dim,
            kv.data_ptr(), kv.stride(0), H, D, self.dim, code, _lib.current_stream())
        _lib.check(rc, "b200_latent_expand_rotkeys")
        o_x = (torch.empty if plan["rest"] is None else torch.zeros)((t, H, D), dtype=q3.dtype, device=q3.device)
        esz = kv.element_size()
        rc = lib.b200_attn_extend_window(
            q_x.data_ptr(), H * D, kv.data_ptr(), kv.data_ptr() + H * D * esz, kv.stride(0),
            o_x.data_ptr(), H * D, plan["rtt"].data_ptr(), plan["rtt"].stride(0), plan["rows"].data_ptr(),
            plan["seq"].data_ptr(), plan["prefix"].data_ptr(), plan["ext_len"].data_ptr(),
            plan["ext_start"].data_ptr(), plan["bs"], plan["max_ext"], H, H, D, D, self.scale, 0.0, 1.0, 1,
            self.window, code, _lib.current_stream())
        _lib.check(rc, "b200_attn_extend_window")
        return o_x[:, :, :self.vdim]                                               # [t, H, vdim], strided

    def forward(self, h: torch.Tensor, forward_batch) -> torch.Tensor:
        fb = forward_batch
        t = h.shape[0]
        lib = _lib.load()
        code = _lib.dtype_code(h.dtype)
        pool = fb.token_to_kv_pool
        cache = pool.get_kv_buffer(self.layer_id)
        raw, _ = self.down_proj(h)
        direct = self.q_up_proj is None
        cq = None if direct else torch.empty((t, self.q_rank), dtype=h.dtype, device=h.device)
        kv_raw = raw[:, self.q_part:] if self.owns_kv else None
        inv_freq = self.rotary.inv_freq
        rc = lib.b200_latent_prep_scaled(
            None if direct else raw.data_ptr(), raw.stride(0), 0 if direct else self.q_rank,
            _lib.ptr(self.q_norm_weight), _lib.ptr(cq), cq.stride(0) if cq is not None else 0,
            _lib.ptr(kv_raw), raw.stride(0), self.kv_rank, self.rot_dim, self.rotary.dims,
            self.kv_norm_weight.data_ptr(), _lib.ptr(inv_freq), fb.tok_pos.data_ptr(),
            fb.out_cache_loc.data_ptr(), cache.data_ptr(), cache.stride(0), float(self.eps), self.rot_scale, t,
            code, _lib.current_stream())
        _lib.check(rc, "b200_latent_prep")
        if direct:
            q = raw[:, :self.q_part]
        else:
            q, _ = self.q_up_proj(cq)
        q3 = q.view(t, self.heads, self.dim + self.rot_dim)
        plan = self._expand_plan(fb) if h.dtype != torch.float32 else False
        if plan and plan["rest"] is None:
            heads3 = self._forward_expanded(q3, cache, plan, fb)
        else:
            heads3 = self._forward_absorbed(q, q3, cache, fb, plan["rest"] if plan else None)
            if plan:                  # a divided step: long portions expanded, the rest absorbed
                heads3 = torch.where(plan["tok_mask"][:, None, None], self._forward_expanded(q3, cache, plan, fb),
                                     heads3)
        # heads3: [t, H, vdim] in either memory order; gate and lay out token-major in one pass
        if self.gate:
            z = raw[:, self.q_part + self.kv_part:]
            heads_out = torch.empty((t, self.heads * self.vdim), dtype=h.dtype, device=h.device)
            rc = lib.b200_sigmoid_gate_mul(heads3.data_ptr(), heads3.stride(0), heads3.stride(1), z.data_ptr(),
                                           z.stride(0), 0, heads_out.data_ptr(), heads_out.stride(0), t,
                                           self.heads, self.vdim, code, _lib.current_stream())
            _lib.check(rc, "b200_sigmoid_gate_mul")
        else:
            heads_out = heads3.reshape(t, self.heads * self.vdim)
        out, _ = self.o_proj(heads_out)
        return out

    def _forward_absorbed(self, q: torch.Tensor, q3: torch.Tensor, cache: torch.Tensor, fb, rest) -> torch.Tensor:
        """-> [T, H, vdim] (a view of the head-major product).  `rest`: the batch entries to run (None:
        all); rows of other entries are left for the caller to fill."""
        lib = _lib.load()
        h, t, inv_freq = q, q.shape[0], self.rotary.inv_freq
        code = _lib.dtype_code(q.dtype)
        q_lat = _bmm_f32(q3[:, :, :self.dim].transpose(0, 1), self.w_uk)           # [H, T, R] fp32
        o_lat = (torch.empty if rest is None else torch.zeros)((self.heads, t, self.kv_rank), dtype=h.dtype,
                                                               device=h.device)
        max_seq = int(fb.max_seq_len) if rest is None else rest["max_seq"]
        ext_start, ext_len = (fb.ext_start, fb.ext_len) if rest is None else (rest["ext_start"], rest["ext_len"])
        req_pool, bs = (fb.req_pool_indices, fb.batch_size) if rest is None else (rest["req_pool"], rest["bs"])
        # few tokens with many keys each (decoding): spread every token's keys over several CTAs
        keys = min(self.window, max_seq) if self.window else max_seq
        ctas = (t if rest is None else rest["tokens"]) * ((self.heads + 63) // 64)
        splits = 1
        if h.dtype != torch.float32 and ctas < _SM_COUNT and keys > 128:
            splits = max(1, min((keys + 63) // 64, (2 * _SM_COUNT) // ctas, 64))
        ws = ((torch.empty if rest is None else torch.zeros)(
            splits * t * self.heads * (self.kv_rank + 2), dtype=torch.float32, device=h.device)
            if splits > 1 else None)
        rc = lib.b200_latent_attn(
            q_lat.data_ptr(), q_lat.stride(1), q_lat.stride(0), q.data_ptr(), q3.stride(0), q3.stride(1),
            self.dim, cache.data_ptr(), cache.stride(0), fb.req_to_token_pool.req_to_token.data_ptr(),
            fb.req_to_token_pool.req_to_token.stride(0), req_pool.data_ptr(),
            fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), ext_start.data_ptr(), ext_len.data_ptr(),
            bs, _lib.ptr(inv_freq), self.rotary.dims, t,
            self.heads, self.kv_rank, self.rot_dim, self.window, max_seq, self.scale,
            o_lat.data_ptr(), o_lat.stride(1), o_lat.stride(0), splits, _lib.ptr(ws),
            ws.numel() if ws is not None else 0, code, _lib.current_stream())
        _lib.check(rc, "b200_latent_attn")
        return torch.bmm(o_lat, self.w_uv_t).transpose(0, 1)                       # [H, T, vdim] -> [T, H, vdim]
