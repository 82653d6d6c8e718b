"""Kisilix mechanisms one by one on the GPU against the plain float64 restatement: the layer norm after
the residual sum, the clamped gated activation, the gate-before-norm group norm, the short convolution
with its carried inputs, both recurrences (portions down to one token, bit-identical to token by token,
reused state rows), the grouped softmax router, and the attention over window + pooled blocks with a key
that stands out placed at every edge."""
import math
from types import SimpleNamespace

import pytest
import torch

import kisilix_plain as P
import kisilix_util as U
from sglang_security_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"
F64 = torch.float64


def _gen(seed):
    return torch.Generator().manual_seed(seed)


# ---- row kernels ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width, top", [(48, 3), (27, 1), (1031, 2)])
def test_layer_norm_after_the_sum(dtype, width, top):
    from sglang_security_b200.layers.residual_norm import PostSumLayerNorm

    g, t = _gen(1), 9
    norm = PostSumLayerNorm(width, 1e-5, alpha=2.5).to(DEV)
    norm.weight.data.copy_(1 + 0.3 * torch.randn(width, generator=g))
    norm.bias.data.copy_(0.3 * torch.randn(width, generator=g))
    x = torch.randn(t, width, generator=g)
    a, b = torch.randn(t, width, generator=g).to(dtype), torch.randn(t, width, generator=g).to(dtype)
    rows = torch.randn(t * top, width, generator=g).to(dtype)
    wts = torch.rand(t, top, generator=g)
    want = P.layer_norm(2.5 * x.double() + a.double() + b.double()
                        + (wts.double().unsqueeze(-1) * rows.double().view(t, top, width)).sum(1),
                        norm.weight.double().cpu(), norm.bias.double().cpu(), 1e-5)
    xd = x.to(DEV)
    h = norm(xd, a=a.to(DEV), b=b.to(DEV), rows=rows.to(DEV), row_weights=wts.to(DEV), out_dtype=dtype)
    assert (xd.double().cpu() - want).abs().max() < 2e-5
    assert (h.double().cpu() - want).abs().max() < (2e-5 if dtype == torch.float32 else 3e-2)
    # one term only, and the plain norm that leaves the residual alone
    x2 = x.to(DEV)
    norm(x2, a=a.to(DEV))
    assert (x2.double().cpu() - P.layer_norm(2.5 * x.double() + a.double(), norm.weight.double().cpu(),
                                             norm.bias.double().cpu(), 1e-5)).abs().max() < 2e-5
    x3 = x.to(DEV)
    y = norm(x3, out_dtype=torch.float32, in_place=False)
    assert torch.equal(x3.cpu(), x)
    assert (y.double().cpu() - P.layer_norm(x.double(), norm.weight.double().cpu(), norm.bias.double().cpu(),
                                            1e-5)).abs().max() < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gated_activation(dtype):
    from sglang_security_b200.layers.activation import ClampedGluAndMul

    z = (3 * torch.randn(7, 2 * 37, generator=_gen(2))).to(dtype)
    got = ClampedGluAndMul(1.25)(z.to(DEV)).double().cpu()
    g = torch.clamp(z[:, :37].double(), max=1.25)
    u = torch.clamp(z[:, 37:].double(), -1.25, 1.25)
    want = g * torch.sigmoid(1.702 * g) * (u + 1)
    assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2)
    assert (g < -1.25).any() and (z[:, :37] > 1.25).any()      # the gate is clamped from above only


@pytest.mark.parametrize("parts", [1, 3])
def test_group_norm_with_the_gate_before_it(parts):
    from sglang_security_b200.layers.recurrent.linear_recurrence import gated_group_rmsnorm

    g, n = _gen(3), 3 * 14
    o, z, w = torch.randn(5, n, generator=g), torch.randn(5, n, generator=g), 1 + 0.2 * torch.randn(n, generator=g)
    got = gated_group_rmsnorm(o.to(DEV), w.to(DEV), z.to(DEV), n // parts, 1e-5, torch.float32, gate="silu_before")
    y = o.double() * P.silu(z.double())
    want = P.rms_div(y.view(5, parts, n // parts), 1e-5).reshape(5, n) * w.double()
    assert (got.double().cpu() - want).abs().max() < 1e-5
    other = gated_group_rmsnorm(o.to(DEV), w.to(DEV), z.to(DEV), n // parts, 1e-5, torch.float32)
    assert (other.double().cpu() - want).abs().max() > 1e-2    # the gate's place matters


# ---- short convolution -----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps, bias", [(1, False), (2, True), (4, False), (7, True)])
def test_short_convolution_carries_its_inputs(dtype, taps, bias):
    from sglang_security_b200.layers.recurrent.delta_recurrence import causal_conv_silu

    g, C = _gen(4), 300
    w = (0.6 * torch.randn(C, taps, generator=g))
    bv = 0.3 * torch.randn(C, generator=g) if bias else None
    seqs = {0: torch.randn(41, C + 5, generator=g).to(dtype), 1: torch.randn(23, C + 5, generator=g).to(dtype),
            2: torch.randn(9, C + 5, generator=g).to(dtype)}
    state = torch.full((3, (taps - 1) * C + 11), 7.0, device=DEV)       # stale values everywhere
    hb = U.HandBatch(3, 64)
    got = {r: [] for r in seqs}
    at = {r: 0 for r in seqs}
    sizes, step = [1, 3, 2, 1, 10, 5], 0
    while any(at[r] < len(seqs[r]) for r in seqs):
        entries = [(r, min(sizes[(step + r) % len(sizes)], len(seqs[r]) - at[r])) for r in seqs if at[r] < len(seqs[r])]
        fb = hb.step(entries)
        x = torch.cat([seqs[r][at[r]:at[r] + n] for r, n in entries]).to(DEV)
        y = causal_conv_silu(x[:, 2:2 + C], w.to(DEV), bv.to(DEV) if bias else None, state[:, 3:], fb)
        o = 0
        for r, n in entries:
            got[r].append(y[o:o + n].double().cpu())
            o += n
            at[r] += n
        step += 1
    tol = 1e-5 if dtype == torch.float32 else 8e-3          # relative: the output is rounded to 16 bits
    for r, s in seqs.items():
        want = P.causal_conv_silu(s[:, 2:2 + C].double(), w.double(), bv.double() if bias else None)
        assert ((torch.cat(got[r]) - want).abs() / (1 + want.abs())).max() < tol, r
    # a row that is used again: the new sequence starts from zeros, whatever the row holds
    hb.release(1)
    s = torch.randn(6, C + 5, generator=g).to(dtype)
    y = causal_conv_silu(s.to(DEV)[:, 2:2 + C], w.to(DEV), bv.to(DEV) if bias else None, state[:, 3:], hb.step([(1, 6)]))
    want = P.causal_conv_silu(s[:, 2:2 + C].double(), w.double(), bv.double() if bias else None)
    assert ((y.double().cpu() - want).abs() / (1 + want.abs())).max() < tol


# ---- recurrences -----------------------------------------------------------------------------------
GEOMETRIES = [(4, 2, 16, 24), (3, 3, 10, 6), (1, 1, 40, 70), (2, 1, 72, 33), (2, 2, 130, 8), (2, 1, 1, 1)]


def _run_recurrence(mode, H, G, D, E, dtype, lens, sizes, seed, state=None, hb=None, rows=None):
    """Feeds sequences (one per state row) in portions -> ({row: fp32 output}, {row: oracle}, state, hb)."""
    from sglang_security_b200.layers.recurrent.delta_recurrence import delta_recurrence

    g = _gen(seed)
    rows = rows or list(range(len(lens)))
    nd = H * D if mode == "delta" else H
    bias, a_log = torch.randn(nd, generator=g) - 1.0, 0.7 * torch.randn(H, generator=g) - 0.5
    skip = torch.randn(H, generator=g)
    seqs = {}
    for r, n in zip(rows, lens):
        seqs[r] = dict(q=torch.randn(n, G * D, generator=g).to(dtype), k=torch.randn(n, G * D, generator=g).to(dtype),
                       v=torch.randn(n, H * E, generator=g).to(dtype),
                       d=(1.5 * torch.randn(n, nd, generator=g)).to(dtype),
                       b=(1.5 * torch.randn(n, H, generator=g)).to(dtype))
    if state is None:
        state = torch.full((max(rows) + 2, H * D * E + 5), 3.0, device=DEV)     # stale values
        hb = U.HandBatch(max(rows) + 2, 512)
    got, at, step = {r: [] for r in rows}, {r: 0 for r in rows}, 0
    while any(at[r] < len(seqs[r]["q"]) for r in rows):
        entries = [(r, min(sizes[(step + r) % len(sizes)], len(seqs[r]["q"]) - at[r])) for r in rows
                   if at[r] < len(seqs[r]["q"])]
        fb = hb.step(entries)
        cat = {n: torch.cat([seqs[r][n][at[r]:at[r] + c] for r, c in entries]).to(DEV) for n in "qkvdb"}
        if mode == "delta":
            o = delta_recurrence(cat["q"], cat["k"], cat["v"], cat["d"], bias.to(DEV), a_log.to(DEV), H, G, D, E,
                                 state[:, 2:], fb, beta_raw=cat["b"], q_scale=D ** -0.5)
        else:
            o = delta_recurrence(cat["q"], cat["k"], cat["v"], cat["d"], bias.to(DEV), a_log.to(DEV), H, G, D, E,
                                 state[:, 2:], fb, skip=skip.to(DEV))
        i = 0
        for r, c in entries:
            got[r].append(o[i:i + c].cpu())
            i += c
            at[r] += c
        step += 1
    want = {}
    for r in rows:
        s = {n: t.double() for n, t in seqs[r].items()}
        n = len(s["q"])
        q, k, v = s["q"].view(n, G, D), s["k"].view(n, G, D), s["v"].view(n, H, E)
        if mode == "delta":
            gdec = torch.exp(-torch.exp(a_log.double()).view(1, H, 1) * P.softplus(s["d"] + bias.double()).view(n, H, D))
            want[r] = P.delta_rule_scan(P.unit(q) * D ** -0.5, P.unit(k), v, gdec, torch.sigmoid(s["b"])).reshape(n, H * E)
        else:
            dt = P.softplus(s["d"] + bias.double())
            want[r] = P.state_space_scan(q, k, v, torch.exp(-torch.exp(a_log.double()) * dt), dt, skip.double()).reshape(n, H * E)
    return {r: torch.cat(got[r]) for r in rows}, want, state, hb


@pytest.mark.parametrize("mode", ["delta", "ssm"])
@pytest.mark.parametrize("H, G, D, E", GEOMETRIES)
def test_recurrence_in_portions_matches_and_equals_token_by_token(mode, H, G, D, E):
    lens = [45, 19, 70]
    got, want, _, _ = _run_recurrence(mode, H, G, D, E, torch.float32, lens, [1, 3, 17, 2, 1, 40], seed=5)
    for r in got:
        scale = want[r].abs().max().clamp_min(1e-6)
        assert (got[r].double() - want[r]).abs().max() / scale < 2e-5, (r, mode)
    one, _, _, _ = _run_recurrence(mode, H, G, D, E, torch.float32, lens, [1], seed=5)
    whole, _, _, _ = _run_recurrence(mode, H, G, D, E, torch.float32, lens, [100], seed=5)
    for r in got:                      # the cut of a sequence changes no bit
        assert torch.equal(got[r], one[r]) and torch.equal(got[r], whole[r])


@pytest.mark.parametrize("mode", ["delta", "ssm"])
def test_recurrence_16_bit_inputs_long_decoding_and_a_reused_row(mode):
    H, G, D, E = 4, 2, 24, 40
    got, want, state, hb = _run_recurrence(mode, H, G, D, E, torch.bfloat16, [330], [20, 1], seed=6)
    assert (got[0].double() - want[0]).abs().max() / want[0].abs().max() < 2e-5     # inputs are exact in both
    hb.release(0)
    got, want, _, _ = _run_recurrence(mode, H, G, D, E, torch.bfloat16, [12], [5], seed=7, state=state, hb=hb, rows=[0])
    assert (got[0].double() - want[0]).abs().max() / want[0].abs().max() < 2e-5


@pytest.mark.parametrize("mode", ["delta", "ssm"])
def test_recurrence_of_many_sequences_on_wider_ctas(mode):
    """Enough (sequence, head) pairs that the launch takes its two-warp CTAs: same bits as a sequence alone."""
    H, G, D, E, n = 4, 2, 16, 24, 90
    got, want, _, _ = _run_recurrence(mode, H, G, D, E, torch.float32, [7] * n, [4, 1], seed=12)
    alone, _, _, _ = _run_recurrence(mode, H, G, D, E, torch.float32, [7], [7], seed=12)
    assert torch.equal(got[0], alone[0])
    for r in (0, 41, n - 1):
        assert (got[r].double() - want[r]).abs().max() / want[r].abs().max() < 2e-5


def test_delta_rule_overwrites_a_key():
    """One head, decay 1, write strength 1: writing value b under a key that held a replaces a (the delta
    rule's defining property), which a plain additive memory would not do."""
    from sglang_security_b200.layers.recurrent.delta_recurrence import delta_recurrence

    D, E = 8, 4
    k = torch.zeros(2, D)
    k[:, 3] = 5.0
    v = torch.tensor([[1., 2., 3., 4.], [-4., 0., 9., 1.]])
    hb = U.HandBatch(1, 16)
    o = delta_recurrence(k.to(DEV), k.to(DEV), v.to(DEV), torch.full((2, D), -40.0, device=DEV),
                         torch.zeros(D, device=DEV), torch.zeros(1, device=DEV), 1, 1, D, E,
                         torch.zeros(1, D * E, device=DEV), hb.step([(0, 2)]),
                         beta_raw=torch.full((2, 1), 40.0, device=DEV), q_scale=1.0, unit_eps=0.0)
    assert (o.cpu() - v).abs().max() < 1e-5


# ---- router ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, top, groups, keep", [(8, 2, 4, 2), (6, 6, 1, 1), (33, 3, 1, 1), (40, 5, 8, 3),
                                                   (9, 1, 9, 1), (64, 8, 4, 4)])
def test_grouped_softmax_router(dtype, n, top, groups, keep):
    from sglang_security_b200.layers.moe.fused_moe import GroupedSoftmaxRouter

    g, width, t = _gen(8), 56, 150
    r = GroupedSoftmaxRouter(width, n, top, groups, keep).to(DEV)
    r.weight.data.copy_(torch.randn(n, width, generator=g) * 0.5)
    r.correction.data.copy_(torch.randn(n, generator=g) * 0.2 - 0.1)
    h = torch.randn(t, width, generator=g).to(dtype)
    ids, wts = r(h.to(DEV))
    W = {"router": r.weight.double().cpu(), "correction": r.correction.double().cpu()}
    spec = {"experts": n, "top": top, "groups": {"count": groups, "keep": keep}}
    want_ids, want_w = P.route(h.double(), W, "", spec)
    same = 0
    for i in range(t):
        a, b = dict(zip(ids[i].tolist(), wts[i].tolist())), dict(zip(want_ids[i].tolist(), want_w[i].tolist()))
        if set(a) == set(b):
            same += 1
            assert max(abs(a[e] - b[e]) for e in a) < 1e-5
        assert abs(sum(a.values()) - 1.0) < 1e-5 and len(a) == top
    assert same >= t - 2            # a near-tie may fall either way


# ---- attention over a window and pooled blocks --------------------------------------------------------
def _attention_batch(H, G, D, E, window, pool, page, seqs, sizes, dtype, scale=1.0, head_scale=None, seed=0):
    """seqs: {row: (q [n, H, D], k [n, G, D], v [n, G, E])} already normed / rotated.  Writes the rows into a
    paged pool in ragged steps, forms the block means and attends; -> {row: [n, H * E]}."""
    lib, st = _lib.load(), _lib.current_stream()
    code = _lib.dtype_code(dtype)
    hb = U.HandBatch(max(seqs) + 1, 512, page=page, seed=seed)
    width = G * (D + E)
    kv = torch.full((hb.pool_rows, width), 9.0, dtype=dtype, device=DEV)          # stale values
    pdiv = pool if pool and page % pool == 0 else 1
    summary = torch.full((hb.pool_rows // pdiv + 1, width), 9.0, device=DEV) if pool else None
    got, at, step = {r: [] for r in seqs}, {r: 0 for r in seqs}, 0
    while any(at[r] < len(seqs[r][0]) for r in seqs):
        entries = [(r, min(sizes[(step + r) % len(sizes)], len(seqs[r][0]) - at[r])) for r in seqs
                   if at[r] < len(seqs[r][0])]
        fb = hb.step(entries)
        q = torch.cat([seqs[r][0][at[r]:at[r] + c].reshape(c, H * D) for r, c in entries]).float().to(DEV)
        if head_scale is not None:
            q = q * head_scale.to(DEV).repeat_interleave(D)
        rows = torch.cat([torch.cat([seqs[r][1][at[r]:at[r] + c].reshape(c, G * D),
                                     seqs[r][2][at[r]:at[r] + c].reshape(c, G * E)], 1) for r, c in entries])
        kv[fb.out_cache_loc] = rows.to(dtype).to(DEV)
        r2t = fb.req_to_token
        if pool:
            rc = lib.b200_pool_block_means(kv.data_ptr(), kv.stride(0), width, summary.data_ptr(), summary.stride(0),
                                           pool, pdiv, r2t.data_ptr(), r2t.stride(0), fb.req_pool_indices.data_ptr(),
                                           fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), fb.total, code, st)
            _lib.check(rc, "pool_block_means")
        out = torch.empty((fb.total, H * E), dtype=dtype, device=DEV)
        rc = lib.b200_pooled_window_attn(
            q.data_ptr(), q.stride(0), kv.data_ptr(), kv.stride(0), 0, G * D, _lib.ptr(summary),
            summary.stride(0) if pool else 0, pool, pdiv, r2t.data_ptr(), r2t.stride(0),
            fb.req_pool_indices.data_ptr(), fb.tok_pos.data_ptr(), fb.tok_b.data_ptr(), scale, window, None, None, 1,
            out.data_ptr(), out.stride(0), fb.total, H, G, D, E, None, max(hb.lens), code, st)
        _lib.check(rc, "pooled_window_attn")
        i = 0
        for r, c in entries:
            got[r].append(out[i:i + c].double().cpu())
            i += c
            at[r] += c
        step += 1
    return {r: torch.cat(got[r]) for r in seqs}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, D, E, window, pool, page", [
    (4, 2, 16, 24, 20, 4, 16), (3, 1, 6, 10, 7, 7, 16), (2, 2, 24, 8, 33, 5, 16), (6, 1, 64, 64, 40, 8, 64),
    (1, 1, 8, 130, 1, 1, 16), (2, 1, 12, 4, 50, 0, 16), (2, 2, 16, 16, 0, 0, 16), (5, 5, 40, 36, 9, 3, 32)])
def test_attention_over_window_and_blocks(dtype, H, G, D, E, window, pool, page):
    g = _gen(9)
    seqs = {}
    for r, n in enumerate([150, 61, 23]):
        mk = lambda *s: torch.randn(*s, generator=g).to(dtype)
        seqs[r] = (mk(n, H, D), mk(n, G, D), mk(n, G, E))
    hs = 1 + 0.4 * torch.randn(H, generator=g)
    got = _attention_batch(H, G, D, E, window, pool, page, seqs, [150, 1, 2, 33, 1, 7], dtype, scale=0.9 / D ** 0.5,
                           head_scale=hs)
    for r, (q, k, v) in seqs.items():
        want = P.attend(q.double(), k.double(), v.double(), window, pool, 0.9 / D ** 0.5 * hs.double())
        err = (got[r] - want.reshape(len(q), H * E)).abs().max()
        assert err < (2e-5 if dtype == torch.float32 else 2e-2), r


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window, pool, page", [(24, 4, 16), (10, 5, 16), (16, 16, 64), (30, 0, 16)])
def test_a_key_that_stands_out_at_every_edge(window, pool, page, decode):
    """All keys are small but one, which matches the queries exactly and carries a value of its own.  The
    last position's output then tells whether that key is seen as a token (its value alone), through its
    block's mean (the block's average value), or not at all; it is placed right inside and outside the
    window, at both ends of a block, at page borders, at position 0 and far back."""
    H, G, D, E, n = 2, 1, 16, 8, 140
    g = _gen(10)
    last = n - 1
    spots = {0, 1, last, last - 1, last - window + 1, last - window, last - window - 1, page - 1, page, 2 * page - 1, 5}
    if pool:
        done = (last - window + 1) // pool          # blocks wholly before the window
        spots |= {done * pool - 1, done * pool, done * pool - pool, done * pool + pool - 1, pool - 1, pool}
    for j in sorted(s for s in spots if 0 <= s <= last):
        k = 0.05 * torch.randn(n, G, D, generator=g)
        v = torch.randn(n, G, E, generator=g)
        q = torch.zeros(n, H, D)
        q[:, :, 2] = 6.0
        k[j, 0, 2] = 6.0
        v[j] = 10.0 + torch.arange(E)
        sizes = [n - 20, 1] if decode else [57, 2, 64]
        got = _attention_batch(H, G, D, E, window, pool, page, {0: (q, k, v)}, sizes, torch.float32, scale=1.0)[0]
        want = P.attend(q.double(), k.double(), v.double(), window, pool, torch.ones(H, dtype=F64)).reshape(n, H * E)
        assert (got - want).abs().max() < 1e-4, j
        # the oracle itself tells the three cases apart
        toks, blocks = P.visible(last, window, pool)
        peak = want[last, :E]
        if j in toks:
            assert (peak - v[j, 0].double()).abs().max() < 1e-2, j
        elif pool and j // pool in blocks:
            assert (peak - v[j, 0].double()).abs().max() > 1.0, j
            if pool <= 5:                      # the block's mean key still wins the softmax
                assert abs(float(peak[0]) - 10.0 / pool) < 1.2, j
        else:
            assert float(peak.abs().max()) < 5.0, j


def _to_neighbours(n, dims):
    """Order that puts coordinate i and i + dims/2 of the half pairing side by side."""
    return [x for i in range(dims // 2) for x in (i, i + dims // 2)] + list(range(dims, n))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing", ["half", "neighbour"])
def test_attention_layer_with_norms_rotations_and_rotated_values(dtype, pairing):
    """The whole mixer (fused projection, head norms, rotation of q, k and of the values, block means,
    attention, counter-rotation, W_o) through a real pool, in ragged portions of two sequences, one of
    them at positions beyond 1200; the same tokens at other positions must give another output (the value
    rotation is relative only together with the counter-rotation).  The neighbour pairing is run on
    weights whose coordinates are reordered so that it must give the half pairing's result."""
    from sglang_security_b200.layers.attention.pooled_window_attention import PooledWindowAttention
    from sglang_security_b200.mem_cache.latent_pool import LatentTokenToKVPool

    g, W_, H, G, D, E, R = _gen(11), 40, 4, 2, 12, 10, 8
    att = PooledWindowAttention(W_, H, G, D, E, 0.3, 0, 1e-5, window=19, pool=4, rope_base=300.0, rope_dims=R,
                                pairing=pairing, params_dtype=dtype).to(DEV)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": E, "scale": 0.3, "mask": {"size": 19, "pool": 4},
         "rot": {"base": 300.0, "dims": R}}
    w = {k: v for k, v in U.random_weights(U.config([(U.attn(H, G, D, E, 19, 4, R, 300.0, 0.3), None)], width=W_), 3).items()
         if k.startswith("l0.mix.")}
    pk = torch.tensor(_to_neighbours(D, R) if pairing == "neighbour" else list(range(D)))
    pv = torch.tensor(_to_neighbours(E, E) if pairing == "neighbour" else list(range(E)))
    heads = {"q": (H, D, pk), "k": (G, D, pk), "v": (G, E, pv)}
    for n, (cnt, size, perm) in heads.items():
        rows = (torch.arange(cnt).view(-1, 1) * size + perm.view(1, -1)).reshape(-1)
        att.load_part(n, w[f"l0.mix.{n}"][rows].to(DEV))
        att.load_part(n, w[f"l0.mix.{n}.b"][rows].to(DEV), is_bias=True)
    att.q_norm_weight.data.copy_(w["l0.mix.q.norm"].float()[pk])
    att.k_norm_weight.data.copy_(w["l0.mix.k.norm"].float()[pk])
    att.head_scale.data.copy_(w["l0.mix.temp"].float())
    att.o_proj.weight.data.copy_(w["l0.mix.o"][:, (torch.arange(H).view(-1, 1) * E + pv.view(1, -1)).reshape(-1)])
    page, slots, ctx, far = 16, 2, 1300, 1200
    pool = LatentTokenToKVPool(slots * ctx, page, dtype, {0: att.row_width}, {}, DEV, block_summaries={0: 4})
    hb = U.HandBatch(slots, ctx, page=page)
    hs = {0: torch.randn(90, W_, generator=g).to(dtype), 1: torch.randn(37, W_, generator=g).to(dtype)}
    # sequence 1 is fed zero inputs up to position `far` in big portions, then its tokens
    full = {0: hs[0], 1: torch.cat([torch.zeros(far, W_, dtype=dtype), hs[1]])}
    outs, at, step, sizes = {0: [], 1: []}, {0: 0, 1: 0}, 0, [31, 1, 2, 9]
    while any(at[r] < len(full[r]) for r in full):
        entries = []
        for r in full:
            if at[r] < len(full[r]):
                c = sizes[(step + r) % len(sizes)] if (r == 0 or at[r] >= far) else min(600, far - at[r])
                entries.append((r, min(c, len(full[r]) - at[r])))
        t = hb.step(entries)
        fb = SimpleNamespace(token_to_kv_pool=pool, req_to_token_pool=SimpleNamespace(req_to_token=t.req_to_token),
                             out_cache_loc=t.out_cache_loc, tok_pos=t.tok_pos, tok_b=t.tok_b,
                             req_pool_indices=t.req_pool_indices, max_seq_len=max(hb.lens), batch_size=len(entries))
        y = att(torch.cat([full[r][at[r]:at[r] + c] for r, c in entries]).to(DEV), fb)
        i = 0
        for r, c in entries:
            outs[r].append(y[i:i + c].double().cpu())
            i += c
            at[r] += c
        step += 1
    Wd = {k: v.double() for k, v in w.items()}
    tol = 2e-4 if dtype == torch.float32 else 5e-2
    first = {0: 0, 1: far}
    for r in full:
        want = P.attention(full[r].double(), Wd, "l0.mix.", m, 1e-5)
        assert (torch.cat(outs[r]) - want)[first[r]:].abs().max() < tol * want.abs().max(), r
    moved = P.attention(hs[1].double(), Wd, "l0.mix.", m, 1e-5)            # the same tokens from position 0
    assert (moved - torch.cat(outs[1])[far:]).abs().max() > 0.05 * moved.abs().max()
