"""The mechanisms the Kulesun design adds, one at a time: the row kernels against fp64 torch, and each
option of the two mixers alone in a one-layer model whose other options are neutralised by its weights
(identity head mix, zero gate weights, no cap, no temperature), against the plain restatement."""
import math

import pytest
import torch

import kulesun_plain as P
import kulesun_util as U

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _err(got, want):
    return float((got.double().cpu() - want.double().cpu()).abs().max() / want.double().abs().max().clamp_min(1e-9))


# ---- row kernels ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 27, 1024])
def test_add_normed_emits_the_next_prenorm(dtype, width):
    from sglang_security_b200.layers.residual_norm import AddNormed

    g = torch.Generator().manual_seed(width)
    T = 9
    x = torch.randn(T, width, generator=g)
    y = (3.0 * torch.randn(T, width, generator=g)).to(dtype)
    wb, wn = 1 + 0.3 * torch.randn(width, generator=g), 1 + 0.3 * torch.randn(width, generator=g)
    layer = AddNormed(width, 1e-5).to(DEV)
    layer.weight.data.copy_(wb)
    xd = x.to(DEV)
    h = layer(xd, a=y.to(DEV), out_dtype=dtype, next_weight=wn.to(DEV))
    want_x = x.double() + P.unit_rms(y.double(), 1e-5) * wb.double()
    want_h = P.unit_rms(want_x, 1e-5) * wn.double()
    assert _err(xd, want_x) <= 2e-6
    assert h.dtype == dtype and _err(h, want_h) <= (2e-6 if dtype == torch.float32 else 6e-3)
    # without a next weight the copy is the residual itself
    xd2 = x.to(DEV)
    h2 = layer(xd2, a=y.to(DEV), out_dtype=dtype)
    assert _err(h2, want_x) <= (2e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype,planes_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                                (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("H,G,E", [(6, 2, 24), (3, 3, 5), (8, 1, 64), (96, 4, 8)])
def test_head_mix_and_gate(dtype, planes_dtype, H, G, E):
    from sglang_security_b200 import _lib

    g = torch.Generator().manual_seed(H * E)
    T = 7
    planes = torch.randn(G, T, H * E, generator=g).to(planes_dtype)
    mix = torch.randn(H, H, generator=g)
    z = torch.randn(T, H + 3, generator=g).to(dtype)                  # a wider row: the gate is a slice
    out = torch.empty((T, H * E), dtype=dtype, device=DEV)
    pd, md, zd = planes.to(DEV), mix.to(DEV), z.to(DEV)
    for gate in (zd, None):
        rc = _lib.load().b200_head_mix_gate(pd.data_ptr(), pd.stride(1), pd.stride(0), _lib.dtype_code(planes_dtype),
                                            md.data_ptr(), _lib.ptr(gate), zd.stride(0), out.data_ptr(),
                                            out.stride(0), T, H, G, E, _lib.dtype_code(dtype), 0)
        _lib.check(rc, "head_mix_gate")
        a = planes.double().view(G, T, H, E)
        want = torch.stack([sum(mix[h, j].double() * a[h // (H // G), :, j] for j in range(H)) for h in range(H)], 1)
        if gate is not None:
            want = want * torch.sigmoid(z[:, :H].double())[:, :, None]
        assert _err(out.view(T, H, E), want) <= (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_head", [0, 1])
def test_sigmoid_gate_on_a_head_major_product(dtype, per_head):
    from sglang_security_b200 import _lib

    g = torch.Generator().manual_seed(5)
    T, H, E = 6, 5, 12
    x = torch.randn(H, T, E, generator=g).to(dtype).to(DEV)           # as a batched product leaves it
    z = torch.randn(T, H if per_head else H * E, generator=g).to(dtype).to(DEV)
    out = torch.empty((T, H * E), dtype=dtype, device=DEV)
    x3 = x.transpose(0, 1)
    rc = _lib.load().b200_sigmoid_gate_mul(x3.data_ptr(), x3.stride(0), x3.stride(1), z.data_ptr(), z.stride(0),
                                           per_head, out.data_ptr(), out.stride(0), T, H, E, _lib.dtype_code(dtype), 0)
    _lib.check(rc, "sigmoid_gate_mul")
    gate = torch.sigmoid(z.double().cpu())
    gate = gate[:, :, None] if per_head else gate.view(T, H, E)
    assert _err(out.view(T, H, E), x3.double().cpu() * gate) <= (1e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,E,every", [(4, 2, 16, 24, 7), (3, 3, 10, 5, 1), (2, 1, 8, 70, 64), (16, 8, 8, 8, 3)])
def test_prep_temperature_unit_values_and_value_mix(dtype, H, G, D, E, every):
    """Positions on both sides of every step of the temperature; values of unit RMS per head, then mixed
    with another pool's row of the same token."""
    from sglang_security_b200 import _lib

    g = torch.Generator().manual_seed(every)
    pos = sorted({0, 1, every - 2, every - 1, every, 2 * every - 2, 2 * every - 1, 2 * every, 9 * every - 1,
                  9 * every, 1000 * every - 1, 1000 * every} - {-1})
    T, coef, lam, eps = len(pos), 0.37, 0.3, 1e-3
    q, k, v = (torch.randn(T, n, generator=g).to(dtype) for n in (H * D, G * D, G * E))
    v = v * 5.0
    first = torch.randn(T + 1, 3 + G * E, generator=g).to(dtype)      # values behind 3 other columns
    pool = torch.zeros((T + 1, G * (D + E)), dtype=dtype, device=DEV)
    loc = torch.arange(1, T + 1, dtype=torch.int64, device=DEV)
    tok_pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
    q32 = torch.empty((T, H * D), dtype=torch.float32, device=DEV)
    qd, kd, vd, fd = q.to(DEV), k.to(DEV), v.to(DEV), first.to(DEV)
    lam_d = torch.tensor(lam, dtype=torch.float32, device=DEV)
    for mix in (False, True):
        rc = _lib.load().b200_qkv_prep_write(
            qd.data_ptr(), qd.stride(0), kd.data_ptr(), kd.stride(0), vd.data_ptr(), vd.stride(0), None, None, 0, 0,
            eps, None, None, 0, tok_pos.data_ptr(), loc.data_ptr(), pool.data_ptr(), pool.stride(0), 0, G * D,
            q32.data_ptr(), q32.stride(0), None, 0, T, H, G, D, E, coef, every, 1,
            lam_d.data_ptr() if mix else None, fd.data_ptr() if mix else None, fd.stride(0), 3,
            _lib.dtype_code(dtype), 0)
        _lib.check(rc, "prep")
        temp = P.query_temperature(torch.tensor(pos), coef, every)
        assert _err(q32, q.double() * temp[:, None]) <= 2e-6
        assert torch.equal(pool[1:, :G * D].cpu(), k)
        want_v = P.unit_rms(v.double().view(T, G, E), eps).view(T, G * E)
        if mix:
            want_v = (1 - lam) * want_v + lam * first[1:, 3:].double()
        assert _err(pool[1:, G * D:], want_v) <= (2e-6 if dtype == torch.float32 else 6e-3)
    assert P.query_temperature(torch.tensor([every - 2]), coef, every)[0] == 1.0 or every == 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,rot,factor", [(40, 8, 4.0), (16, 32, 8.0), (24, 6, None)])
def test_scaled_half_pairing_rotation_of_the_cached_key_part(dtype, R, rot, factor):
    """Rows reordered as a checkpoint in the half pairing is loaded, rotated as neighbours, multiplied by
    the squared amplitude: the same numbers as the half-pairing rotation of the plain model, reordered."""
    from sglang_security_b200 import _lib
    from sglang_security_b200.layers.rotary_embedding import PairedRotary, ramp_scaled_frequencies

    spec = {"dims": rot, "base": 5000.0}
    freqs, amp = None, 1.0
    if factor:
        spec["scaling"] = {"factor": factor, "original": 128, "fast": 8.0, "slow": 1.0}
        freqs, amp = ramp_scaled_frequencies(rot, 5000.0, factor, 128, 8.0, 1.0)
    rotary = PairedRotary(rot, 5000.0, pairing="half", frequencies=freqs, amplitude=amp).to(DEV)
    g = torch.Generator().manual_seed(R)
    pos = [0, 1, 2, 63, 64, 500, 4097]
    T = len(pos)
    raw = torch.randn(T, R + rot, generator=g).to(dtype)
    order = rotary.row_order(rot)
    fed = torch.cat([raw[:, :R], raw[:, R:][:, order]], 1).to(DEV).contiguous()
    wkv = (1 + 0.2 * torch.randn(R, generator=g)).to(DEV)
    cache = torch.zeros((T + 1, R + rot), dtype=dtype, device=DEV)
    loc = torch.arange(1, T + 1, dtype=torch.int64, device=DEV)
    tok_pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
    rc = _lib.load().b200_latent_prep_scaled(None, 0, 0, None, None, 0, fed.data_ptr(), fed.stride(0), R, rot, rot,
                                             wkv.data_ptr(), rotary.inv_freq.data_ptr(), tok_pos.data_ptr(),
                                             loc.data_ptr(), cache.data_ptr(), cache.stride(0), 1e-5, amp * amp, T,
                                             _lib.dtype_code(dtype), 0)
    _lib.check(rc, "latent_prep")
    want_c = P.unit_rms(raw[:, :R].double(), 1e-5) * wkv.double().cpu()
    want_r = P.rotate_half_pairs(raw[:, R:].double(), torch.tensor(pos), spec)[:, order] * amp   # amp once more
    tol = 2e-5 if dtype == torch.float32 else 6e-3                     # angles are fp32: 4097 * f rounds
    assert _err(cache[1:, :R], want_c) <= tol
    assert _err(cache[1:, R:], want_r) <= tol


# ---- one mixer option at a time, through the engine --------------------------------------------------
def _neutral(cfg, w):
    """Weights that switch the attention mixer's options off: heads do not mix, gates are one half."""
    for i, L in enumerate(cfg["layers"]):
        if L["type"] == "attention":
            H = L["mixer"]["heads"]
            w[f"l{i}.mix.talk"] = torch.eye(H).to(torch.bfloat16)
            w[f"l{i}.mix.g"] = torch.zeros_like(w[f"l{i}.mix.g"])
    return w


VARIANTS = {
    "plain": dict(softcap=None, every=0),
    "temperature": dict(softcap=None, every=5, coef=1.5),
    "cap": dict(softcap=2.0, every=0, scale=1.0),
    "talk": dict(softcap=None, every=0),
    "gate": dict(softcap=None, every=0),
    "value_mix": dict(softcap=None, every=0),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("variant", list(VARIANTS))
def test_attention_options_one_at_a_time(tmp_path, variant, dtype):
    kw = VARIANTS[variant]
    layers = [(U.attention(heads=4, kv_heads=2, dim=16, vdim=12, v_mix=variant == "value_mix", **kw), None)]
    if variant == "value_mix":
        layers.append((U.attention(heads=2, kv_heads=2, dim=8, vdim=12, v_mix=True, **kw), None))
    cfg = U.config(layers, width=32)
    w = U.random_weights(cfg, 3)
    keep = {k: w[k] for k in w if (variant == "talk" and k.endswith("talk")) or (variant == "gate" and k.endswith("mix.g"))}
    w = _neutral(cfg, w)
    w.update(keep)
    folder = U.write_model(str(tmp_path / variant), cfg, w)
    toks = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(1)).tolist()
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, dtype)
    d.step([("r", toks[:40])])
    d.step([("r", toks[40:43])])
    for t in toks[43:]:
        d.step([("r", [t])])
    assert U.rel_err(d.result("r"), want, dtype) <= (1e-4 if dtype == torch.float32 else 6e-2)
    if variant != "plain":      # the option matters: the neutral model's logits differ
        base_cfg = U.config([(U.attention(heads=4, kv_heads=2, dim=16, vdim=12, v_mix=False, **VARIANTS["plain"]), None)],
                            width=32)
        base = P.forward(base_cfg, _neutral(base_cfg, U.random_weights(base_cfg, 3)), toks)
        if len(layers) == 1:
            assert float(U.rel_errs(want, base).max()) > 1e-2


def test_unit_sink_and_first_tokens(tmp_path):
    """With tiny scores every weight is 1 / (n + 1): at position 0 the sink takes half, so the first
    tokens show at once whether it is there."""
    cfg = U.config([(U.attention(heads=2, kv_heads=1, dim=8, vdim=8, scale=1e-4, softcap=None, every=0, v_mix=False), None)],
                   width=16)
    w = _neutral(cfg, U.random_weights(cfg, 4))
    folder = U.write_model(str(tmp_path / "m"), cfg, w)
    toks = [3, 9, 27, 81, 50]
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, torch.float32)
    for t in toks:
        d.step([("r", [t])])
    assert U.rel_err(d.result("r"), want) <= 1e-4
    # the restatement without the sink is visibly another function at the first positions
    h = P.norm_one_plus(w["embed"].double()[torch.tensor(toks)] * 0.7, w["l0.norm1"].double(), 1e-5)
    v = P.unit_rms((h @ w["l0.mix.v"].double().T + w["l0.mix.v.b"].double()).view(5, 1, 8), 1e-5)
    with_sink = v[0, 0] * 0.5 * 0.5                                    # weight 1/2, gate 1/2
    got0 = P.talking_attention(h, w, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5, None)
    o0 = torch.cat([with_sink, with_sink]) @ w["l0.mix.o"].double().T + w["l0.mix.o.b"].double()
    assert (got0[0] - o0).abs().max() <= 1e-3


@pytest.mark.parametrize("decode", [False, True])
def test_far_keys_page_borders_and_the_causal_edge(tmp_path, decode):
    """One key is made to stand out for the last query: the query projection is the key projection with
    its input coordinates reversed, and the key token's embedding is the query token's reversed, so
    q(query) = k(key) and their score is |k|^2 while every other score is a random one.  Whether that key
    is seen decides the output.  It sits at position 0, hundreds of tokens back, on either side of a
    page border, right before the query; a copy placed after the query must not be seen."""
    H, D, E, W, T = 2, 64, 16, 32, 330
    cfg = U.config([(U.attention(heads=H, kv_heads=1, dim=D, vdim=E, scale=1.0, softcap=30.0, every=0, v_mix=False), None)],
                   width=W, vocab=64, embed_scale=1.0)
    w = _neutral(cfg, U.random_weights(cfg, 6))
    w["l0.mix.k"] = w["l0.mix.k"] * 0.3
    w["l0.mix.q"] = torch.cat([w["l0.mix.k"].flip(1)] * H)
    w["l0.mix.q.b"], w["l0.mix.k.b"] = torch.zeros_like(w["l0.mix.q.b"]), torch.zeros_like(w["l0.mix.k.b"])
    w["l0.norm1"] = torch.zeros_like(w["l0.norm1"])
    g = torch.Generator().manual_seed(7)
    w["embed"] = torch.randn(64, W, generator=g).to(torch.bfloat16)
    w["embed"][62] = w["embed"][63].flip(0)          # token 63: the query's; token 62: its stand-out key
    folder = U.write_model(str(tmp_path / "m"), cfg, w)
    base = torch.randint(0, 60, (T,), generator=g).tolist()
    base[-1] = 63
    outs = {}
    for key in (0, 1, 63, 64, 65, 127, 128, 200, T - 2, None):
        toks = list(base)
        if key is not None:
            toks[key] = 62
        want = P.forward(cfg, w, toks)[T - 1]
        d = U.Driver(folder, torch.float32)
        if decode:
            d.step([("r", toks[:T - 3])])
            for t in toks[T - 3:]:
                d.step([("r", [t])])
        else:
            d.step([("r", toks + [62, 62])])          # copies after the query, in the same portion
        got = d.result("r")[T - 1]
        assert float(U.rel_errs(got[None], want[None]).max()) <= 1e-4, key
        outs[key] = want
    for key in outs:
        if key is not None:       # seeing the key moves the logits a lot
            assert float(U.rel_errs(outs[key][None], outs[None][None]).max()) > 0.05, key


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("form", ["absorbed", "expanded"])
@pytest.mark.parametrize("sizes", [dict(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40),
                                   dict(heads=2, dim=8, rot_dim=32, vdim=16, kv_rank=24, factor=None),
                                   dict(heads=5, dim=6, rot_dim=6, vdim=7, kv_rank=13, factor=16.0, original=32)])
def test_gated_latent_attention_alone(tmp_path, monkeypatch, dtype, form, sizes):
    from sglang_security_b200.layers.attention.latent_attention import LatentAttention

    if form == "expanded" and dtype == torch.float32:
        pytest.skip("the expanded form is a 16-bit form")
    monkeypatch.setattr(LatentAttention, "force_form", form)
    cfg = U.config([(U.latent(**sizes), None)], width=32)
    w = U.random_weights(cfg, 8)
    folder = U.write_model(str(tmp_path / "m"), cfg, w)
    toks = torch.randint(0, cfg["vocab"], (150,), generator=torch.Generator().manual_seed(2)).tolist()
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, dtype)
    d.step([("r", toks[:100])])
    d.step([("r", toks[100:130])])
    for t in toks[130:]:
        d.step([("r", [t])])
    assert U.rel_err(d.result("r"), want, dtype) <= (1e-4 if dtype == torch.float32 else 6e-2)


def test_rotation_amplitude_and_frequencies_matter(tmp_path):
    """The scaled rotation is not the unscaled one: both the stretched frequencies and the amplitude
    change the plain model's logits, so agreement above is agreement on them."""
    a = U.config([(U.latent(factor=4.0), None)], width=32)
    b = U.config([(U.latent(factor=None), None)], width=32)
    w = U.random_weights(a, 8)
    toks = list(range(60))
    assert float(U.rel_errs(P.forward(a, w, toks), P.forward(b, w, toks)).max()) > 1e-2
    f, amp = P.rotation_table(a["layers"][0]["mixer"]["rot"])
    assert amp == pytest.approx(0.1 * math.log(4.0) + 1) and f[-1] < 0.3 * 10000.0 ** (-2 * 3 / 8)
