"""Host-side pieces of the Kulesun family (no GPU): configuration parsing and its checks, the scaled
rotation's frequency table and the row order that turns the half pairing into neighbours, the model's
construction and checkpoint bookkeeping, and the registry."""
import math

import pytest
import torch

import kulesun_plain as P
import kulesun_util as U


def test_config_reads_every_size_and_constant():
    from sglang_security_b200.configs.kulesun import kulesun_config

    raw = U.config([(U.attention(heads=6, kv_heads=3, dim=10, vdim=14, softcap=7.5, coef=0.25, every=9), U.dense(33)),
                    (U.latent(heads=5, dim=12, rot_dim=6, vdim=9, kv_rank=21, base=777.0, factor=3.0, original=48,
                              fast=5.0, slow=0.5), None)],
                   vocab=71, width=28, eps=3e-4, embed_scale=1.7, logit_scale=0.4)
    cfg = kulesun_config(raw)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.embedding_scale, cfg.logit_scale) == (71, 28, 3e-4, 1.7, 0.4)
    a, b = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.softcap, a.temp_coef, a.temp_every, a.v_mix) == (6, 3, 10, 14, 7.5, 0.25, 9, True)
    assert (b.heads, b.dim, b.rot_dim, b.vdim, b.kv_rank) == (5, 12, 6, 9, 21)
    assert (b.rot.dims, b.rot.base, b.rot.factor, b.rot.original, b.rot.fast, b.rot.slow) == (6, 777.0, 3.0, 48.0, 5.0, 0.5)
    assert cfg.layers[0].mlp.ff == 33 and cfg.layers[1].mlp is None and cfg.first_v_mix_layer == 0


def test_config_rejects_what_the_layers_cannot_run():
    from sglang_security_b200.configs.kulesun import kulesun_config

    with pytest.raises(ValueError):
        kulesun_config(U.config([(U.attention(heads=5, kv_heads=2), None)]))
    with pytest.raises(ValueError):        # mixed values of another shape than the first mixing layer's
        kulesun_config(U.config([(U.attention(kv_heads=2, vdim=24), None), (U.attention(kv_heads=2, vdim=16), None)]))
    with pytest.raises(ValueError):
        kulesun_config(U.config([({"type": "convolution", "mixer": {}}, None)]))
    bad = U.config([(U.latent(rot_dim=8), None)])
    bad["layers"][0]["mixer"]["rot"]["dims"] = 10
    with pytest.raises(ValueError):
        kulesun_config(bad)
    ok = kulesun_config(U.config([(U.attention(v_mix=False), None), (U.attention(kv_heads=3, vdim=8, v_mix=False), None)]))
    assert ok.first_v_mix_layer is None


@pytest.mark.parametrize("dims,base,factor,original,fast,slow", [(32, 5e5, 4.0, 2048, 16.0, 2.0), (8, 1e4, 4.0, 64, 16.0, 1.0),
                                                                  (16, 500.0, 32.0, 16, 4.0, 0.5), (6, 1e4, 2.0, 4096, 1.0, 1.0)])
def test_scaled_frequency_table(dims, base, factor, original, fast, slow):
    from sglang_security_b200.layers.rotary_embedding import ramp_scaled_frequencies

    f, amp = ramp_scaled_frequencies(dims, base, factor, original, fast, slow)
    want, want_amp = P.rotation_table({"dims": dims, "base": base,
                                       "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}})
    assert torch.allclose(f, want, rtol=1e-12, atol=0) and amp == pytest.approx(want_amp)
    plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    assert (f <= plain * (1 + 1e-12)).all() and (f >= plain / factor * (1 - 1e-12)).all()


def test_row_order_turns_the_half_pairing_into_neighbours():
    """Rotating neighbours of the reordered vector is the half-pairing rotation, reordered; a dot product
    of two vectors reordered alike is unchanged."""
    from sglang_security_b200.layers.rotary_embedding import PairedRotary

    dims, width = 8, 11
    rot = PairedRotary(dims, 100.0, pairing="half", amplitude=1.3)
    order = rot.row_order(width)
    assert sorted(order.tolist()) == list(range(width)) and order[dims:].tolist() == list(range(dims, width))
    x = torch.randn(5, width, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    pos = torch.tensor([0, 1, 7, 100, 1000])
    want = P.rotate_half_pairs(x, pos, {"dims": dims, "base": 100.0})[:, order]
    y = x[:, order].clone()
    for i in range(dims // 2):
        a = pos.double() * rot.inv_freq[i].double()
        u, v = y[:, 2 * i].clone(), y[:, 2 * i + 1].clone()
        y[:, 2 * i], y[:, 2 * i + 1] = u * torch.cos(a) - v * torch.sin(a), v * torch.cos(a) + u * torch.sin(a)
    assert torch.allclose(y, want, atol=1e-3, rtol=0)      # the layer's frequencies are rounded to fp32
    assert (y - x[:, order]).abs().max() > 0.1              # and the rotation is not the identity
    assert PairedRotary(dims, 100.0).row_order(width).tolist() == list(range(width))


def test_model_builds_and_accounts_for_its_tensors():
    from sglang_security_b200.configs.kulesun import kulesun_config
    from sglang_security_b200.models.registry import resolve_model_cls, supported_architectures

    assert "Kulesun" in supported_architectures()
    raw = U.config([(U.latent(), U.dense()), (U.attention(), None), (U.attention(heads=4, kv_heads=2, dim=8), U.dense())])
    w = U.random_weights(raw)
    model = resolve_model_cls("Kulesun")(kulesun_config(raw), params_dtype=torch.float32)
    model.load_weights(w.items())
    spec = model.cache_spec()
    assert spec.kind == "rows" and spec.row_dims == {0: 48, 1: 2 * (16 + 24), 2: 2 * (8 + 24)} and not spec.state_widths
    assert model.layers[1].mix.v_first_layer is None and model.layers[2].mix.v_first_layer == 1
    # norms are stored around zero
    assert torch.allclose(model.layers[0].norm1.weight, 1 + w["l0.norm1"].float())
    assert torch.allclose(model.final_norm.weight, 1 + w["final.norm"].float())
    # the rotated rows of a latent layer's query and key projections are reordered alike
    m, att = raw["layers"][0]["mixer"], model.layers[0].mix
    order = att.rotary.row_order(m["rot_dim"])
    got_kr = att.down_proj.weight[att.q_part + m["kv_rank"]:att.q_part + m["kv_rank"] + m["rot_dim"]]
    assert torch.equal(got_kr, w["l0.mix.dkv"].float()[m["kv_rank"]:][order])
    q0 = att.down_proj.weight[:m["dim"] + m["rot_dim"]]
    assert torch.equal(q0[:m["dim"]], w["l0.mix.q"].float()[:m["dim"]])
    assert torch.equal(q0[m["dim"]:], w["l0.mix.q"].float()[m["dim"]:m["dim"] + m["rot_dim"]][order])
    # a missing or unknown tensor is an error; the first mixing layer's mix weight is not needed
    for drop in ("l1.mix.talk", "l0.mix.g", "l2.mix.vmix", "l2.norm2b"):
        with pytest.raises(ValueError):
            resolve_model_cls("Kulesun")(kulesun_config(raw), params_dtype=torch.float32).load_weights(
                (k, v) for k, v in w.items() if k != drop)
    resolve_model_cls("Kulesun")(kulesun_config(raw), params_dtype=torch.float32).load_weights(
        (k, v) for k, v in w.items() if k != "l1.mix.vmix")
    with pytest.raises(ValueError):
        model.load_weights(list(w.items()) + [("l1.mix.sink", torch.zeros(6))])


def test_temperature_steps():
    t = P.query_temperature(torch.arange(0, 30), 0.5, 7)
    assert t[5] == 1.0 and t[6] == pytest.approx(1 + 0.5 * math.log(2)) and t[12] == t[6] and t[13] > t[12]
