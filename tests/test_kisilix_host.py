"""Kisilix on the host: configuration read-out and rejections, registry, tensor names, sizes taken from
the checkpoint's shapes, and self-checks of the plain restatement (what a position sees)."""
import pytest
import torch

import kisilix_plain as P
import kisilix_util as U
from sglang_security_b200.configs.kisilix import (ChannelDeltaSpec, ClampedMLPSpec, GroupedExpertsSpec,
                                                  PooledAttentionSpec, StateSpaceSpec, kisilix_config)
from sglang_security_b200.configs.model_config import ModelConfig
from sglang_security_b200.models.registry import resolve_model_cls, supported_architectures


def _cfg():
    return U.config([(U.delta(), U.dense()), (U.ssm(), U.moe()), (U.attn(), U.moe(shared=0, groups=0)),
                     (U.attn(window=None, rot_dims=0), None)])


def test_configuration_reads_every_size_from_the_file():
    c = kisilix_config(U.clean(_cfg()))
    assert (c.vocab, c.width, c.alpha, c.eps, c.max_positions, c.num_layers) == (97, 48, 2.0, 1e-5, 600, 4)
    d, s, a, b = (L.mixer for L in c.layers)
    assert isinstance(d, ChannelDeltaSpec) and (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (4, 2, 16, 24, 4)
    assert isinstance(s, StateSpaceSpec) and (s.heads, s.vdim, s.state, s.groups, s.norm_groups, s.conv) == (4, 12, 16, 2, 2, 2)
    assert isinstance(a, PooledAttentionSpec) and (a.window, a.pool, a.rope_dims, a.rope_base) == (20, 4, 8, 1000.0)
    assert (b.window, b.pool, b.rope_dims) == (None, 0, 0)
    f0, f1, f2, f3 = (L.mlp for L in c.layers)
    assert isinstance(f0, ClampedMLPSpec) and (f0.ff, f0.limit) == (40, 1.5)
    assert isinstance(f1, GroupedExpertsSpec) and (f1.experts, f1.top, f1.groups, f1.keep, f1.shared_ff) == (8, 2, 4, 2, 32)
    assert (f2.groups, f2.keep, f2.shared_ff) == (1, 1, 0) and f3 is None


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "cannot share"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "norm groups"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "rotated"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=23), "even value size"),
    (lambda c: c["layers"][2]["mixer"].update(mask={"pool": 4}), "need a window"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top 9"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=8), "cannot give"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown feed-forward"),
])
def test_inconsistent_configurations_are_rejected(edit, text):
    c = U.clean(_cfg())
    edit(c)
    with pytest.raises(ValueError, match=text):
        kisilix_config(c)


def test_registry_and_tensor_names(tmp_path):
    assert "Kisilix" in supported_architectures()
    cfg = _cfg()
    w = U.random_weights(cfg)
    folder = U.write_model(str(tmp_path / "m"), U.clean(cfg), w)
    mc = ModelConfig(folder)
    assert mc.architecture == "Kisilix"
    mc.hf_config.resolve_shapes({k: tuple(v.shape) for k, v in w.items()})
    assert (mc.hf_config.layers[0].mixer.decay_rank, mc.hf_config.layers[0].mixer.gate_rank) == (8, 16)
    model = resolve_model_cls("Kisilix")(mc.hf_config, params_dtype=torch.bfloat16)
    assert model.expected_tensor_names() == set(w)
    model.load_weights(w.items())
    spec = model.cache_spec()
    assert set(spec.row_dims) == {2, 3} and spec.block_summaries == {2: 4} and set(spec.state_widths) == {0, 1}
    d, s = model.layers[0].mix, model.layers[1].mix
    assert spec.state_widths[0] == 3 * (2 * 2 * 16 + 4 * 24) + 4 * 16 * 24
    assert spec.state_widths[1] == 1 * (4 * 12 + 2 * 2 * 16) + 4 * 16 * 12
    # fused input projection [q ; k ; v ; a1 ; g1 ; b] and the shared output-norm weight, once per head
    assert torch.equal(d.in_proj.weight[32:64], w["l0.mix.k"]) and torch.equal(d.in_proj.weight[-4:], w["l0.mix.b"])
    assert torch.equal(d.norm_weight.view(4, 24)[3], w["l0.mix.norm"].float())
    assert torch.equal(d.conv_weight[64:], w["l0.mix.v.conv"].float()) and s.conv_bias is not None
    with pytest.raises(ValueError, match="lacks"):
        model.load_weights((k, v) for k, v in w.items() if k != "l1.mix.D")
    with pytest.raises(ValueError, match="unexpected"):
        model.load_weights(list(w.items()) + [("l3.mlp.gate", w["l0.mlp.gate"])])


def test_what_a_position_sees():
    assert P.visible(5, 0, 0) == (list(range(6)), [])
    assert P.visible(9, 4, 0) == ([6, 7, 8, 9], [])
    # window 4, blocks of 3: position 9 sees 6..9 and the blocks that end at or before 5: {0,1,2}, {3,4,5}
    assert P.visible(9, 4, 3) == ([6, 7, 8, 9], [0, 1])
    assert P.visible(8, 4, 3) == ([5, 6, 7, 8], [0])          # block 1 ends at 5 > 8 - 4: token 3, 4 unseen
    assert P.visible(3, 4, 3) == ([0, 1, 2, 3], [])
    assert P.visible(6, 1, 1) == ([6], [0, 1, 2, 3, 4, 5])


def test_router_choice_and_weights():
    W = {"r.router": torch.eye(6, dtype=torch.float64) * 2.0,
         "r.correction": torch.tensor([0., 0., 0., 0., 5., -5.], dtype=torch.float64)}
    h = torch.tensor([[3., 2.5, 0., 0., 0., 2.9]], dtype=torch.float64)
    ids, w = P.route(h, W, "r.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    # the correction lifts expert 4 and its group {4, 5}; only that group may be chosen, and the weights
    # are the plain scores of 4 and 5 renormalised (5 far larger than 4)
    assert sorted(ids[0].tolist()) == [4, 5]
    s = torch.softmax(h @ W["r.router"].T, -1)[0]
    got = dict(zip(ids[0].tolist(), w[0].tolist()))
    assert abs(got[5] - float(s[5] / (s[4] + s[5]))) < 1e-12 and got[5] > 0.99
