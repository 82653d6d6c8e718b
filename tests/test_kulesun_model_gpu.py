"""Kulesun through the engine (loader, ModelRunner, pools, scheduler) against the plain restatement:
whole prompts, per-layer residuals, token-by-token decoding, portions down to two tokens, unequal
requests in one batch with pages and request slots freed and used again, peaked softmaxes, long
decoding, the tensor-core kernels beside decoded tokens, and greedy generation through Engine.generate."""
import pytest
import torch

import kulesun_plain as P
import kulesun_util as U

pytestmark = pytest.mark.gpu

CONFIGS = {
    # attention - latent - latent - attention (mixing with the first) - latent without feed-forward
    "a": lambda: U.config([(U.attention(), U.dense()), (U.latent(), U.dense()), (U.latent(heads=2, kv_rank=24), U.dense(32)),
                           (U.attention(heads=4, kv_heads=2, dim=8), U.dense()), (U.latent(), None)]),
    # other sizes: a latent layer first, one key/value head per query head, five query heads on one
    # key/value head, no cap, a temperature step of one position, no rotation scaling, a latent size that is
    # no multiple of 8, the first mixing layer not the first attention layer, scales of one
    "b": lambda: U.config([(U.latent(heads=1, dim=10, rot_dim=6, vdim=12, kv_rank=20, factor=None, base=500.0), None),
                           (U.attention(heads=3, kv_heads=3, dim=10, vdim=6, softcap=None, every=1, v_mix=False), U.dense(40)),
                           (U.attention(heads=5, kv_heads=1, dim=12, vdim=9, every=48, coef=0.9), None),
                           (U.latent(heads=4, dim=16, rot_dim=16, vdim=8, kv_rank=32, factor=32.0, original=16, fast=4.0, slow=0.5), U.dense(16)),
                           (U.attention(heads=2, kv_heads=1, dim=20, vdim=9, softcap=3.0, every=0), U.dense(24))],
                          vocab=131, width=72, eps=1e-3, embed_scale=1.0, logit_scale=1.0),
    # sizes that are multiples of nothing, one head everywhere
    "c": lambda: U.config([(U.attention(heads=1, kv_heads=1, dim=6, vdim=11, every=3), U.dense(9)),
                           (U.latent(heads=1, dim=5, rot_dim=2, vdim=3, kv_rank=7), None),
                           (U.attention(heads=1, kv_heads=1, dim=6, vdim=11, every=2, coef=2.0), None)],
                          vocab=53, width=27, eps=1e-4, embed_scale=2.0, logit_scale=0.05),
    # sizes the tensor-core kernels take: attention key size = value size = 64 grouped 2 : 1 and 128
    # (two value heads per launch; capped in the one-pass form and uncapped), three key/value heads (a pair
    # and a single one) with a cap too large for the one-pass form, one key/value head, latent heads that
    # expand to 64
    "d": lambda: U.config([(U.attention(heads=4, kv_heads=2, dim=64, vdim=64, every=40), U.dense(64)),
                           (U.latent(heads=2, dim=32, rot_dim=32, vdim=32, kv_rank=64), None),
                           (U.attention(heads=4, kv_heads=2, dim=64, vdim=64, every=64, softcap=None), None),
                           (U.attention(heads=2, kv_heads=2, dim=128, vdim=128, v_mix=False, softcap=None), U.dense(64)),
                           (U.attention(heads=4, kv_heads=2, dim=128, vdim=128, v_mix=False, softcap=25.0), None),
                           (U.attention(heads=6, kv_heads=3, dim=64, vdim=64, v_mix=False, every=0, softcap=60.0), None),
                           (U.attention(heads=2, kv_heads=1, dim=64, vdim=64, v_mix=False, softcap=8.0), None)],
                          vocab=101, width=64),
    # attention only, no layer mixes values; latent only
    "e": lambda: U.config([(U.attention(v_mix=False), None), (U.attention(heads=2, kv_heads=2, v_mix=False), U.dense())],
                          vocab=61, width=48),
    "f": lambda: U.config([(U.latent(), U.dense()), (U.latent(heads=6, dim=8, rot_dim=4, vdim=8, kv_rank=16), None)],
                          vocab=61, width=32),
}


def _model(tmp_path, name, seed=0, sharp=False):
    cfg = CONFIGS[name]()
    if sharp:        # peaked softmaxes: a key more or less moves the logits a lot (uncapped scores grow
        for L in cfg["layers"]:          # without bound, and fp32 rounding with them: a smaller factor there)
            L["mixer"]["scale"] *= 5.0 if L["mixer"].get("softcap") else 2.5
    w = U.random_weights(cfg, seed)
    return cfg, w, U.write_model(str(tmp_path / name), cfg, w)


def _tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


TOL = {torch.float32: 1e-4, torch.bfloat16: 6e-2}
TOL_SHARP = {torch.float32: 1e-4, torch.bfloat16: 0.15}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_plain_model(tmp_path, name, dtype):
    cfg, w, folder = _model(tmp_path, name)
    toks = _tokens(cfg, 150, 1)
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, dtype)
    d.step([("r", toks)], end=["r"])
    assert U.rel_err(d.result("r"), want, dtype) <= TOL[dtype]


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_layer_outputs_match_plain_model_fp32(tmp_path, name):
    from sglang_security_b200.managers.schedule_batch import Req, StepItem

    cfg, w, folder = _model(tmp_path, name)
    toks = _tokens(cfg, 40, 2)
    want = []
    P.forward(cfg, w, toks, layer_outputs=want)
    d = U.Driver(folder, torch.float32)
    req = Req(rid="x", input_ids=list(toks))
    d.runner.admit(req)
    got = []
    d.sched.run_step([StepItem(req, list(toks), want=[0])], layer_hook=lambda i, x: got.append(x.double().cpu().clone()))
    assert len(got) == len(want)
    for g, t in zip(got, want):
        assert (g - t).abs().max() <= 2e-5 * t.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["a", "b"])
def test_prefill_then_token_by_token(tmp_path, name, dtype):
    cfg, w, folder = _model(tmp_path, name, sharp=True)
    toks = _tokens(cfg, 130, 3)
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, dtype)
    d.step([("r", toks[:60])])
    for t in toks[60:]:
        d.step([("r", [t])])
    assert U.rel_err(d.result("r"), want, dtype) <= TOL_SHARP[dtype]
    d2 = U.Driver(folder, dtype)                 # from the very first token on, one at a time
    for t in toks[:40]:
        d2.step([("s", [t])])
    assert U.rel_err(d2.result("s"), want[:40], dtype) <= TOL_SHARP[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [[2], [3, 64, 2, 17, 1], [64, 5]])
def test_portions_of_a_prompt(tmp_path, dtype, sizes):
    cfg, w, folder = _model(tmp_path, "a", sharp=True)
    toks = _tokens(cfg, 140, 4)
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, dtype)
    at = 0
    for n in U.cut(len(toks), sizes):
        d.step([("r", toks[at:at + n])])
        at += n
    assert U.rel_err(d.result("r"), want, dtype) <= TOL_SHARP[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["a", "b", "c", "f"])
def test_unequal_requests_in_one_batch_with_slots_and_pages_reused(tmp_path, name, dtype):
    cfg, w, folder = _model(tmp_path, name)
    lens = {"p": 150, "q": 37, "r": 90, "s": 1, "t": 64, "u": 129, "v": 20}
    toks = {k: _tokens(cfg, n, 10 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: P.forward(cfg, w, t) for k, t in toks.items()}
    d = U.Driver(folder, dtype, max_tokens=512, max_requests=3)      # fewer slots and pages than requests need
    at = {k: 0 for k in lens}
    waiting, live, sizes, step = list(lens), [], [33, 1, 2, 64, 1, 7], 0
    while waiting or live:
        while waiting and len(live) < 3 and sum(-(-lens[k] // 64) for k in live + [waiting[0]]) <= 8:
            live.append(waiting.pop(0))
        portions, ended = [], []
        for j, k in enumerate(live):
            n = min(sizes[(step + j) % len(sizes)], lens[k] - at[k])
            portions.append((k, toks[k][at[k]:at[k] + n]))
            at[k] += n
            if at[k] == lens[k]:
                ended.append(k)
        d.step(portions, end=ended)
        live = [k for k in live if k not in ended]
        step += 1
    for k in lens:
        assert U.rel_err(d.result(k), want[k], dtype) <= TOL[dtype], k
    assert d.runner.free_token_slots() == d.runner.max_total_tokens


def test_batch_does_not_change_a_request_fp32(tmp_path):
    cfg, w, folder = _model(tmp_path, "a")
    a, b = _tokens(cfg, 80, 20), _tokens(cfg, 45, 21)
    alone = U.Driver(folder, torch.float32)
    alone.step([("a", a)], end=["a"])
    both = U.Driver(folder, torch.float32)
    both.step([("b", b[:30]), ("a", a[:50])])
    both.step([("a", a[50:]), ("b", b[30:31])])
    assert (alone.result("a") - both.result("a")).abs().max() <= 1e-4


@pytest.mark.parametrize("sharp", [False, True])
def test_long_portions_on_the_tensor_core_kernels_beside_decoded_tokens(tmp_path, monkeypatch, sharp):
    """Portions of 16 tokens and more take the tcgen05 kernel (one launch per value head), shorter ones
    and decoded tokens the CUDA-core kernel, in the same step; the latent layers divide the step between
    their two forms.  Every cut must give the whole prompt's logits."""
    from sglang_security_b200.layers.attention.latent_attention import LatentAttention
    from sglang_security_b200.layers.attention.talking_heads_attention import TalkingHeadsAttention

    monkeypatch.setattr(TalkingHeadsAttention, "tensor_core_min_tokens", 16)
    monkeypatch.setattr(LatentAttention, "force_form", "split")
    cfg, w, folder = _model(tmp_path, "d", sharp=sharp)
    a, b = _tokens(cfg, 300, 40), _tokens(cfg, 170, 41)
    want_a, want_b = P.forward(cfg, w, a), P.forward(cfg, w, b)
    tol = (TOL_SHARP if sharp else TOL)[torch.bfloat16]
    d = U.Driver(folder, torch.bfloat16)
    d.step([("a", a)], end=["a"])
    assert U.rel_err(d.result("a"), want_a, torch.bfloat16) <= tol
    d = U.Driver(folder, torch.bfloat16)
    d.step([("a", a[:130]), ("b", b[:5])])
    d.step([("a", a[130:131]), ("b", b[5:150])])
    d.step([("a", a[131:290]), ("b", b[150:151])])
    d.step([("a", a[290:]), ("b", b[151:])])
    assert U.rel_err(d.result("a"), want_a, torch.bfloat16) <= tol
    assert U.rel_err(d.result("b"), want_b, torch.bfloat16) <= tol
    monkeypatch.setattr(TalkingHeadsAttention, "tensor_core_min_tokens", 0)   # the CUDA-core kernel alone agrees
    monkeypatch.setattr(LatentAttention, "force_form", "absorbed")
    d = U.Driver(folder, torch.bfloat16)
    d.step([("a", a)], end=["a"])
    assert U.rel_err(d.result("a"), want_a, torch.bfloat16) <= tol


def test_long_decoding(tmp_path):
    cfg, w, folder = _model(tmp_path, "a")
    toks = _tokens(cfg, 430, 5)
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, torch.float32)
    d.step([("r", toks[:30])])
    for t in toks[30:]:
        d.step([("r", [t])])
    assert U.rel_err(d.result("r"), want) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_engine(tmp_path, dtype):
    from sglang_security_b200.entrypoints.engine import Engine
    from sglang_security_b200.managers.schedule_batch import SamplingParams

    cfg, w, folder = _model(tmp_path, "a")
    prompts = [_tokens(cfg, n, 30 + i) for i, n in enumerate([70, 9, 130, 33, 2])]     # more requests than slots
    eng = Engine(folder, dtype, max_total_tokens=1024, max_running_requests=3, chunked_prefill_size=48)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    assert eng.runner.free_token_slots() == eng.runner.max_total_tokens
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = P.forward(cfg, w, p + o[:-1])[len(p) - 1:]
        # teacher-forced: every generated token is (within rounding) the oracle's best token there
        best = logits.max(-1).values
        took = logits[torch.arange(len(o)), torch.tensor(o)]
        slack = 1e-3 if dtype == torch.float32 else 0.15
        assert ((best - took) <= slack * logits.std(-1)).all()
