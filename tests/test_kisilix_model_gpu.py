"""Kisilix through the engine (loader, ModelRunner, pools, scheduler) against the plain restatement:
whole prompts, per-layer residuals, token-by-token decoding, portions down to two tokens, unequal
requests in one batch with pages and request slots freed and used again, window and block edges made
visible by a peaked softmax, long decoding, and greedy generation through Engine.generate."""
import pytest
import torch

import kisilix_plain as P
import kisilix_util as U

pytestmark = pytest.mark.gpu

CONFIGS = {
    # every mixer and both feed-forwards; blocks of 4 (divide the page) and of 5 (do not).  The experts
    # sit in the last layer: with random weights 16-bit rounding flips a router's choice between two
    # near-equal experts now and then, and a flip in a middle layer would reach every later token through
    # the recurrences ("m" below has the experts in the middle and runs in 32 bits, where flips are rare)
    "a": lambda: U.config([(U.delta(), U.dense()), (U.ssm(), U.dense(24, 0.8)), (U.attn(), U.dense()),
                           (U.attn(heads=2, kv_heads=2, dim=24, vdim=8, window=33, pool=5, rot_dims=24), None),
                           (U.delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=2, ranks=(4, 4)), U.moe(6, 3, 16, 3, 2, 0))]),
    "m": lambda: U.config([(U.ssm(), U.moe()), (U.attn(), U.moe(9, 3, 16, 3, 2, 24)),
                           (U.delta(), U.moe(6, 2, 16, 0, 0, 8)), (U.attn(window=12, pool=3), U.moe(4, 4, 8, 2, 2, 0))]),
    # sizes that are multiples of nothing, a convolution of one tap, top = experts, no groups, no shared
    # expert, attention first, 3 : 1 grouping, block = window
    "b": lambda: U.config([(U.attn(heads=3, kv_heads=1, dim=6, vdim=10, window=7, pool=7, rot_dims=2, base=50.0), U.dense(21, 0.7)),
                           (U.delta(heads=3, kv_heads=3, dim=10, vdim=6, conv=1, ranks=(3, 5)), None),
                           (U.ssm(heads=2, vdim=7, state=5, groups=1, norm_groups=1, conv=3), U.moe(6, 6, 9, 0, 0, 0))],
                          vocab=131, width=27, eps=1e-3, alpha=1.0),
    # ones: one head, window 1 with blocks of 1, top 1, one group kept; no window at all; a window without
    # blocks; no rotation; memories wider than a warp's rows (key sizes 40 and 72, 70 value columns)
    "c": lambda: U.config([(U.attn(heads=1, kv_heads=1, dim=8, vdim=8, window=1, pool=1, rot_dims=4), U.moe(4, 1, 8, 4, 1, 8)),
                           (U.attn(heads=2, kv_heads=1, dim=8, vdim=6, window=None, pool=0, rot_dims=8), None),
                           (U.attn(heads=2, kv_heads=2, dim=8, vdim=6, window=9, pool=0, rot_dims=0), None),
                           (U.delta(heads=1, kv_heads=1, dim=40, vdim=70, conv=3, ranks=(5, 7)), None),
                           (U.ssm(heads=2, vdim=9, state=72, groups=2, norm_groups=3, conv=5), None)],
                          vocab=33, width=24, alpha=5.0),
    # attention sizes the tensor-core kernel takes (key size = value size = 64 / 128), 4 : 1 and 1 : 1, with
    # and without blocks, with and without a window
    "d": lambda: U.config([(U.attn(heads=4, kv_heads=1, dim=64, vdim=64, window=50, pool=8, rot_dims=32), U.dense(32)),
                           (U.ssm(heads=2, vdim=16, state=16, groups=1, norm_groups=1), None),
                           (U.attn(heads=2, kv_heads=2, dim=128, vdim=128, window=70, pool=0, rot_dims=128), None),
                           (U.attn(heads=2, kv_heads=1, dim=64, vdim=64, window=None, pool=0, rot_dims=64), None)],
                          vocab=101, width=64),
    # recurrent layers only (no token pool rows at all)
    "f": lambda: U.config([(U.ssm(), U.dense()), (U.delta(), None)], vocab=61, width=32),
    # attention only
    "g": lambda: U.config([(U.attn(window=30, pool=6), None), (U.attn(window=8, pool=2, rot_dims=16), U.dense())],
                          vocab=61, width=48),
}


def _model(tmp_path, name, seed=0, sharp=0.0):
    cfg = CONFIGS[name]()
    if sharp:        # a peaked softmax: one key or block more or less in sight moves the logits a lot
        for L in cfg["layers"]:
            if L["type"] == "attention":
                L["mixer"]["scale"] *= sharp
    w = U.random_weights(cfg, seed)
    return cfg, w, U.write_model(str(tmp_path / name), U.clean(cfg), w)


def _tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# 16 bits: five layers with gains above one carry the rounding of every stored activation to the logits
# (90th percentile, see rel_err); a dtype-specific fault is of order one
TOL = {torch.float32: 1e-4, torch.bfloat16: 0.15}
# a peaked softmax also amplifies rounding (16-bit keys times a six-fold scale would drown the edges, so
# the 16-bit runs sharpen less); a key or block wrongly seen or missed moves the fp32 logits by 1e-1 and more
SHARP = {torch.float32: 6.0, torch.bfloat16: 2.0}
TOL_SHARP = {torch.float32: 1e-3, torch.bfloat16: 0.3}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "f", "g"])
def test_whole_prompt_matches_plain_model(tmp_path, name, dtype):
    cfg, w, folder = _model(tmp_path, name)
    toks = _tokens(cfg, 150, 1)
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, dtype)
    d.step([("r", toks)], end=["r"])
    assert U.rel_err(d.result("r"), want, dtype) <= TOL[dtype]


@pytest.mark.parametrize("name", ["m", "g"])
def test_experts_in_the_middle_fp32(tmp_path, name):
    cfg, w, folder = _model(tmp_path, name)
    toks = _tokens(cfg, 150, 6)
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, torch.float32)
    at = 0
    for n in U.cut(len(toks), [40, 1, 2, 70]):
        d.step([("r", toks[at:at + n])])
        at += n
    assert U.rel_err(d.result("r"), want) <= TOL[torch.float32]


@pytest.mark.parametrize("name", ["a", "b", "c", "m"])
def test_layer_outputs_match_plain_model_fp32(tmp_path, name):
    from sglang_security_b200.managers.schedule_batch import Req, StepItem

    cfg, w, folder = _model(tmp_path, name)
    toks = _tokens(cfg, 40, 2)
    want = []
    P.forward(cfg, w, toks, layers_out=want)
    d = U.Driver(folder, torch.float32)
    req = Req(rid="x", input_ids=list(toks))
    d.runner.admit(req)
    got = []
    d.sched.run_step([StepItem(req, list(toks), want=[0])], layer_hook=lambda i, x: got.append(x.double().cpu().clone()))
    assert len(got) == len(want)
    for g, t in zip(got, want):
        assert (g - t).abs().max() <= 2e-5 * t.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_prefill_then_token_by_token(tmp_path, name, dtype):
    cfg, w, folder = _model(tmp_path, name, sharp=SHARP[dtype])
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
    cfg, w, folder = _model(tmp_path, "a", sharp=SHARP[dtype])
    toks = _tokens(cfg, 140, 4)
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, dtype)
    at = 0
    for n in U.cut(len(toks), sizes):
        d.step([("r", toks[at:at + n])])
        at += n
    assert U.rel_err(d.result("r"), want, dtype) <= TOL_SHARP[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["a", "b", "f", "g"])
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


@pytest.mark.parametrize("sharp", [0.0, 2.0])
def test_long_portions_on_the_tensor_core_kernel_beside_decoded_tokens(tmp_path, monkeypatch, sharp):
    """Portions of 16 tokens and more take the tcgen05 kernel for the window, the CUDA-core kernel for the
    blocks and the joining launch; shorter ones and decoded tokens the CUDA-core kernel alone, in the same
    step; every cut must give the whole prompt's logits."""
    from sglang_security_b200.layers.attention.pooled_window_attention import PooledWindowAttention

    monkeypatch.setattr(PooledWindowAttention, "tensor_core_min_tokens", 16)
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
    err_a, err_b = U.rel_err(d.result("a"), want_a, torch.bfloat16), U.rel_err(d.result("b"), want_b, torch.bfloat16)
    assert err_a <= tol and err_b <= tol
    monkeypatch.setattr(PooledWindowAttention, "tensor_core_min_tokens", 0)    # the CUDA-core kernel alone agrees
    d = U.Driver(folder, torch.bfloat16)
    d.step([("a", a)], end=["a"])
    core = U.rel_err(d.result("a"), want_a, torch.bfloat16)
    assert core <= tol and err_a <= 2.0 * core + 0.02        # the divided step is as close to the oracle


def test_long_decoding(tmp_path):
    cfg, w, folder = _model(tmp_path, "a")
    toks = _tokens(cfg, 430, 5)
    want = P.forward(cfg, w, toks)
    d = U.Driver(folder, torch.float32)
    d.step([("r", toks[:30])])
    for t in toks[30:]:
        d.step([("r", [t])])
    assert U.rel_err(d.result("r"), want) <= 1e-4


def test_the_table_of_positions_bounds_a_sequence(tmp_path):
    from sglang_security_b200.managers.schedule_batch import OutOfCache

    cfg = U.config([(U.ssm(), None)], vocab=31, width=16, max_positions=70)
    folder = U.write_model(str(tmp_path / "short"), U.clean(cfg), U.random_weights(cfg))
    d = U.Driver(folder, torch.float32, max_tokens=256)
    assert d.runner.context_length == 70
    d.step([("r", _tokens(cfg, 70, 1))])
    with pytest.raises(OutOfCache):
        d.step([("r", [1])])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_engine(tmp_path, dtype):
    from sglang_security_b200.entrypoints.engine import Engine
    from sglang_security_b200.managers.schedule_batch import SamplingParams

    cfg, w, folder = _model(tmp_path, "a")
    prompts = [_tokens(cfg, n, 30 + i) for i, n in enumerate([70, 9, 130, 33, 2])]     # more requests than slots
    eng = Engine(folder, dtype, max_total_tokens=1024, max_running_requests=3, chunked_prefill_size=48)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    assert eng.runner.free_token_slots() == eng.runner.max_total_tokens
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o) == 12
        if dtype == torch.float32:
            # teacher-forced: every generated token is (within rounding) the oracle's best token there
            logits, slack = P.forward(cfg, w, p + o[:-1])[len(p) - 1:], 1e-3
        else:
            # 16 bits: held to the same engine fed the same tokens as one prompt (the scheduler's cuts, slots
            # and pages must not matter); the fp32 run holds the engine to the oracle
            d = U.Driver(folder, dtype)
            d.step([(f"r{i}", p + o[:-1])], end=[f"r{i}"])
            logits, slack = d.result(f"r{i}").double()[len(p) - 1:], 0.1
        best = logits.max(-1).values
        took = logits[torch.arange(len(o)), torch.tensor(o)]
        assert ((best - took) <= slack * logits.std(-1)).all()
