"""Prefill and decode throughput of the Desirax, Dozetar, Kulesun and Kisilix designs at layer sizes that resemble
a real model's, beside the Llama-family decoder stack of this package at equal width / heads / head size /
layer count and equal active feed-forward size (random weights, bf16).  Driven by
`bench.py --arch-compare` (sizes named "dz-..." are Dozetar's, "ku-..." Kulesun's; a Kulesun size also
runs the Desirax stack, its closest relative, at equal width, heads, latent sizes, layers and feed-forward;
"ki-..." are Kisilix's, which also run the Dozetar stack — recurrent memories of the same shape, windowed
attention with the same heads, experts of the same size).

Timing: CUDA events on the launching stream around whole engine steps, after warm-up steps; every step
touches more weight and cache bytes than L2 holds at the larger size.  Per-kernel times come from the
library's timing registry (events around each launch) in a separate pass."""
from __future__ import annotations

import json
import statistics
import time
from types import SimpleNamespace

import torch

from .. import _lib

SIZES = {
    # dense feed-forward everywhere: the direct counterpart of a Llama layer
    "w1024-dense": dict(width=1024, heads=8, dim=64, rot=64, vdim=128, kv_rank=256, q_rank=384, window=1024,
                        layers=4, ff=4096, moe=None, vocab=32000),
    # mixture of experts with a shared expert; active feed-forward 4 * 1024 + 1024
    "w2048-moe": dict(width=2048, heads=16, dim=64, rot=64, vdim=128, kv_rank=512, q_rank=768, window=4096,
                      layers=4, ff=5120, moe=dict(experts=32, top=4, ff=1024, shared=1024), vocab=32000),
}
# Dozetar: layers alternate the gated matrix-memory mixer and the parallel (attention | decayed
# linear attention) mixer; every layer has experts.  `ff` is the Llama-like stack's dense size = the
# active expert size top * expert_ff.
DOZETAR_SIZES = {
    "dz-w1024": dict(width=1024, layers=4, vocab=32000, heads=8, kv_heads=2, dim=128, vdim=128, window=1024,
                     keep_first=4, rot=64, m_heads=8, m_dim=64, m_vdim=128, r_heads=8, r_dim=64, r_vdim=128,
                     experts=16, top=2, expert_ff=1024, ff=2048, rot_llama=0),
    "dz-w2048": dict(width=2048, layers=4, vocab=32000, heads=16, kv_heads=4, dim=128, vdim=128, window=4096,
                     keep_first=4, rot=64, m_heads=16, m_dim=128, m_vdim=128, r_heads=16, r_dim=64, r_vdim=128,
                     experts=32, top=4, expert_ff=1024, ff=4096, rot_llama=0),
}
# Kulesun: layers alternate the talking-heads attention mixer and two latent-attention mixers; dense
# silu feed-forward everywhere.  The latent sizes are those of the Desirax row it is compared with.
KULESUN_SIZES = {
    "ku-w1024": dict(width=1024, layers=4, vocab=32000, heads=8, kv_heads=2, adim=128, avdim=128, dim=64, rot=64,
                     vdim=128, kv_rank=256, q_rank=384, window=1 << 20, ff=4096, moe=None, rot_llama=64),
    "ku-w2048": dict(width=2048, layers=4, vocab=32000, heads=16, kv_heads=2, adim=128, avdim=128, dim=64, rot=64,
                     vdim=128, kv_rank=512, q_rank=768, window=1 << 20, ff=8192, moe=None, rot_llama=64),
}
# Kisilix: delta rule, attention (window + pooled blocks), state space, attention; experts with a shared
# expert in every layer.  The memories have the shapes of the Dozetar row's (mlstm = delta rule, decayed =
# state space), the attention its heads, the experts its sizes.
KISILIX_SIZES = {
    "ki-w1024": dict(DOZETAR_SIZES["dz-w1024"], pool=64, conv=4, rank=64, groups=4, keep=2, shared=1024),
    "ki-w2048": dict(DOZETAR_SIZES["dz-w2048"], pool=64, conv=4, rank=128, groups=4, keep=2, shared=1024),
}
WORK = dict(prefill_reqs=4, prefill_len=2048, decode_bs=32, decode_ctx=2048)


def _dozetar_cfg(s):
    mlstm = {"type": "mlstm", "mixer": {"heads": s["m_heads"], "dim": s["m_dim"], "vdim": s["m_vdim"], "gate_cap": 15.0}}
    par = {"type": "parallel", "mixer": {
        "left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"],
                 "scale": s["dim"] ** -0.5, "mask": {"size": s["window"], "keep_first": s["keep_first"]},
                 "rot": {"base": 1e6, "dims": s["rot"]}},
        "right": {"heads": s["r_heads"], "dim": s["r_dim"], "vdim": s["r_vdim"],
                  "decay": [1.0 - 2.0 ** (-3 - 5 * i / max(1, s["r_heads"] - 1)) for i in range(s["r_heads"])]},
        "left_scale": 0.7, "right_scale": 0.7}}
    f = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"]}}
    return {"architecture": "Dozetar", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "residual_mult": 0.7, "logit_softcap": 50.0,
            "layers": [dict(mlstm if i % 2 == 0 else par, mlp=f) for i in range(s["layers"])]}


def _desirax_cfg(s):
    m = {"dim": s["dim"], "heads": s["heads"], "kv_rank": s["kv_rank"], "q_rank": s["q_rank"],
         "rot_dim": s["rot"], "vdim": s["vdim"], "rot": {"base": 1e6, "dims": s["rot"]},
         "scale": (s["dim"] + s["rot"]) ** -0.5, "mask": {"size": s["window"]}}
    if s["moe"]:
        f = {"kind": "moe", "router": {"experts": s["moe"]["experts"], "top": s["moe"]["top"]},
             "expert": {"ff": s["moe"]["ff"]}, "shared": {"ff": s["moe"]["shared"]}}
    else:
        f = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Desirax", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
            "layers": [{"type": "latent_attention", "mixer": dict(m), "mlp": f} for _ in range(s["layers"])]}


def _timed(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    return statistics.median(ms)


def _kernel_times(fn, names):
    _lib.timing_enable(True)
    _lib.timing_read("")
    fn()
    torch.cuda.synchronize()
    out = {}
    for n in names:
        k, ms = _lib.timing_read(n)
        if k:
            out[n] = {"launches": k, "ms": round(ms, 4)}
    _lib.timing_enable(False)
    _lib.timing_read("")
    return out


def bench_desirax(name, s, steps, warmup, device="cuda"):
    from ..configs.desirax import desirax_config
    from ..managers.schedule_batch import Req, StepItem
    from ..managers.scheduler import Scheduler
    from ..models.registry import resolve_model_cls
    from .model_runner import ModelRunner

    cfg = desirax_config(_desirax_cfg(s))
    torch.manual_seed(0)
    with torch.device(device):
        model = resolve_model_cls("Desirax")(cfg, params_dtype=torch.bfloat16)
    for n_, p in model.named_parameters():
        if p.dim() == 0:
            p.data.fill_(1.0)
        elif n_.endswith("mu"):
            p.data.uniform_(0, 1)
        elif "norm_weight" in n_:
            p.data.fill_(1.0)
        else:
            p.data.normal_(0, 0.02)
    W = WORK
    bs = max(W["prefill_reqs"], W["decode_bs"])
    tokens = W["decode_bs"] * (W["decode_ctx"] + 64) + W["prefill_reqs"] * W["prefill_len"]
    runner = ModelRunner(None, torch.bfloat16, max_total_tokens=tokens, max_running_requests=bs + 1,
                         context_length=max(W["prefill_len"], W["decode_ctx"] + 64), device=device,
                         model=model.eval(), model_config=SimpleNamespace(architecture="Desirax", hf_config=cfg))
    sched = Scheduler(runner)
    g = torch.Generator().manual_seed(1)
    rnd = lambda n: torch.randint(0, s["vocab"], (n,), generator=g).tolist()

    def prefill():
        reqs = [Req(rid=f"p{i}", input_ids=rnd(W["prefill_len"])) for i in range(W["prefill_reqs"])]
        for r in reqs:
            assert runner.admit(r)
        sched.run_step([StepItem(r, r.input_ids, want=[len(r.input_ids) - 1]) for r in reqs])
        for r in reqs:
            runner.release(r)

    row = {"arch": "desirax", "size": name}
    ms = _timed(prefill, steps, warmup)
    ntok = W["prefill_reqs"] * W["prefill_len"]
    row["prefill_ms"], row["prefill_tokens_per_s"] = round(ms, 3), round(ntok / ms * 1e3)
    attn_names = ["latent_attn", "attn_extend", "latent_expand", "latent_prep", "moe_grouped_gemm",
                  "moe_route", "moe_align", "scalar_rmsnorm_shift", "residual_combine", "act_and_mul"]
    row["prefill_kernels"] = _kernel_times(prefill, attn_names)
    # the same prompts with the attention pinned to its absorbed (latent) form
    from ..layers.attention.latent_attention import LatentAttention
    LatentAttention.force_form = "absorbed"
    try:
        row["prefill_absorbed_ms"] = round(_timed(prefill, steps, warmup), 3)
        row["prefill_absorbed_kernels"] = _kernel_times(prefill, ["latent_attn"])
    finally:
        LatentAttention.force_form = None
    # decode: bs requests at the decode context
    reqs = [Req(rid=f"d{i}", input_ids=rnd(W["decode_ctx"])) for i in range(W["decode_bs"])]
    for r in reqs:
        assert runner.admit(r)
    for i in range(0, len(reqs), 4):
        sched.run_step([StepItem(r, r.input_ids) for r in reqs[i:i + 4]])
    state = {"n": 0}

    def decode():
        state["n"] += 1
        assert state["n"] < 60
        sched.run_step([StepItem(r, [7], want=[0]) for r in reqs])

    ms = _timed(decode, steps, warmup)
    row["decode_ms"], row["decode_tokens_per_s"] = round(ms, 3), round(W["decode_bs"] / ms * 1e3)
    row["decode_kernels"] = _kernel_times(decode, attn_names)
    # a mixed step, as the scheduler forms them: every running request decodes one token beside one
    # 512-token portion of a new prompt (the long portion runs expanded, the decodes absorbed)
    def mixed():
        state["n"] += 1
        assert state["n"] < 60
        new = Req(rid=f"m{state['n']}", input_ids=rnd(512))
        assert runner.admit(new)
        sched.run_step([StepItem(r, [7], want=[0]) for r in reqs] + [StepItem(new, new.input_ids, want=[511])])
        runner.release(new)

    row["mixed_ms"] = round(_timed(mixed, min(steps, 8), 3), 3)
    LatentAttention.force_form = "absorbed"
    try:
        row["mixed_absorbed_ms"] = round(_timed(mixed, min(steps, 8), 3), 3)
    finally:
        LatentAttention.force_form = None
    H, R, rot, Wn = s["heads"], s["kv_rank"], s["rot"], min(s["window"], W["prefill_len"])
    # latent attention, algorithmic work of one launch (all tokens, one layer)
    keys_prefill = sum(min(p + 1, s["window"]) for p in range(W["prefill_len"])) * W["prefill_reqs"]
    row["latent_attn_prefill_flops"] = 2 * keys_prefill * H * (2 * R + rot)
    d_exp = 64 if max(s["dim"] + rot, s["vdim"]) <= 64 else 128
    row["expanded_attn_prefill_flops"] = 2 * keys_prefill * H * 2 * d_exp
    keys_decode = W["decode_bs"] * min(W["decode_ctx"] + 1, s["window"])
    row["latent_attn_decode_bytes"] = keys_decode * (R + rot) * 2
    row["latent_attn_decode_flops"] = 2 * keys_decode * H * (2 * R + rot)
    del runner, sched, model
    torch.cuda.empty_cache()
    return row


def bench_dozetar(name, s, steps, warmup, device="cuda"):
    from ..configs.dozetar import dozetar_config
    from ..managers.schedule_batch import Req, StepItem
    from ..managers.scheduler import Scheduler
    from ..models.registry import resolve_model_cls
    from .model_runner import ModelRunner

    cfg = dozetar_config(_dozetar_cfg(s))
    torch.manual_seed(0)
    with torch.device(device):
        model = resolve_model_cls("Dozetar")(cfg, params_dtype=torch.bfloat16)
    for n_, p in model.named_parameters():
        if n_.endswith("norm_weight") or n_.endswith("norm1.weight") or n_.endswith("norm2.weight") or \
                n_.endswith("final_norm.weight"):
            p.data.fill_(1.0)
        elif n_.endswith("gate_bias"):
            p.data.fill_(1.0)
        elif n_.endswith("sink") or n_.endswith("bias"):
            p.data.zero_()
        else:
            p.data.normal_(0, 0.02)
    W = WORK
    bs = max(W["prefill_reqs"], W["decode_bs"])
    tokens = W["decode_bs"] * (W["decode_ctx"] + 64) + W["prefill_reqs"] * W["prefill_len"]
    runner = ModelRunner(None, torch.bfloat16, max_total_tokens=tokens, max_running_requests=bs + 1,
                         context_length=max(W["prefill_len"], W["decode_ctx"] + 64), device=device,
                         model=model.eval(), model_config=SimpleNamespace(architecture="Dozetar", hf_config=cfg))
    sched = Scheduler(runner)
    g = torch.Generator().manual_seed(1)
    rnd = lambda n: torch.randint(0, s["vocab"], (n,), generator=g).tolist()

    def prefill():
        reqs = [Req(rid=f"p{i}", input_ids=rnd(W["prefill_len"])) for i in range(W["prefill_reqs"])]
        for r in reqs:
            assert runner.admit(r)
        sched.run_step([StepItem(r, r.input_ids, want=[len(r.input_ids) - 1]) for r in reqs])
        for r in reqs:
            runner.release(r)

    names = ["linear_recurrence", "gated_group_rmsnorm", "sink_attn", "attn_extend", "qk_norm_rope_write",
             "moe_grouped_gemm", "moe_route", "moe_align", "add_normed", "softcap_rows"]
    row = {"arch": "dozetar", "size": name}
    ms = _timed(prefill, steps, warmup)
    ntok = W["prefill_reqs"] * W["prefill_len"]
    row["prefill_ms"], row["prefill_tokens_per_s"] = round(ms, 3), round(ntok / ms * 1e3)
    row["prefill_kernels"] = _kernel_times(prefill, names)
    reqs = [Req(rid=f"d{i}", input_ids=rnd(W["decode_ctx"])) for i in range(W["decode_bs"])]
    for r in reqs:
        assert runner.admit(r)
    for i in range(0, len(reqs), 4):
        sched.run_step([StepItem(r, r.input_ids) for r in reqs[i:i + 4]])
    state = {"n": 0}

    def decode():
        state["n"] += 1
        assert state["n"] < 60
        sched.run_step([StepItem(r, [7], want=[0]) for r in reqs])

    ms = _timed(decode, steps, warmup)
    row["decode_ms"], row["decode_tokens_per_s"] = round(ms, 3), round(W["decode_bs"] / ms * 1e3)
    row["decode_kernels"] = _kernel_times(decode, names)

    def mixed():
        state["n"] += 1
        assert state["n"] < 60
        new = Req(rid=f"m{state['n']}", input_ids=rnd(512))
        assert runner.admit(new)
        sched.run_step([StepItem(r, [7], want=[0]) for r in reqs] + [StepItem(new, new.input_ids, want=[511])])
        runner.release(new)

    row["mixed_ms"] = round(_timed(mixed, min(steps, 8), 3), 3)
    # algorithmic work of one launch (all tokens, one layer)
    L, U = W["prefill_len"], W["prefill_reqs"]
    keys = sum(min(p + 1, s["window"]) + min(s["keep_first"], max(0, p + 1 - s["window"])) for p in range(L)) * U
    row["attn_prefill_flops"] = 2 * keys * s["heads"] * (s["dim"] + s["vdim"])
    keys_d = W["decode_bs"] * (min(W["decode_ctx"] + 1, s["window"]) + s["keep_first"])
    row["attn_decode_bytes"] = keys_d * s["kv_heads"] * (s["dim"] + s["vdim"]) * 2
    # recurrences: 3 fp32 multiply-adds per state element and token (decay, outer product, read-out); a
    # decoded token reads and writes its state once
    row["mlstm_prefill_fma"] = 3 * U * L * s["m_heads"] * s["m_dim"] * s["m_vdim"]
    row["decayed_prefill_fma"] = 3 * U * L * s["r_heads"] * s["r_dim"] * s["r_vdim"]
    row["mlstm_decode_bytes"] = 2 * 4 * W["decode_bs"] * s["m_heads"] * s["m_dim"] * s["m_vdim"]
    row["decayed_decode_bytes"] = 2 * 4 * W["decode_bs"] * s["r_heads"] * s["r_dim"] * s["r_vdim"]
    row["expert_prefill_flops"] = 2 * 2 * U * L * s["top"] * s["expert_ff"] * s["width"]
    del runner, sched, model
    torch.cuda.empty_cache()
    return row


def _kulesun_cfg(s):
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["adim"],
                                          "vdim": s["avdim"], "scale": s["adim"] ** -0.5, "softcap": 30.0,
                                          "q_temp": {"coef": 0.3, "every": 512}, "v_mix": True}}
    lat = {"type": "latent_attention", "mixer": {
        "heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot"], "vdim": s["vdim"], "kv_rank": s["kv_rank"],
        "scale": (s["dim"] + s["rot"]) ** -0.5,
        "rot": {"base": 5e5, "dims": s["rot"], "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}}
    f = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Kulesun", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "logit_scale": 1.0,
            "layers": [dict(att if i % 3 == 0 else lat, mlp=f) for i in range(s["layers"])]}


def bench_kulesun(name, s, steps, warmup, device="cuda"):
    from ..configs.kulesun import kulesun_config
    from ..managers.schedule_batch import Req, StepItem
    from ..managers.scheduler import Scheduler
    from ..models.registry import resolve_model_cls
    from .model_runner import ModelRunner

    cfg = kulesun_config(_kulesun_cfg(s))
    torch.manual_seed(0)
    with torch.device(device):
        model = resolve_model_cls("Kulesun")(cfg, params_dtype=torch.bfloat16)
    for n_, p in model.named_parameters():
        if n_.endswith("norm_weight") or ("norm" in n_ and n_.endswith(".weight")):
            p.data.fill_(1.0)
        elif n_.endswith("head_mix"):
            p.data.copy_(torch.eye(p.shape[0], device=p.device) * 0.8 + 0.02)
        elif n_.endswith("v_mix"):
            p.data.fill_(0.3)
        elif n_.endswith("bias"):
            p.data.zero_()
        else:
            p.data.normal_(0, 0.02)
    W = WORK
    bs = max(W["prefill_reqs"], W["decode_bs"])
    tokens = W["decode_bs"] * (W["decode_ctx"] + 64) + W["prefill_reqs"] * W["prefill_len"]
    runner = ModelRunner(None, torch.bfloat16, max_total_tokens=tokens, max_running_requests=bs + 1,
                         context_length=max(W["prefill_len"], W["decode_ctx"] + 64), device=device,
                         model=model.eval(), model_config=SimpleNamespace(architecture="Kulesun", hf_config=cfg))
    sched = Scheduler(runner)
    g = torch.Generator().manual_seed(1)
    rnd = lambda n: torch.randint(0, s["vocab"], (n,), generator=g).tolist()

    def prefill():
        reqs = [Req(rid=f"p{i}", input_ids=rnd(W["prefill_len"])) for i in range(W["prefill_reqs"])]
        for r in reqs:
            assert runner.admit(r)
        sched.run_step([StepItem(r, r.input_ids, want=[len(r.input_ids) - 1]) for r in reqs])
        for r in reqs:
            runner.release(r)

    names = ["sink_attn", "attn_extend", "qk_norm_rope_write", "head_mix_gate", "sigmoid_gate_mul", "latent_attn",
             "latent_expand", "latent_prep", "add_normed", "act_and_mul", "scalar_rmsnorm_shift"]
    row = {"arch": "kulesun", "size": name}
    ms = _timed(prefill, steps, warmup)
    ntok = W["prefill_reqs"] * W["prefill_len"]
    row["prefill_ms"], row["prefill_tokens_per_s"] = round(ms, 3), round(ntok / ms * 1e3)
    row["prefill_kernels"] = _kernel_times(prefill, names)
    reqs = [Req(rid=f"d{i}", input_ids=rnd(W["decode_ctx"])) for i in range(W["decode_bs"])]
    for r in reqs:
        assert runner.admit(r)
    for i in range(0, len(reqs), 4):
        sched.run_step([StepItem(r, r.input_ids) for r in reqs[i:i + 4]])
    state = {"n": 0}

    def decode():
        state["n"] += 1
        assert state["n"] < 60
        sched.run_step([StepItem(r, [7], want=[0]) for r in reqs])

    ms = _timed(decode, steps, warmup)
    row["decode_ms"], row["decode_tokens_per_s"] = round(ms, 3), round(W["decode_bs"] / ms * 1e3)
    row["decode_kernels"] = _kernel_times(decode, names)

    def mixed():
        state["n"] += 1
        assert state["n"] < 60
        new = Req(rid=f"m{state['n']}", input_ids=rnd(512))
        assert runner.admit(new)
        sched.run_step([StepItem(r, [7], want=[0]) for r in reqs] + [StepItem(new, new.input_ids, want=[511])])
        runner.release(new)

    row["mixed_ms"] = round(_timed(mixed, min(steps, 8), 3), 3)
    # algorithmic work of one attention layer, all tokens.  Heads' weights mixed after the softmax: the
    # cheapest exact one-pass form scores every pair once and applies every head's weights to the values of
    # each of the G key/value heads (2 * pairs * H * (D + G * E)); what runs is one launch per value head
    L, U, H, G, D, E = W["prefill_len"], W["prefill_reqs"], s["heads"], s["kv_heads"], s["adim"], s["avdim"]
    pairs = U * (L * (L + 1) // 2)
    row["attn_prefill_flops_needed"] = 2 * pairs * H * (D + G * E)
    row["attn_prefill_flops_run"] = 2 * pairs * H * G * (D + E)
    row["attn_layers"] = sum(1 for x in cfg.layers if x.type == "attention")
    keys_d = W["decode_bs"] * (W["decode_ctx"] + 1)
    row["attn_decode_bytes"] = keys_d * G * (D + E) * 2
    R, rot = s["kv_rank"], s["rot"]
    row["latent_attn_prefill_flops"] = 2 * pairs * H * (2 * R + rot)
    d_exp = 64 if max(s["dim"] + rot, s["vdim"]) <= 64 else 128
    row["expanded_attn_prefill_flops"] = 2 * pairs * H * 2 * d_exp
    row["latent_attn_decode_bytes"] = keys_d * (R + rot) * 2
    del runner, sched, model
    torch.cuda.empty_cache()
    return row


def _kisilix_cfg(s):
    delta = {"type": "channel_delta", "mixer": {"heads": s["m_heads"], "kv_heads": s["m_heads"], "dim": s["m_dim"],
                                                "vdim": s["m_vdim"], "conv": s["conv"]}}
    ssm = {"type": "mamba2", "mixer": {"heads": s["r_heads"], "vdim": s["r_vdim"], "state": s["r_dim"], "groups": 1,
                                       "norm_groups": 1, "conv": s["conv"]}}
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"],
                                          "vdim": s["vdim"], "scale": s["dim"] ** -0.5,
                                          "mask": {"size": s["window"], "pool": s["pool"]},
                                          "rot": {"base": 1e6, "dims": s["rot"]}}}
    f = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"],
                                   "groups": {"count": s["groups"], "keep": s["keep"]}},
         "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared"]}}
    order = [delta, att, ssm, att]
    return {"architecture": "Kisilix", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "postln_alpha": 2.0, "max_positions": 4096,
            "layers": [dict(order[i % 4], mlp=f) for i in range(s["layers"])]}


def bench_kisilix(name, s, steps, warmup, device="cuda"):
    from ..configs.kisilix import kisilix_config
    from ..managers.schedule_batch import Req, StepItem
    from ..managers.scheduler import Scheduler
    from ..models.registry import resolve_model_cls
    from .model_runner import ModelRunner

    cfg = kisilix_config(_kisilix_cfg(s))
    for L in cfg.layers:
        if L.type == "channel_delta":
            L.mixer.decay_rank = L.mixer.gate_rank = s["rank"]
    torch.manual_seed(0)
    with torch.device(device):
        model = resolve_model_cls("Kisilix")(cfg, params_dtype=torch.bfloat16)
    for n_, p in model.named_parameters():
        if n_.endswith("norm_weight") or n_.endswith("norm1.weight") or n_.endswith("norm2.weight") or \
                n_.endswith("final_norm.weight") or n_.endswith("head_scale"):
            p.data.fill_(1.0)
        elif n_.endswith("bias") or n_.endswith("correction") or n_.endswith("a_log") or n_.endswith("skip"):
            p.data.zero_()
        elif n_.endswith("conv_weight"):
            p.data.normal_(0, 0.5)
        else:
            p.data.normal_(0, 0.02)
    W = WORK
    bs = max(W["prefill_reqs"], W["decode_bs"])
    tokens = W["decode_bs"] * (W["decode_ctx"] + 64) + W["prefill_reqs"] * W["prefill_len"]
    runner = ModelRunner(None, torch.bfloat16, max_total_tokens=tokens, max_running_requests=bs + 1,
                         context_length=max(W["prefill_len"], W["decode_ctx"] + 64), device=device,
                         model=model.eval(), model_config=SimpleNamespace(architecture="Kisilix", hf_config=cfg))
    sched = Scheduler(runner)
    g = torch.Generator().manual_seed(1)
    rnd = lambda n: torch.randint(0, s["vocab"], (n,), generator=g).tolist()

    def prefill():
        reqs = [Req(rid=f"p{i}", input_ids=rnd(W["prefill_len"])) for i in range(W["prefill_reqs"])]
        for r in reqs:
            assert runner.admit(r)
        sched.run_step([StepItem(r, r.input_ids, want=[len(r.input_ids) - 1]) for r in reqs])
        for r in reqs:
            runner.release(r)

    names = ["delta_recurrence", "ssm_recurrence", "causal_conv_silu", "gated_group_rmsnorm", "pooled_window_attn",
             "attn_extend", "pooled_merge_unrotate", "headnorm_rot_write", "pool_block_means", "moe_grouped_gemm", "moe_route", "moe_align",
             "scaled_add_layernorm", "act_and_mul"]
    row = {"arch": "kisilix", "size": name}
    ms = _timed(prefill, steps, warmup)
    ntok = W["prefill_reqs"] * W["prefill_len"]
    row["prefill_ms"], row["prefill_tokens_per_s"] = round(ms, 3), round(ntok / ms * 1e3)
    row["prefill_kernels"] = _kernel_times(prefill, names)
    reqs = [Req(rid=f"d{i}", input_ids=rnd(W["decode_ctx"])) for i in range(W["decode_bs"])]
    for r in reqs:
        assert runner.admit(r)
    for i in range(0, len(reqs), 4):
        sched.run_step([StepItem(r, r.input_ids) for r in reqs[i:i + 4]])
    state = {"n": 0}

    def decode():
        state["n"] += 1
        assert state["n"] < 60
        sched.run_step([StepItem(r, [7], want=[0]) for r in reqs])

    ms = _timed(decode, steps, warmup)
    row["decode_ms"], row["decode_tokens_per_s"] = round(ms, 3), round(W["decode_bs"] / ms * 1e3)
    row["decode_kernels"] = _kernel_times(decode, names)

    def mixed():
        state["n"] += 1
        assert state["n"] < 60
        new = Req(rid=f"m{state['n']}", input_ids=rnd(512))
        assert runner.admit(new)
        sched.run_step([StepItem(r, [7], want=[0]) for r in reqs] + [StepItem(new, new.input_ids, want=[511])])
        runner.release(new)

    row["mixed_ms"] = round(_timed(mixed, min(steps, 8), 3), 3)
    # algorithmic work of one launch (all tokens, one layer)
    L, U = W["prefill_len"], W["prefill_reqs"]
    vis = lambda p: min(p + 1, s["window"]) + max(0, p + 1 - s["window"]) // s["pool"]
    keys = sum(vis(p) for p in range(L)) * U
    row["attn_prefill_flops"] = 2 * keys * s["heads"] * (s["dim"] + s["vdim"])
    row["attn_decode_bytes"] = W["decode_bs"] * (min(W["decode_ctx"] + 1, s["window"]) * 2 + (
        max(0, W["decode_ctx"] + 1 - s["window"]) // s["pool"]) * 4) * s["kv_heads"] * (s["dim"] + s["vdim"])
    # recurrences: fp32 multiply-adds per memory element and token: the delta rule has four (decay, S^T k,
    # the write, the read-out), the state-space form three; a decoded token reads and writes its memory once
    row["delta_prefill_fma"] = 4 * U * L * s["m_heads"] * s["m_dim"] * s["m_vdim"]
    row["ssm_prefill_fma"] = 3 * U * L * s["r_heads"] * s["r_dim"] * s["r_vdim"]
    row["delta_decode_bytes"] = 2 * 4 * W["decode_bs"] * s["m_heads"] * s["m_dim"] * s["m_vdim"]
    row["ssm_decode_bytes"] = 2 * 4 * W["decode_bs"] * s["r_heads"] * s["r_dim"] * s["r_vdim"]
    row["expert_prefill_flops"] = 2 * 3 * U * L * s["top"] * s["expert_ff"] * s["width"]
    del runner, sched, model
    torch.cuda.empty_cache()
    return row


def bench_llama_like(name, s, steps, warmup, device="cuda"):
    """The package's Llama-family stack (B200DecoderLayer: fused RMSNorm, rotary + KV write, paged
    attention, gated silu MLP) at the same width, heads, head size 128, layers, GQA 4:1, bf16."""
    from .decode_step import B200DecodeStep, ModelGeometry
    from .forward_batch_info import ForwardBatch, ForwardMode

    W = WORK
    hd = s["dim"] + s.get("rot_llama", s["rot"])
    geo = ModelGeometry(name, s["width"], s["heads"], max(1, s["heads"] // 4), hd, s["ff"], s["layers"],
                        s["vocab"], 1e6, False)
    bs = W["decode_bs"]
    ctx_cap = max(W["prefill_len"], W["decode_ctx"] + 64)
    model = B200DecodeStep(geo, None, device, max_bs=bs, max_ctx=ctx_cap, fill_kv=True)
    dev = device
    rows = torch.arange(bs, device=dev)
    model.req_to_token_pool.req_to_token[:bs, :ctx_cap] = (
        1 + rows[:, None] * ctx_cap + torch.arange(ctx_cap, device=dev)[None]).to(torch.int32)
    U, L = W["prefill_reqs"], W["prefill_len"]
    ids = torch.randint(0, s["vocab"], (U * L,), device=dev)
    pos = torch.arange(L, device=dev).repeat(U)
    ext = torch.full((U,), L, dtype=torch.int32)
    pre = torch.zeros(U, dtype=torch.int32)
    start = torch.arange(U, dtype=torch.int32) * L
    loc = model.req_to_token_pool.req_to_token[:U, :L].reshape(-1).to(torch.int64)
    fb = ForwardBatch(forward_mode=ForwardMode.EXTEND, batch_size=U,
                      req_pool_indices=torch.arange(U, dtype=torch.int64, device=dev),
                      seq_lens=ext.to(torch.int64).to(dev), out_cache_loc=loc, seq_lens_sum=U * L,
                      seq_lens_cpu=ext.to(torch.int64), extend_seq_lens=ext.to(dev), extend_prefix_lens=pre.to(dev),
                      extend_start_loc=start.to(dev), extend_seq_lens_cpu=[L] * U, extend_prefix_lens_cpu=[0] * U,
                      extend_num_tokens=U * L, req_to_token_pool=model.req_to_token_pool,
                      token_to_kv_pool=model.token_to_kv_pool, attn_backend=model.attn_backend)
    last = (start + ext - 1).to(torch.int64).to(dev)
    out = torch.empty((U,), dtype=torch.int64, device=dev)
    model.attn_backend.init_forward_metadata(fb)
    row = {"arch": "llama-like", "size": name}
    prefill = lambda: model.forward_extend(ids, pos, fb, last, out)
    ms = _timed(prefill, steps, warmup)
    row["prefill_ms"], row["prefill_tokens_per_s"] = round(ms, 3), round(U * L / ms * 1e3)
    names = ["attn_extend", "attn_decode_split", "attn_decode", "attn_merge", "rmsnorm", "silu_and_mul", "rope_kv_write"]
    row["prefill_kernels"] = _kernel_times(prefill, names)
    p = W["decode_ctx"]
    d_len = torch.full((bs,), p + 1, dtype=torch.int64, device=dev)
    d_loc = model.req_to_token_pool.req_to_token[:bs, p].to(torch.int64)
    fbd = model.make_forward_batch(bs, torch.arange(bs, dtype=torch.int64, device=dev), d_len, d_loc, bs * (p + 1))
    model.attn_backend.init_forward_metadata(fbd)
    d_ids = torch.randint(0, s["vocab"], (bs,), device=dev)
    d_pos = torch.full((bs,), p, dtype=torch.int64, device=dev)
    d_out = torch.empty((bs,), dtype=torch.int64, device=dev)
    decode = lambda: model.forward(d_ids, d_pos, fbd, d_out)
    ms = _timed(decode, steps, warmup)
    row["decode_ms"], row["decode_tokens_per_s"] = round(ms, 3), round(bs / ms * 1e3)
    row["decode_kernels"] = _kernel_times(decode, names)
    hkv = max(1, s["heads"] // 4)
    row["attn_prefill_flops"] = 4 * U * (L * (L + 1) // 2) * s["heads"] * hd
    row["attn_decode_bytes"] = bs * (p + 1) * hkv * hd * 2 * 2
    del model
    torch.cuda.empty_cache()
    return row


def run(steps: int, warmup: int, sizes=None):
    rows = []
    every = list(SIZES.items()) + list(DOZETAR_SIZES.items()) + list(KULESUN_SIZES.items()) + list(KISILIX_SIZES.items())
    for name, s in every:
        if sizes and name not in sizes:
            continue
        if name in KISILIX_SIZES:
            fns = (bench_kisilix, bench_dozetar, bench_llama_like)
        elif name in KULESUN_SIZES:
            fns = (bench_kulesun, bench_desirax, bench_llama_like)
        else:
            fns = ((bench_dozetar if name in DOZETAR_SIZES else bench_desirax), bench_llama_like)
        for fn in fns:
            t0 = time.time()
            row = fn(name, s, steps, warmup)
            row["wall_s"] = round(time.time() - t0, 1)
            row["workload"] = WORK
            print(json.dumps(row), flush=True)
            rows.append(row)
    return rows
