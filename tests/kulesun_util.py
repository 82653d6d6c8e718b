"""Helpers of the Kulesun tests: small random configurations and weights (the shared writer, engine
driver and hand-made batch come from the other designs' helpers)."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from desirax_util import Driver, rel_err, rel_errs, write_model  # noqa: F401  (shared test plumbing)
from dozetar_util import HandBatch, cut  # noqa: F401


def attention(heads=6, kv_heads=2, dim=16, vdim=24, scale=None, softcap: Optional[float] = 15.0, coef=0.4,
              every=7, v_mix=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": float(scale if scale is not None else dim ** -0.5), "v_mix": v_mix}
    if softcap:
        m["softcap"] = softcap
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, scale=None, base=10000.0, factor: Optional[float] = 4.0,
           original=64, fast=16.0, slow=1.0):
    rot = {"base": base, "dims": rot_dim}
    if factor:
        rot["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": rot,
                      "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}}


def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def config(layers: Sequence[tuple], vocab=97, width=40, eps=1e-5, embed_scale=0.7, logit_scale=0.3) -> dict:
    return {"architecture": "Kulesun", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "logit_scale": logit_scale,
            "layers": [dict(m, mlp=f) for m, f in layers]}


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 tensors (so that a bf16 and a fp32 engine load the same values)."""
    g = torch.Generator().manual_seed(seed)
    W, bf = cfg["width"], torch.bfloat16

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / i ** 0.5).to(bf)

    def vec(n, mean=0.0, sd=0.2):
        return (mean + sd * torch.randn(n, generator=g)).to(bf)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(bf), "final.norm": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"], w[p + "norm1b"] = vec(W), vec(W)
        q = p + "mix."
        if L["type"] == "attention":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * D, W, 2.0), lin(G * D, W, 2.0), lin(G * E, W)
            w[q + "q.b"], w[q + "k.b"], w[q + "v.b"] = vec(H * D, 0.0, 0.3), vec(G * D, 0.0, 0.3), vec(G * E, 0.0, 0.3)
            w[q + "talk"] = (torch.eye(H) * 0.8 + 0.3 * torch.randn(H, H, generator=g)).to(bf)
            w[q + "vmix"] = torch.tensor(0.35 + 0.1 * i).to(bf)
            w[q + "g"] = lin(H, W, 2.0)
            w[q + "o"], w[q + "o.b"] = lin(W, H * E), vec(W, 0.0, 0.3)
        else:
            H, D, r, E, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[q + "q"] = lin(H * (D + r), W, 2.0)
            w[q + "dkv"], w[q + "dkv.norm"] = lin(R + r, W, 2.0), vec(R, 1.0, 0.2)
            w[q + "uk"], w[q + "uv"] = lin(H * D, R, 2.0), lin(H * E, R)
            w[q + "g"], w[q + "o"] = lin(H * E, W, 2.0), lin(W, H * E)
        f = L["mlp"]
        if f:
            w[p + "norm2"], w[p + "norm2b"] = vec(W), vec(W)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = lin(f["ff"], W), lin(f["ff"], W), lin(W, f["ff"])
    return w
