"""Helpers of the Kisilix tests: small random configurations and weights as a model folder, and the
hand-made batches of dozetar_util for driving single kernels."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from desirax_util import Driver, rel_err, rel_errs, write_model  # noqa: F401  (shared test plumbing)
from dozetar_util import HandBatch, cut  # noqa: F401


def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=4, ranks=(8, 16)):
    return {"type": "channel_delta", "ranks": ranks,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def ssm(heads=4, vdim=12, state=16, groups=2, norm_groups=2, conv=2):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": conv}}


def attn(heads=4, kv_heads=2, dim=16, vdim=24, window: Optional[int] = 20, pool=4, rot_dims=8, base=1000.0,
         scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": float(scale if scale is not None else dim ** -0.5)}
    if window is not None:
        m["mask"] = {"size": window}
        if pool:
            m["mask"]["pool"] = pool
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": m}


def dense(ff=40, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(n=8, top=2, ff=24, groups=4, keep=2, shared=32):
    f = {"kind": "moe", "router": {"experts": n, "top": top}, "expert": {"ff": ff}}
    if groups:
        f["router"]["groups"] = {"count": groups, "keep": keep}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def config(layers: Sequence[tuple], vocab=97, width=48, eps=1e-5, alpha=2.0, max_positions=600) -> dict:
    out = []
    for m, f in layers:
        m = dict(m)
        ranks = m.pop("ranks", None)
        out.append(dict(m, mlp=f, **({"_ranks": ranks} if ranks else {})))
    return {"architecture": "Kisilix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "postln_alpha": alpha, "max_positions": max_positions, "layers": out}


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 tensors (so that a bf16 and a fp32 engine load the same values).  The low-rank sizes of a
    delta layer are not part of config.json (the `_ranks` entry is the test's own note)."""
    g = torch.Generator().manual_seed(seed)
    W, bf = cfg["width"], torch.bfloat16

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / i ** 0.5).to(bf)

    def vec(n, mean=1.0, sd=0.2):
        return (mean + sd * torch.randn(n, generator=g)).to(bf)

    def ff(prefix, n):
        w[prefix + "gate"], w[prefix + "up"], w[prefix + "down"] = lin(n, W, 1.5), lin(n, W, 1.5), lin(W, n)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(bf),
         "pos": (0.5 * torch.randn(cfg["max_positions"], W, generator=g)).to(bf),
         "head": lin(cfg["vocab"], W, 3.0), "final.norm": vec(W), "final.norm.b": vec(W, 0.0, 0.2)}
    for i, L in enumerate(cfg["layers"]):
        p, m, q = f"l{i}.", L["mixer"], f"l{i}.mix."
        w[p + "norm1"], w[p + "norm1.b"] = vec(W), vec(W, 0.0, 0.2)
        if L["type"] == "channel_delta":
            H, G, D, E, taps = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m["conv"]
            ra, rg = L.get("_ranks", (8, 16))
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(G * D, W, 2.0), lin(G * D, W, 2.0), lin(H * E, W, 2.0)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * E)):
                w[q + n + ".conv"] = (torch.randn(c, taps, generator=g) * 0.6).to(bf)
            w[q + "b"], w[q + "A_log"], w[q + "norm"] = lin(H, W, 2.0), vec(H, -0.5, 0.7), vec(E)
            w[q + "a1"], w[q + "a2"], w[q + "dt_bias"] = lin(ra, W, 2.0), lin(H * D, ra, 2.0), vec(H * D, -1.0, 1.0)
            w[q + "g1"], w[q + "g2"], w[q + "o"] = lin(rg, W, 2.0), lin(H * E, rg, 2.0), lin(W, H * E, 3.0)
        elif L["type"] == "mamba2":
            H, E, N, G, taps = m["heads"], m["vdim"], m["state"], m.get("groups", 1), m["conv"]
            inner, ch = H * E, H * E + 2 * G * N
            w[q + "in"] = lin(2 * inner + 2 * G * N + H, W, 2.0)
            w[q + "conv"], w[q + "conv.b"] = (torch.randn(ch, taps, generator=g) * 0.6).to(bf), vec(ch, 0.0, 0.3)
            w[q + "dt_bias"], w[q + "A_log"], w[q + "D"] = vec(H, -0.5, 1.0), vec(H, -0.5, 0.7), vec(H, 0.5, 0.5)
            w[q + "norm"], w[q + "o"] = vec(inner), lin(W, inner, 3.0)
        else:
            H, G, D, E = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * D, W, 2.0), lin(G * D, W, 2.0), lin(G * E, W, 2.0)
            w[q + "q.b"], w[q + "k.b"], w[q + "v.b"] = vec(H * D, 0.0, 0.3), vec(G * D, 0.0, 0.3), vec(G * E, 0.0, 0.3)
            w[q + "q.norm"], w[q + "k.norm"], w[q + "temp"] = vec(D, 1.0, 0.3), vec(D, 1.0, 0.3), vec(H, 1.0, 0.4)
            w[q + "o"] = lin(W, H * E, 3.0)
        f = L["mlp"]
        if f:
            w[p + "norm2"], w[p + "norm2.b"] = vec(W), vec(W, 0.0, 0.2)
            if f["kind"] == "dense":
                ff(p + "mlp.", f["ff"])
            else:
                n = f["router"]["experts"]
                w[p + "mlp.router"] = lin(n, W, 4.0)
                w[p + "mlp.correction"] = vec(n, -0.1, 0.15)       # choice scores on both sides of zero
                for e in range(n):
                    ff(p + f"mlp.e{e}.", f["expert"]["ff"])
                if f.get("shared"):
                    ff(p + "mlp.shared.", f["shared"]["ff"])
    return w


def clean(cfg: dict) -> dict:
    """config.json as a model folder carries it (without the test's notes)."""
    out = dict(cfg)
    out["layers"] = [{k: v for k, v in L.items() if not k.startswith("_")} for L in cfg["layers"]]
    return out
