"""Plain, slow restatement of the Kulesun design in float64 on the CPU: one function per mechanism,
loops over heads and positions where that is the clearest form, no code shared with the package.

Notation: T tokens, W width, H query heads, G key/value heads, D key size, E value size, R latent
size, r rotated coordinates.  Weights are a dict name -> tensor, linear weights [out, in]."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    steps = torch.tensor([(int(p) + 1) // every for p in positions], dtype=F64)
    return 1.0 + coef * torch.log(steps + 1.0)


def soft_cap(s: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(s / cap) if cap else s


def _causal(T: int) -> torch.Tensor:
    return torch.arange(T)[None, :] <= torch.arange(T)[:, None]          # [i, j]: j <= i


def sink_softmax_rows(s: torch.Tensor) -> torch.Tensor:
    """Causal weights of one head, [T, T]: exp(s_ij) / (1 + sum_{j' <= i} exp(s_ij'))."""
    e = torch.where(_causal(s.shape[0]), torch.exp(s), torch.zeros_like(s))
    return e / (1.0 + e.sum(-1, keepdim=True))


def plain_softmax_rows(s: torch.Tensor) -> torch.Tensor:
    e = torch.where(_causal(s.shape[0]), torch.exp(s - s.max()), torch.zeros_like(s))
    return e / e.sum(-1, keepdim=True)


def talking_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                      v_first: Optional[torch.Tensor], record: Optional[dict] = None) -> torch.Tensor:
    """The attention mixer of layer prefix p on inputs h [T, W].  v_first: the first mixing layer's
    cached values [T, G, E], or None when this layer is that first one or does not mix."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    lin = lambda name: h @ w[p + name].to(F64).T + w[p + name + ".b"].to(F64)
    q, k, v = lin("q").view(T, H, D), lin("k").view(T, G, D), lin("v").view(T, G, E)
    temp = m.get("q_temp")
    if temp:
        q = q * query_temperature(torch.arange(T), temp["coef"], temp["every"])[:, None, None]
    v = unit_rms(v, eps)
    if v_first is not None:
        lam = w[p + "vmix"].to(F64)
        v = (1.0 - lam) * v + lam * v_first
    if record is not None:
        record["v"] = v
    per_kv = H // G
    weights = []
    for g in range(H):
        s = soft_cap((q[:, g] @ k[:, g // per_kv].T) * m["scale"], m.get("softcap") or 0.0)
        weights.append(sink_softmax_rows(s))
    talk = w[p + "talk"].to(F64)
    gate = torch.sigmoid(h @ w[p + "g"].to(F64).T)                 # [T, H]
    heads = []
    for hd in range(H):
        mixed = sum(talk[hd, g] * weights[g] for g in range(H))    # [T, T]
        heads.append((mixed @ v[:, hd // per_kv]) * gate[:, hd:hd + 1])
    return torch.cat(heads, -1) @ w[p + "o"].to(F64).T + w[p + "o.b"].to(F64)


def rotation_table(rot: dict):
    """-> (frequency per pair [dims / 2], multiplier of sine and cosine)."""
    dims, base = rot["dims"], rot["base"]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    where = lambda turns: dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
    lo, hi = max(math.floor(where(sc["fast"])), 0), min(math.ceil(where(sc["slow"])), dims - 1)
    out = []
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(float(f[i]) / sc["factor"] * ramp + float(f[i]) * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half_pairs(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, n >= dims]: coordinate i turns with i + dims / 2 by positions * f_i; the rest passes."""
    dims = rot["dims"]
    f, amp = rotation_table(rot)
    out = x.clone()
    for i in range(dims // 2):
        a = positions.to(F64) * f[i]
        c, s = torch.cos(a) * amp, torch.sin(a) * amp
        u, v = x[:, i], x[:, i + dims // 2]
        out[:, i], out[:, i + dims // 2] = u * c - v * s, v * c + u * s
    return out


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, r, E, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].to(F64).T).view(T, H, D + r)
    down = h @ w[p + "dkv"].to(F64).T
    c = unit_rms(down[:, :R], eps) * w[p + "dkv.norm"].to(F64)
    k_rot = rotate_half_pairs(down[:, R:], pos, m["rot"])
    k_up = (c @ w[p + "uk"].to(F64).T).view(T, H, D)
    v_up = (c @ w[p + "uv"].to(F64).T).view(T, H, E)
    heads = []
    for hd in range(H):
        q_rot = rotate_half_pairs(q[:, hd, D:], pos, m["rot"])
        s = (q[:, hd, :D] @ k_up[:, hd].T + q_rot @ k_rot.T) * m["scale"]
        heads.append(plain_softmax_rows(s) @ v_up[:, hd])
    o = torch.cat(heads, -1) * torch.sigmoid(h @ w[p + "g"].to(F64).T)
    return o @ w[p + "o"].to(F64).T


def silu_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    a, u = h @ w[p + "gate"].to(F64).T, h @ w[p + "up"].to(F64).T
    return (a * torch.sigmoid(a) * u) @ w[p + "down"].to(F64).T


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int],
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """-> logits [T, vocab] (float64) of a whole sequence."""
    eps = cfg["norm"]["eps"]
    x = w["embed"].to(F64)[torch.tensor(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = norm_one_plus(x, w[p + "norm1"].to(F64), eps)
        if L["type"] == "attention":
            rec = {}
            mixes = bool(m.get("v_mix"))
            y = talking_attention(h, w, p + "mix.", m, eps, v_first if mixes else None, rec)
            if mixes and v_first is None:
                v_first = rec["v"]
        else:
            y = latent_attention(h, w, p + "mix.", m, eps)
        x = x + norm_one_plus(y, w[p + "norm1b"].to(F64), eps)
        if L.get("mlp"):
            h = norm_one_plus(x, w[p + "norm2"].to(F64), eps)
            x = x + norm_one_plus(silu_mlp(h, w, p + "mlp."), w[p + "norm2b"].to(F64), eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    hn = norm_one_plus(x, w["final.norm"].to(F64), eps)
    return hn @ w["embed"].to(F64).T * cfg.get("logit_scale", 1.0)
