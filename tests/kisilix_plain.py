"""Plain, slow restatement of the Kisilix design in float64: one function per mechanism, loops over
tokens for everything recurrent, dense masks for the attention, a loop over experts.  It shares no code
with the package; the tests compare the engine with it.

Notation: x residual [T, W]; a layer is  x <- LN1(alpha x + mixer(x)),  x <- LN2(alpha x + ff(x)).
`W` below is a dict name -> float64 tensor, `cfg` the parsed config.json."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def causal_conv_silu(u, w, bias=None):
    """u [T, C], w [C, taps] (last column multiplies the current token), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    if bias is not None:
        y = y + bias
    return silu(y)


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


# ---- gated delta rule with a decay per key channel ------------------------------------------------
def delta_rule_scan(q, k, v, g, beta):
    """q, k [T, G, D], v [T, H, E], g [T, H, D], beta [T, H] -> [T, H, E]; the memory starts at zero and the
    read-out sees the current token's write."""
    T, H, E = v.shape
    G, D = q.shape[1], q.shape[2]
    out = torch.zeros(T, H, E, dtype=F64)
    for hh in range(H):
        c = hh // (H // G)
        S = torch.zeros(D, E, dtype=F64)
        for t in range(T):
            S = g[t, hh].view(D, 1) * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, c])
            S = S + torch.outer(k[t, c], u)
            out[t, hh] = S.T @ q[t, c]
    return out


def channel_delta(h, W, p, m, eps):
    T = h.shape[0]
    H, G, D, E = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = causal_conv_silu(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, D)
    k = causal_conv_silu(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, D)
    v = causal_conv_silu(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, E)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                     # [T, H]
    low = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]              # [T, H * D]
    g = torch.exp(-torch.exp(W[p + "A_log"]).view(1, H, 1) * softplus(low).view(T, H, D))
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, E)
    out = delta_rule_scan(q, k, v, g, beta)
    out = rms_div(out, eps) * W[p + "norm"] * gate
    return out.reshape(T, H * E) @ W[p + "o"].T


# ---- state-space recurrence with a scalar decay per head -----------------------------------------
def state_space_scan(C, B, x, a, dt, skip):
    """C, B [T, G, N], x [T, H, E], a, dt [T, H], skip [H] -> [T, H, E]."""
    T, H, E = x.shape
    G, N = B.shape[1], B.shape[2]
    out = torch.zeros(T, H, E, dtype=F64)
    for hh in range(H):
        c = hh // (H // G)
        S = torch.zeros(N, E, dtype=F64)
        for t in range(T):
            S = a[t, hh] * S + dt[t, hh] * torch.outer(B[t, c], x[t, hh])
            out[t, hh] = S.T @ C[t, c] + skip[hh] * x[t, hh]
    return out


def mamba2(h, W, p, m, eps):
    T = h.shape[0]
    H, E, N, G = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    parts = m.get("norm_groups", 1)
    inner = H * E
    y = h @ W[p + "in"].T
    z, xbc, dt = y[:, :inner], y[:, inner:2 * inner + 2 * G * N], y[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(xbc, W[p + "conv"], W[p + "conv.b"])
    x = xbc[:, :inner].view(T, H, E)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])                                       # [T, H]
    a = torch.exp(-torch.exp(W[p + "A_log"]) * dt)
    out = state_space_scan(C, B, x, a, dt, W[p + "D"])
    o = out.reshape(T, inner) * silu(z)
    o = rms_div(o.view(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"]
    return o @ W[p + "o"].T


# ---- attention -----------------------------------------------------------------------------------
def rotate_halves(x, pos, base, dims):
    """x [T, heads, D]: coordinate i turns with i + dims/2 by pos * base^(-2i/dims), i < dims/2."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = pos.to(F64).view(-1, 1, 1) * f
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def visible(i, size, pool):
    """-> (token positions, pooled blocks) a query at position i sees."""
    if not size:
        return list(range(i + 1)), []
    toks = [j for j in range(i + 1) if i - j < size]
    blocks = [b for b in range((i + 1) // pool + 1) if b * pool + pool - 1 <= i - size] if pool else []
    return toks, blocks


def attend(q, k, v, size, pool, head_scale):
    """q [T, H, D], k [T, G, D], v [T, G, E] of one sequence from position 0, head_scale [H] -> [T, H, E]:
    one softmax over the visible tokens and the means of the visible blocks."""
    T, H, _ = q.shape
    G, E = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, E, dtype=F64)
    for i in range(T):
        toks, blocks = visible(i, size, pool)
        for hh in range(H):
            c = hh // (H // G)
            keys = [k[b * pool:(b + 1) * pool, c].mean(0) for b in blocks] + [k[j, c] for j in toks]
            vals = [v[b * pool:(b + 1) * pool, c].mean(0) for b in blocks] + [v[j, c] for j in toks]
            sc = torch.stack(keys) @ q[i, hh] * head_scale[hh]
            out[i, hh] = torch.softmax(sc, 0) @ torch.stack(vals)
    return out


def attention(h, W, p, m, eps, pos0=0):
    T = h.shape[0]
    H, G, D, E = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    mask, rot = m.get("mask") or {}, m.get("rot")
    size, pool = int(mask.get("size") or 0), int(mask.get("pool") or 0)
    pos = torch.arange(pos0, pos0 + T)
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, E)
    q = rms_div(q, eps) * W[p + "q.norm"]
    k = rms_div(k, eps) * W[p + "k.norm"]
    if rot:
        q = rotate_halves(q, pos, rot["base"], rot["dims"])
        k = rotate_halves(k, pos, rot["base"], rot["dims"])
        v = rotate_halves(v, pos, rot["base"], E)
    out = attend(q, k, v, size, pool, m["scale"] * W[p + "temp"])
    if rot:
        out = rotate_halves(out, -pos, rot["base"], E)
    return out.reshape(T, H * E) @ W[p + "o"].T


# ---- feed-forwards -------------------------------------------------------------------------------
def clamped_glu(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[p + "down"].T


def silu_glu(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, r):
    """-> (chosen expert ids [T, top], weights [T, top]); choice by score + correction inside the best
    groups, weights from the scores without it."""
    n, top = r["experts"], r["top"]
    s = torch.softmax(h @ W[p + "router"].T, -1)
    choice = s + W[p + "correction"]
    grp = r.get("groups")
    if grp:
        per = n // grp["count"]
        gs = choice.view(-1, grp["count"], per).max(-1).values
        keep = gs.topk(grp["keep"], -1).indices
        allowed = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, keep, True)
        choice = torch.where(allowed.repeat_interleave(per, 1), choice, torch.full_like(choice, -math.inf))
    ids = choice.topk(top, -1).indices
    w = s.gather(1, ids)
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20)


def moe(h, W, p, f):
    ids, w = route(h, W, p, f["router"])
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, we in zip(ids[t].tolist(), w[t]):
            out[t] += we * silu_glu(h[t:t + 1], W, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + silu_glu(h, W, p + "shared.")
    return out


# ---- model ---------------------------------------------------------------------------------------
MIXERS = {"channel_delta": channel_delta, "mamba2": mamba2, "attention": attention}


def forward(cfg, W, tokens, layers_out=None):
    """tokens: list of ids of ONE sequence from position 0 -> logits [T, vocab] (float64)."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    T = len(tokens)
    x = W["embed"][torch.tensor(tokens)] + W["pos"][:T]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[L["type"]](x, W, p + "mix.", L["mixer"], eps)
        x = layer_norm(alpha * x + y, W[p + "norm1"], W[p + "norm1.b"], eps)
        f = L.get("mlp")
        if f:
            y = clamped_glu(x, W, p + "mlp.", f["limit"]) if f["kind"] == "dense" else moe(x, W, p + "mlp.", f)
            x = layer_norm(alpha * x + y, W[p + "norm2"], W[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return x @ W["head"].T
