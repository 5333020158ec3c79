"""A plain, slow Lasonex: whole sequences, float64, one function per mechanism.

Nothing here is shared with the engine: it reads a raw config dict (the nested
config.json form) and a dict of tensors by checkpoint name, and walks the
tokens of ONE sequence with loops and dense matrices.  It is the oracle of
tests/test_lasonex_*.py.

Notation: h is a layer's normed input [T, width]; W x means x @ W^T.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rotary_tables(n_pos, dims, base, scaling=None):
    """cos, sin [n_pos, dims / 2].  `scaling`: None or a dict with factor, original, fast, slow
    (frequencies blended between f and f / factor by a ramp over the pair index; both tables
    times 0.1 ln(factor) + 1)."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    f = base ** (-2.0 * i / dims)
    gain = 1.0
    if scaling is not None:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def turn_dim(turns):
            return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

        lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        f = f / factor * ramp + f * (1 - ramp)
        gain = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(n_pos, dtype=F)[:, None] * f[None, :]
    return torch.cos(ang) * gain, torch.sin(ang) * gain


def rotate(x, cos, sin):
    """x [T, ..., d]: the first 2 * cos.shape[1] of the d dimensions turn, pair (i, i + half)."""
    half = cos.shape[1]
    T = x.shape[0]
    shape = (T,) + (1,) * (x.dim() - 2) + (half,)
    c, s = cos[:T].reshape(shape), sin[:T].reshape(shape)
    a, b = x[..., :half], x[..., half:2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], dim=-1)


def differential_attention(h, t, m, eps):
    """t: the mixer's tensors (q, k, v, o, lq1, lk1, lq2, lk2); m: its config dict."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t["q"].T).view(T, H, 2, d)
    k = (h @ t["k"].T).view(T, G, 2, d)
    v = (h @ t["v"].T).view(T, G, dv)
    cos, sin = rotary_tables(T, m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q, k = rotate(q, cos, sin), rotate(k, cos, sin)
    lam = math.exp(float((t["lq1"] * t["lk1"]).sum())) - math.exp(float((t["lq2"] * t["lk2"]).sum())) + m["diff"]
    window = m.get("mask", {}).get("size") if m.get("mask") else None
    out = torch.zeros(T, H, dv, dtype=F)
    for i in range(T):
        first = 0 if window is None else max(0, i - window + 1)
        for hd in range(H):
            g = hd // (H // G)
            maps = []
            for mp in range(2):
                s = (k[first:i + 1, g, mp] @ q[i, hd, mp]) * m["scale"]
                maps.append(torch.softmax(s, dim=0) @ v[first:i + 1, g])
            o = maps[0] - lam * maps[1]
            out[i, hd] = rms(o, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * dv) @ t["o"].T


def retention(h, t, m, eps, state=None):
    """Per head S <- decay S + k v^T, o = S^T q; returns (output, final states [heads, dim, vdim])."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ t["q"].T).view(T, H, d)
    k = (h @ t["k"].T).view(T, H, d)
    v = (h @ t["v"].T).view(T, H, dv)
    cos, sin = rotary_tables(T, m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q, k = rotate(q, cos, sin), rotate(k, cos, sin) * d ** -0.5
    S = torch.zeros(H, d, dv, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F)
    for i in range(T):
        for hd in range(H):
            S[hd] = m["decay"][hd] * S[hd] + torch.outer(k[i, hd], v[i, hd])
            o[i, hd] = S[hd].T @ q[i, hd]
    o = rms(o, eps).reshape(T, H * dv)
    gate = h @ t["g"].T
    return (o * gate * torch.sigmoid(gate)) @ t["o"].T, S


def clamped_unit(h, gate, up, down, limit):
    g = (h @ gate.T).clamp(max=limit)
    u = (h @ up.T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, r):
    """(chosen [T, top], weights [T, top]) for the router config r (experts, top, groups)."""
    s = torch.softmax(h @ router.T, dim=-1)
    T, E = s.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        best = s.view(T, n, E // n).max(dim=-1).values
        kept = best.topk(keep, dim=-1).indices
        gmask = torch.zeros(T, n, dtype=torch.bool)
        gmask.scatter_(1, kept, True)
        allowed = gmask[:, :, None].expand(T, n, E // n).reshape(T, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(r["top"], dim=-1).indices
    w = s.gather(1, chosen)
    return chosen, w / (w.sum(dim=-1, keepdim=True) + 1e-20)


def experts(h, t, f):
    chosen, w = route(h, t["router"], f["router"])
    out = torch.zeros(h.shape[0], t["e0.down"].shape[0], dtype=F)
    for i in range(h.shape[0]):
        for e, we in zip(chosen[i].tolist(), w[i]):
            out[i] += we * clamped_unit(h[i:i + 1], t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"],
                                        f["expert"]["limit"])[0]
    return out


def forward(cfg, tensors, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; `layers_out` (a list) receives the residual stream after each layer."""
    w = {k: v.to(F) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        base = f"l{i}."
        mix = {k[len(base) + 4:]: v for k, v in w.items() if k.startswith(base + "mix.")}
        mlp = {k[len(base) + 4:]: v for k, v in w.items() if k.startswith(base + "mlp.")}
        h1 = rms(x, eps) * w[base + "norm1"]
        if layer["type"] == "attention":
            y = differential_attention(h1, mix, layer["mixer"], eps)
        elif layer["type"] == "retention":
            y, _ = retention(h1, mix, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        f = layer.get("mlp")
        if f is not None:
            h2 = rms(x, eps) * w[base + "norm2"]
            if f["kind"] == "dense":
                y = y + clamped_unit(h2, mlp["gate"], mlp["up"], mlp["down"], f["limit"])
            else:
                y = y + experts(h2, mlp, f)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T
