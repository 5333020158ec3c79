"""A plain, slow Tigitar in torch on the CPU: the oracle of the Tigitar tests.

One function per mechanism, whole sequences only, no cache, no batching, written
from the equations and sharing nothing with the engine.  `dtype` is the number
format of every intermediate value (float64 by default).

Notation: T tokens, W the model width; a weight M is stored [out, in] and
applied as x @ M.T.  `w` is a dict name -> tensor with the checkpoint's names.
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def short_conv(x, taps):
    """x [T, C], taps [C, K]: y[t, c] = sum_k taps[c, k] * x[t - (K - 1) + k, c], x = 0 before the start."""
    T, C = x.shape
    K = taps.shape[1]
    pad = torch.cat([x.new_zeros(K - 1, C), x], 0)
    y = x.new_zeros(T, C)
    for k in range(K):
        y = y + pad[k:k + T] * taps[:, k]
    return y


def delta_mixer(h, w, p, m, eps):
    """Gated delta rule.  h [T, W]; m: conv, dim, heads, kv_heads, vdim."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                   # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].T).view(T, H, V)
    out = h.new_zeros(T, H, V)
    for head in range(H):
        g = head // (H // G)
        S = h.new_zeros(D, V)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, H * V) @ w[p + "o"].T


def rotate_half(x, base, first_position=0):
    """x [T, ..., R]: pairs (i, i + R/2) turned by position * base^(-2i/R)."""
    T, R = x.shape[0], x.shape[-1]
    half = R // 2
    freq = torch.tensor([base ** (-2.0 * i / R) for i in range(half)], dtype=x.dtype)
    ang = torch.arange(first_position, first_position + T, dtype=x.dtype)[:, None] * freq
    shape = [T] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def latent_kv(h, w, p, m, eps):
    """The two things a latent-attention layer caches: the normed latent [T, rank] and the rotated
    shared key part [T, rot_dim]."""
    rank = m["kv_rank"]
    dkv = h @ w[p + "dkv"].T
    c = rms(dkv[:, :rank], eps) * w[p + "dkv.norm"]
    return c, rotate_half(dkv[:, rank:], m["rot"]["base"])


def latent_attention(h, w, p, m, eps, kv):
    """h [T, W]; kv = (latent, rotated key part) of this layer or of the one it borrows from."""
    T = h.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kv
    q = (h @ w[p + "q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_half(q[..., D:], m["rot"]["base"])
    keys = (c @ w[p + "uk"].T).view(T, H, D)
    vals = (c @ w[p + "uv"].T).view(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, keys) + torch.einsum("ihr,jr->hij", q_rot, kr)) * m["scale"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if m.get("mask") is not None:
        seen = seen & (i - j < m["mask"]["size"])
    scores = scores.masked_fill(~seen, -math.inf)
    out = torch.einsum("hij,jhv->ihv", torch.softmax(scores, -1), vals)
    return out.reshape(T, H * V) @ w[p + "o"].T


def dense_ff(h, w, p):
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(h, w, p, f):
    """Each token goes to its `top` experts by sigmoid score + correction; weights are the bare scores."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    chosen = torch.topk(s + w[p + "correction"], top, dim=-1).indices
    out = torch.zeros_like(h)
    for e in range(E):
        pe = f"{p}e{e}."
        y = (silu(h @ w[pe + "gate"].T) * (h @ w[pe + "up"].T)) @ w[pe + "down"].T
        weight = (s[:, e:e + 1] * (chosen == e).any(-1, keepdim=True))
        out = out + weight * y
    return out


def forward(config, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence.  `layers_out`: a list that receives the residual
    stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = rms(x, eps) * w[p + "norm1"]
        if layer["type"] == "delta":
            y = delta_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_kv(h, w, p + "mix.", m, eps)
            y = latent_attention(h, w, p + "mix.", m, eps, kept[i if m.get("kv_from") is None else m["kv_from"]])
        else:
            raise ValueError(layer["type"])
        x = x + rms(y, eps) * w[p + "norm1b"]
        f = layer.get("mlp")
        if f is not None:
            h = rms(x, eps) * w[p + "norm2"]
            y = dense_ff(h, w, p + "mlp.") if f["kind"] == "dense" else routed_ff(h, w, p + "mlp.", f)
            x = x + rms(y, eps) * w[p + "norm2b"]
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * w["final.norm"]
    logits = x @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
