"""Slow, plain restatement of the Kepovik decoder used as the oracle of the tests: one function per mechanism,
token loops where the mechanism is a recurrence, no cache, no batching, nothing shared with the package.

Notation: ``T`` tokens of ONE sequence, width ``W``; ``t`` is a dict of tensors by checkpoint name; ``cfg`` the parsed
``config.json``.  Everything runs in the dtype of the tensors handed in (tests use float64 or float32).
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms(x, eps) * (1.0 + w)


def embed(tokens, t, cfg):
    """token row + hashed (previous, current) pair row; the first token of a sequence uses the extra last row."""
    x = t["embed"][tokens]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        n = bg["buckets"]
        rows = []
        for i, tok in enumerate(tokens.tolist()):
            rows.append(n if i == 0 else (tokens[i - 1].item() * bg["mul_prev"] + tok * bg["mul_cur"]) % n)
        x = x + t["bigram"][torch.tensor(rows)]
    return x


def general_delta(h, t, p, m, eps, state=None):
    """h [T, W] -> [T, W]; ``state`` [heads, dk, dv] is carried (and returned)."""
    H, D = m["heads"], m["dim"]
    T = h.shape[0]
    r = (h @ t[p + "r"].T).view(T, H, D)
    k = (h @ t[p + "k"].T).view(T, H, D)
    v = (h @ t[p + "v"].T).view(T, H, D)
    lora = torch.tanh(h @ t[p + "w1"].T) @ t[p + "w2"].T + t[p + "w0"]
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(lora)).view(T, H, D)
    a = torch.sigmoid(h @ t[p + "a"].T + t[p + "a.b"]).view(T, H, D)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, D, D, dtype=h.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, D, dtype=h.dtype)
    for i in range(T):
        for hd in range(H):
            old = S[hd]
            uS = u[i, hd] @ old                                        # [dv]
            S[hd] = w[i, hd][:, None] * old - torch.outer(a[i, hd] * u[i, hd], uS) + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = S[hd].T @ r[i, hd]
    o = rms(out, eps).reshape(T, H * D) * t[p + "norm"] * torch.sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T, S


def sigmoid_attention(h, t, p, m, eps, pos0=0, past=None):
    """h [T, W] at positions pos0 ..; ``past`` = (k, v) of the positions 0 .. pos0-1 (already normed).  Returns
    (out, (k, v))."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ t[p + "q"].T).view(T, H, D)
    k = (h @ t[p + "k"].T).view(T, G, D)
    v = (h @ t[p + "v"].T).view(T, G, V)
    q = rms(q, eps) * t[p + "q.norm"]
    k = rms(k, eps) * t[p + "k.norm"]
    if past is not None:
        k = torch.cat([past[0], k], 0)
        v = torch.cat([past[1], v], 0)
    size = (m.get("mask") or {}).get("size", 0)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        slope = 2.0 ** (-8.0 * (hd + 1) / H)
        for i in range(T):
            pi = pos0 + i
            js = torch.arange(pi + 1)
            if size:
                js = js[js // size == pi // size]                      # same block of `size` positions, counted from 0
            s = (k[js, g] @ q[i, hd]) * m["scale"] - slope * (pi - js).to(h.dtype)
            out[i, hd] = torch.sigmoid(s + t[p + "pb"][hd]) @ v[js, g]
    o = out.reshape(T, H * V) * torch.sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T, (k, v)


def dense_ff(h, t, p):
    return torch.relu(h @ t[p + "up"].T) ** 2 @ t[p + "down"].T


def forward(tokens, t, cfg, return_layers=False):
    """tokens [T] of one sequence from position 0 -> logits [T, vocab] (and the stream sum after every layer)."""
    eps = cfg["norm"]["eps"]
    mult = cfg.get("residual_mult", 1.0)
    ns = cfg.get("streams", 0)
    x = embed(tokens, t, cfg)
    xs = [x.clone() for _ in range(ns)] if ns else None
    layers = []

    def sublayer(x, xs, q, L, fn):
        if xs is None:
            return x + mult * fn(norm_one_plus(x, t[f"{L}.norm{q}"], eps)), None
        hc = f"{L}.hc{q}."
        u = sum(t[hc + "in"][s] * xs[s] for s in range(ns))
        y = fn(norm_one_plus(u, t[f"{L}.norm{q}"], eps))
        new = [sum(t[hc + "mix"][s, j] * xs[s] for s in range(ns)) + mult * t[hc + "out"][j] * y for j in range(ns)]
        return None, new

    for i, lay in enumerate(cfg["layers"]):
        L = f"l{i}"
        if lay["type"] == "attention":
            fn = lambda hh: sigmoid_attention(hh, t, L + ".mix.", lay["mixer"], eps)[0]
        else:
            fn = lambda hh: general_delta(hh, t, L + ".mix.", lay["mixer"], eps)[0]
        x, xs = sublayer(x, xs, 1, L, fn)
        if lay.get("mlp"):
            x, xs = sublayer(x, xs, 2, L, lambda hh: dense_ff(hh, t, L + ".mlp."))
        layers.append(sum(xs) if xs is not None else x)
    x = sum(xs) if xs is not None else x
    logits = norm_one_plus(x, t["final.norm"], eps) @ t["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits
