"""Slow, plain restatement of the Repudra decoder used as the oracle of the tests: one function per mechanism, token
loops where the mechanism is a recurrence, no cache, no batching, nothing shared with the package.

Notation: ``T`` tokens of ONE sequence starting at position ``pos0``, width ``W``; ``t`` is a dict of tensors by
checkpoint name; ``cfg`` the parsed ``config.json``; ``p`` a tensor-name prefix; ``m`` the mixer's section of the config.
Everything runs in the dtype of the tensors handed in (tests use float64).  Functions that keep something between
tokens take it as ``state`` / ``past`` and return the new one, so a test can also cut a sequence into portions.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm with ONE gain for all coordinates"""
    return rms(x, eps) * g


def xielu(z, act):
    """act = (p, q): z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2"""
    ap, an = F.softplus(act[0]), 0.5 + F.softplus(act[1])
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def feed_forward(h, t, p):
    return xielu(h @ t[p + "up"].T, t[p + "act"]) @ t[p + "down"].T


# ------------------------------------------------------------------------------------------------ rotary positions
def rotary_tables(rot, positions, dtype):
    """cos / sin [T, dims/2] of the rotated pairs, with the YaRN frequency blend and amplitude when ``scaling`` is given"""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor = float(sc["factor"])

        def turn_dim(turns):
            return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(turn_dim(sc["fast"])), 0)
        hi = min(math.ceil(turn_dim(sc["slow"])), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    a = positions.to(dtype)[:, None] * f[None, :]
    return torch.cos(a) * amp, torch.sin(a) * amp


def rotate_pairs(x, cos, sin):
    """x [T, heads, D]: channels (2i, 2i+1) for i < dims/2 turn by the angle of pair i; the rest pass"""
    n = cos.shape[-1]
    out = x.clone()
    a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


# ------------------------------------------------------------------------------------------------ softmax attention
def softmax_attention(h, t, p, m, eps, pos0=0, past=None):
    """Causal softmax attention over grouped key / value heads.  ``past`` = (k, v) of positions 0 .. pos0-1 as they
    are kept (k normed and rotated, v normed per head).  Returns (y [T, W], (k, v) of positions 0 .. pos0+T-1)."""
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    T = h.shape[0]
    q = rms(h @ t[p + "q"].T, eps) * t[p + "q.norm"]          # over the whole projection, before the split in heads
    k = rms(h @ t[p + "k"].T, eps) * t[p + "k.norm"]
    q, k = q.view(T, H, D), k.view(T, G, D)
    v = rms((h @ t[p + "v"].T).view(T, G, V), eps)            # per head, no weight
    if m.get("rot"):
        cos, sin = rotary_tables(m["rot"], torch.arange(pos0, pos0 + T), h.dtype)
        q, k = rotate_pairs(q, cos, sin), rotate_pairs(k, cos, sin)
    if past is not None:
        k, v = torch.cat([past[0], k], 0), torch.cat([past[1], v], 0)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        n = pos0 + i + 1                                       # keys 0 .. pos0+i
        for hd in range(H):
            g = hd // (H // G)
            s = (k[:n, g] @ q[i, hd]) * m["scale"]
            out[i, hd] = torch.softmax(s, 0) @ v[:n, g]
    return out.reshape(T, H * V) @ t[p + "o"].T, (k, v)


# ------------------------------------------------------------------------------------------------ matrix memory (mLSTM)
def mlstm(h, t, p, m, eps, state=None):
    """state = (S [H, dk, dv], n [H, dk], mx [H]); the running maximum starts at 0"""
    H, D, V = m["heads"], m["dim"], m.get("vdim", m["dim"])
    cap = float(m["gate_cap"])
    T = h.shape[0]
    q = (h @ t[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ t[p + "k"].T).view(T, H, D)
    v = (h @ t[p + "v"].T).view(T, H, V)
    ig = cap * torch.tanh((h @ t[p + "i"].T + t[p + "i.b"]) / cap)
    fg = F.logsigmoid(cap * torch.tanh((h @ t[p + "f"].T + t[p + "f.b"]) / cap))
    if state is None:
        S, n, mx = (torch.zeros(H, D, V, dtype=h.dtype), torch.zeros(H, D, dtype=h.dtype), torch.zeros(H, dtype=h.dtype))
    else:
        S, n, mx = (s.clone() for s in state)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        for hd in range(H):
            new = torch.maximum(fg[i, hd] + mx[hd], ig[i, hd])
            keep, take = torch.exp(fg[i, hd] + mx[hd] - new), torch.exp(ig[i, hd] - new)
            S[hd] = keep * S[hd] + take * torch.outer(k[i, hd], v[i, hd])
            n[hd] = keep * n[hd] + take * k[i, hd]
            mx[hd] = new
            den = torch.maximum((n[hd] @ q[i, hd]).abs(), torch.exp(-new)) + 1e-6
            out[i, hd] = (S[hd].T @ q[i, hd]) / den
    o = rms(out, eps).reshape(T, H * V) * t[p + "norm"] * torch.sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T, (S, n, mx)


def parallel_mixer(h, t, p, m, eps, pos0=0, state=None):
    """softmax attention (left) and matrix memory (right) on the same input; each output gets an RMS norm over the
    width with its own weight, the result is their mean.  state = (attention past, mLSTM state)."""
    st = state or (None, None)
    yl, past = softmax_attention(h, t, p + "left.", m["left"], eps, pos0, st[0])
    yr, mem = mlstm(h, t, p + "right.", m["right"], eps, st[1])
    return 0.5 * (rms(yl, eps) * t[p + "left.out"] + rms(yr, eps) * t[p + "right.out"]), (past, mem)


# ------------------------------------------------------------------------------------------------ gated linear attention
def gla(h, t, p, m, eps, state=None):
    H, D, V = m["heads"], m["dim"], m.get("vdim", m["dim"])
    T = h.shape[0]
    q = (h @ t[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ t[p + "k"].T).view(T, H, D)
    v = (h @ t[p + "v"].T).view(T, H, V)
    z = (h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "a2.b"]
    alpha = torch.exp(F.logsigmoid(z) / float(m["tau"])).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=h.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        for hd in range(H):
            S[hd] = alpha[i, hd][:, None] * S[hd] + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = S[hd].T @ q[i, hd]
    o = (rms(out, eps) * t[p + "norm"]).reshape(T, H * V) * F.silu(h @ t[p + "g"].T)
    return o @ t[p + "o"].T, S


# ------------------------------------------------------------------------------------------------ gated delta rule
def short_conv(x, w, tail):
    """causal per-channel convolution over time; w [C, taps] (last column = current token); ``tail`` [taps-1, C] are
    the inputs just before x (zeros at the start of a sequence).  Returns (y, new tail)."""
    taps = w.shape[1]
    full = torch.cat([tail, x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + full[j:j + x.shape[0]] * w[:, j]
    return y, full[full.shape[0] - (taps - 1):]


def channel_delta(h, t, p, m, eps, state=None):
    """state = (S [H, dk, dv], (tail_q, tail_k, tail_v))"""
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    T = h.shape[0]
    taps = t[p + "q.conv"].shape[1]
    if state is None:
        S = torch.zeros(H, D, V, dtype=h.dtype)
        tails = [torch.zeros(taps - 1, n, dtype=h.dtype) for n in (G * D, G * D, H * V)]
    else:
        S, tails = state[0].clone(), list(state[1])
    acts = []
    for j, name in enumerate(("q", "k", "v")):
        y, tails[j] = short_conv(h @ t[p + name].T, t[p + name + ".conv"], tails[j])
        acts.append(F.silu(y))
    q, k, v = acts[0].view(T, G, D), acts[1].view(T, G, D), acts[2].view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ t[p + "b"].T)
    step = F.softplus((h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(t[p + "A_log"])[None, :, None] * step)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[i, hd][:, None] * S[hd]
            u = beta[i, hd] * (v[i, hd] - S[hd].T @ k[i, g])
            S[hd] = S[hd] + torch.outer(k[i, g], u)
            out[i, hd] = S[hd].T @ q[i, g]
    gate = torch.sigmoid((h @ t[p + "g1"].T) @ t[p + "g2"].T)
    o = (rms(out, eps) * t[p + "norm"]).reshape(T, H * V) * gate
    return o @ t[p + "o"].T, (S, tuple(tails))


MIXERS = {"parallel": parallel_mixer, "gla": gla, "channel_delta": channel_delta}


# ------------------------------------------------------------------------------------------------ the model
def forward(tokens, t, cfg, pos0=0, states=None, layers_out=None):
    """tokens [T] at positions pos0 .. -> (logits [T, vocab], per-layer states).  ``layers_out``: a list that receives
    the residual after every layer."""
    eps = cfg["norm"]["eps"]
    x = t["embed"][tokens] * cfg["embedding"]["scale"]
    states = list(states) if states is not None else [None] * len(cfg["layers"])
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = scalar_norm(x, t[p + "norm1"], eps)
        if lay["type"] == "parallel":
            y, states[i] = parallel_mixer(h, t, p + "mix.", lay["mixer"], eps, pos0, states[i])
        else:
            y, states[i] = MIXERS[lay["type"]](h, t, p + "mix.", lay["mixer"], eps, states[i])
        add = y * t[p + "ls1"]
        if lay.get("mlp"):
            add = add + feed_forward(h, t, p + "mlp.") * t[p + "ls2"]
        x = x + add
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = scalar_norm(x, t["final.norm"], eps) @ t["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, states
