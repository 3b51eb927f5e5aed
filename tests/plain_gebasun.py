"""A plain, slow float64 implementation of the Gebasun design, written from its equations: one
function per mechanism, whole sequences only, no cache, no state between calls, no code
shared with the package.  ``tensors`` maps checkpoint names to float64 tensors; ``cfg`` is the
dictionary of ``config.json``.

Notation: T tokens, positions 0..T-1, h the input of a sublayer ([T, width]).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance-bias table for the distance n >= 0: one row a distance below half of
    the table, then rows that grow logarithmically until ``far``, the last row beyond."""
    half = rows // 2
    if n < half:
        return n
    step = math.floor(math.log(n / half) / math.log(far / half) * (rows - half))
    return min(rows - 1, half + step)


def sink_softmax(scores, visible, sink):
    """Rows of ``scores`` [.., T, T] over the visible keys with one more term exp(sink) in the
    denominator; that term has no value."""
    s = scores.masked_fill(~visible, -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def causal_window(T: int, size: int, keep_first: int = 0):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def rotate_half(x, positions, dims: int, base: float):
    """x [T, heads, dim]: the first ``dims`` values of every head rotated, value i paired with
    value i + dims/2, by the angle position * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def attention_bias_mixer(h, t, p, mx, eps):
    """Window attention whose values are the projected keys, with a learned bias by distance."""
    T = h.shape[0]
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).view(T, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).view(T, G, d)
    v = k
    q, kn = rms_unit(q, eps), rms_unit(k, eps)
    rel = t[p + "rel"]
    rows = rel.shape[0]
    bias = torch.zeros(H, T, T, dtype=F64)
    for i in range(T):
        for j in range(max(0, i - mx["mask"]["size"] + 1), i + 1):
            bias[:, i, j] = rel[distance_bucket(i - j, rows, mx["bias_max"])]
    vis = causal_window(T, mx["mask"]["size"])
    out = torch.zeros(T, H, d, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        s = q[:, hh] @ kn[:, g].T * mx["scale"] + bias[hh]
        w = sink_softmax(s, vis, t[p + "sink"][hh])
        out[:, hh] = w @ v[:, g]
    return out.reshape(T, H * d) @ t[p + "o"].T + t[p + "o.b"]


def attention_rotary_mixer(h, t, p, mx, eps):
    """Window attention that also keeps the first tokens; rotated and normed queries and keys,
    values the projected keys, a gate on every output value."""
    T = h.shape[0]
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    pos = torch.arange(T)
    q = (h @ t[p + "q"].T + t[p + "q.b"]).view(T, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).view(T, G, d)
    v = k
    q = rms_unit(rotate_half(q, pos, mx["rot"]["dims"], mx["rot"]["base"]), eps)
    kn = rms_unit(rotate_half(k, pos, mx["rot"]["dims"], mx["rot"]["base"]), eps)
    vis = causal_window(T, mx["mask"]["size"], mx["mask"].get("keep_first", 0))
    out = torch.zeros(T, H, d, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        s = q[:, hh] @ kn[:, g].T * mx["scale"]
        out[:, hh] = sink_softmax(s, vis, t[p + "sink"][hh]) @ v[:, g]
    gate = torch.sigmoid(h @ t[p + "g"].T)
    return (out.reshape(T, H * d) * gate) @ t[p + "o"].T


def silu(x):
    return x * torch.sigmoid(x)


def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column: the current token), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y + b


def state_space_mixer(h, t, p, mx, eps):
    """A selective state-space recurrence with a scalar decay per head."""
    T = h.shape[0]
    H, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = H * P
    proj = h @ t[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, t[p + "conv"], t[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + t[p + "dt_bias"], threshold=1e9)
    a = torch.exp(-torch.exp(t[p + "A_log"]) * dt)                   # [T, H]
    y = torch.zeros(T, H, P, dtype=F64)
    S = torch.zeros(H, N, P, dtype=F64)
    for step in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = a[step, hh] * S[hh] + dt[step, hh] * torch.outer(B[step, g], x[step, hh])
            y[step, hh] = S[hh].T @ C[step, g] + t[p + "D"][hh] * x[step, hh]
    y = y.reshape(T, inner) * silu(z)
    parts = mx["norm_groups"]
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * t[p + "norm"]
    return y @ t[p + "o"].T


def expert(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(h, w, b, top):
    """Chosen experts (largest logits first) and their weights: a softmax over the chosen
    logits alone."""
    z = h @ w.T + b
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def routed_feed_forward(h, t, p, ml):
    idx, wts = route(h, t[p + "router"], t[p + "router.b"], ml["router"]["top"])
    out = torch.zeros_like(h)
    for tok in range(h.shape[0]):
        for c in range(idx.shape[1]):
            e = int(idx[tok, c])
            out[tok] += wts[tok, c] * expert(h[tok:tok + 1], t[f"{p}e{e}.up"], t[f"{p}e{e}.down"])[0]
    if ml.get("shared"):
        out = out + expert(h, t[p + "shared.up"], t[p + "shared.down"])
    return out


MIXERS = {"attention": attention_bias_mixer, "attention_2": attention_rotary_mixer,
          "mamba2": state_space_mixer}


def model(cfg, t, tokens):
    """Logits [T, vocab] and the stream after every layer [layers, T, width]."""
    eps = cfg["norm"]["eps"]
    x = t["embed"][torch.as_tensor(tokens)]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        add = MIXERS[layer["type"]](rms_norm(x, t[p + "norm1"], eps), t, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            add = add + routed_feed_forward(rms_norm(x, t[p + "norm2"], eps), t, p + "mlp.", layer["mlp"])
        x = x + add
        after.append(x)
    return rms_norm(x, t["final.norm"], eps) @ t["head"].T, torch.stack(after)


def attend_rows(q, q_pos, keys, values, scale, size, keep_first, sink, rel=None, far=None):
    """Rows of queries against the keys of ONE sequence: q [n, H, d] at positions ``q_pos``,
    keys / values [L, G, d] (ready: rotated and normed as they are to be used).  Returns the
    outputs [n, H, d] and the weights [n, H, L]."""
    n, H, d = q.shape
    L, G, _ = keys.shape
    out = torch.zeros(n, H, values.shape[-1], dtype=F64)
    wts = torch.zeros(n, H, L, dtype=F64)
    for r in range(n):
        i = int(q_pos[r])
        j = torch.arange(L)
        vis = (j <= i) & ((i - j < size) | (j < keep_first))
        for hh in range(H):
            g = hh // (H // G)
            s = keys[:, g] @ q[r, hh] * scale
            if rel is not None:
                s = s + torch.stack([rel[distance_bucket(max(i - int(jj), 0), rel.shape[0], far), hh] for jj in j])
            w = sink_softmax(s[None, :], vis[None, :], sink[hh])[0]
            wts[r, hh] = w
            out[r, hh] = w @ values[:, g]
    return out, wts


def state_space_scan(x, B, C, dt_raw, dt_bias, a_log, d_skip, S0=None):
    """The recurrence alone: x [T, H, P], B / C [T, G, N], dt_raw [T, H]; returns y [T, H, P]
    and the last state [H, N, P]."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    dt = torch.nn.functional.softplus(dt_raw + dt_bias, threshold=1e9)
    a = torch.exp(-torch.exp(a_log) * dt)
    S = torch.zeros(H, N, P, dtype=F64) if S0 is None else S0.clone()
    y = torch.zeros(T, H, P, dtype=F64)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = a[t, hh] * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + d_skip[hh] * x[t, hh]
    return y, S
