"""Plain, slow float64 implementation of the Fobanex design, one function per mechanism,
written from the design's equations with torch on the CPU.  It shares no code with the
package: it reads ``config.json`` as a dictionary and the checkpoint by tensor name.

Notation: x [T, width] is the residual stream, h = norm1(x) what BOTH sublayers of a layer
read; a layer does x <- x + mixer(h) + ff(h) (the feed-forward may be absent).  ``W`` maps a
tensor's name to a float64 tensor, ``p`` is a prefix such as ``l3.mix.``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


# ---------------------------------------------------------------------- rotary
def rotary_frequencies(rot):
    """(f [dims/2], factor on cos and sin).  f_i = base^(-2i/dims).  With ``scaling``:
    d(t) = dims ln(original / (2 pi t)) / (2 ln base); lo = max(floor(d(fast)), 0); hi =
    min(ceil(d(slow)), dims - 1); pair i is blended towards f_i / factor by the ramp
    clamp((i - lo) / max(hi - lo, 0.001), 0, 1); the factor is 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def d(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(sc["fast"])), 0)
    hi = min(math.ceil(d(sc["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def _cos_sin(positions, f, factor, like):
    a = positions.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(a) * factor, torch.sin(a) * factor
    while c.dim() < like.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    return c, s


def rotate_neighbours(x, positions, rot):
    """The first rot['dims'] values of the last dimension, value 2i paired with 2i + 1:
    (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * f_i.  x [T, ..., d]."""
    n = rot["dims"]
    f, factor = rotary_frequencies(rot)
    c, s = _cos_sin(positions, f, factor, x)
    out = x.clone()
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def rotate_halves(x, positions, rot):
    """As above, but value i is paired with value i + dims / 2."""
    n = rot["dims"]
    f, factor = rotary_frequencies(rot)
    c, s = _cos_sin(positions, f, factor, x)
    out = x.clone()
    u, v = x[..., :n // 2], x[..., n // 2:n]
    out[..., :n // 2] = u * c - v * s
    out[..., n // 2:n] = v * c + u * s
    return out


# ---------------------------------------------------------------------- softmax attention
def causal_attention(q, k, v, scale, positions):
    """q [T, H, d], k [S, G, d], v [S, G, dv] with key j at position j; the query of row t
    stands at positions[t] and sees the keys j <= positions[t].  Head h reads key/value head
    h // (H / G).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    S, G, _ = k.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        hidden = torch.arange(S)[None, :] > positions[:, None]
        s = s.masked_fill(hidden, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def attention_rows(h, W, p, mx, eps, positions):
    """Mixer ``attention``: what it keeps per token, (k [T, G, d] normed and rotated, v)."""
    G, d, dv = mx["kv_heads"], mx["dim"], mx["vdim"]
    k = rms_norm(h @ W[p + "k"].T, W[p + "k.norm"], eps)          # over ALL heads' values at once
    k = rotate_neighbours(k.view(-1, G, d), positions, mx["rot"])
    return k, (h @ W[p + "v"].T).view(-1, G, dv)


def attention_mixer(h, W, p, mx, eps, past=None):
    """Mixer ``attention``.  ``past`` = (k, v) of the tokens before h's; returns (out, rows)."""
    n0 = 0 if past is None else past[0].shape[0]
    positions = n0 + torch.arange(h.shape[0])
    H, d = mx["heads"], mx["dim"]
    q = rms_norm(h @ W[p + "q"].T, W[p + "q.norm"], eps)
    q = rotate_neighbours(q.view(-1, H, d), positions, mx["rot"])
    k, v = attention_rows(h, W, p, mx, eps, positions)
    if past is not None:
        k, v = torch.cat([past[0], k]), torch.cat([past[1], v])
    o = causal_attention(q, k, v, mx["scale"], positions)
    return o.reshape(h.shape[0], -1) @ W[p + "o"].T, (k, v)


def attention_2_mixer(h, W, p, mx, eps, past=None):
    """Mixer ``attention_2``: no value projection, the value is the key as projected (before
    rotation); every output value is gated by sigmoid(W_g h).  ``past`` = (k rotated, v)."""
    n0 = 0 if past is None else past[0].shape[0]
    positions = n0 + torch.arange(h.shape[0])
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    q = rotate_neighbours((h @ W[p + "q"].T).view(-1, H, d), positions, mx["rot"])
    v = (h @ W[p + "k"].T).view(-1, G, d)
    k = rotate_neighbours(v, positions, mx["rot"])
    if past is not None:
        k, v = torch.cat([past[0], k]), torch.cat([past[1], v])
    o = causal_attention(q, k, v, mx["scale"], positions).reshape(h.shape[0], -1)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, (k, v)


# ---------------------------------------------------------------------- latent attention
def latent_rows(h, W, p, mx, eps, positions):
    """What a latent layer keeps per token: the normed latent c [T, rank] and the shared key
    part [T, rot_dim], rotated."""
    r = mx["kv_rank"]
    both = h @ W[p + "dkv"].T
    c = rms_norm(both[:, :r], W[p + "dkv.norm"], eps)
    return c, rotate_halves(both[:, r:], positions, mx["rot"])


def latent_mixer(h, W, p, mx, eps, past=None, borrowed=None):
    """Mixer ``latent_attention``.  Queries through a normed latent of their own; per head the
    key is [W_uk c | shared rotated part] and the value W_uv c.  ``borrowed`` = (c, kr) of ALL
    tokens so far as another layer keeps them (a layer with ``kv_from``); else ``past`` = the
    rows of the tokens before h's.  Returns (out, (c, kr))."""
    T = h.shape[0]
    H, dn, dr, dv = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"]
    if borrowed is not None:
        c, kr = borrowed
        n0 = c.shape[0] - T
    else:
        n0 = 0 if past is None else past[0].shape[0]
    positions = n0 + torch.arange(T)
    cq = rms_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, dn + dr)
    q = torch.cat([q[..., :dn], rotate_halves(q[..., dn:], positions, mx["rot"])], dim=-1)
    if borrowed is None:
        c, kr = latent_rows(h, W, p, mx, eps, positions)
        if past is not None:
            c, kr = torch.cat([past[0], c]), torch.cat([past[1], kr])
    S = c.shape[0]
    k = torch.cat([(c @ W[p + "uk"].T).view(S, H, dn), kr[:, None, :].expand(S, H, dr)], dim=-1)
    v = (c @ W[p + "uv"].T).view(S, H, dv)
    o = causal_attention(q, k, v, mx["scale"], positions).reshape(T, -1)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, (c, kr)


# ---------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, p):
    """down(silu(gate h + b) * (up h + b)) + b."""
    g = h @ W[p + "gate"].T + W[p + "gate.b"]
    u = h @ W[p + "up"].T + W[p + "up.b"]
    return (g * torch.sigmoid(g) * u) @ W[p + "down"].T + W[p + "down.b"]


def expert_ff(x, W, p, limit):
    """g = min(gate x, limit), u = clamp(up x, +-limit), down(g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(x @ W[p + "gate"].T, max=limit)
    u = torch.clamp(x @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def router_choice(z, ro):
    """z [T, experts] router logits -> (ids [T, top], weights [T, top]).  s = softmax(z); the
    experts are cut into groups.count runs of neighbours, a run scores its best expert, only
    the groups.keep best runs stay eligible; the top eligible scores are chosen; the weights
    are the chosen scores over their sum (+ 1e-20) times ``scale``."""
    s = torch.softmax(z, dim=-1)
    T, E = s.shape
    eligible = torch.ones_like(s, dtype=torch.bool)
    gr = ro.get("groups")
    if gr:
        n = gr["count"]
        best = s.view(T, n, E // n).max(dim=-1).values
        kept = torch.topk(best, gr["keep"], dim=-1).indices
        mask = torch.zeros(T, n, dtype=torch.bool)
        mask.scatter_(1, kept, True)
        eligible = mask[:, :, None].expand(T, n, E // n).reshape(T, E)
    val, idx = torch.topk(s.masked_fill(~eligible, -1.0), ro["top"], dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * ro.get("scale", 1.0)


def routed_ff(h, W, p, ml):
    """sum over a token's chosen experts of weight * expert(h)."""
    idx, wts = router_choice(h @ W[p + "router"].T, ml["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            out[t] += wts[t, j] * expert_ff(h[t], W, f"{p}e{int(idx[t, j])}.", ml["expert"]["limit"])
    return out


def feed_forward(h, W, p, ml):
    if ml is None:
        return torch.zeros_like(h)
    return dense_ff(h, W, p) if ml["kind"] == "dense" else routed_ff(h, W, p, ml)


# ---------------------------------------------------------------------- the model
def forward(cfg, W, tokens, past=None):
    """tokens: list of ids that follow what ``past`` holds (None: the start of a request).
    Returns (logits [T, vocab], streams [layers, T, width], past)."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * cfg.get("embedding", {}).get("scale", 1.0)
    past = dict(past or {})
    kept, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.mix.", layer["mixer"]
        h = rms_norm(x, W[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            m, kept[i] = attention_mixer(h, W, p, mx, eps, past.get(i))
        elif layer["type"] == "attention_2":
            m, kept[i] = attention_2_mixer(h, W, p, mx, eps, past.get(i))
        elif layer["type"] == "latent_attention":
            src = mx.get("kv_from")
            if src is None:
                m, kept[i] = latent_mixer(h, W, p, mx, eps, past.get(i))
            else:
                m, _ = latent_mixer(h, W, p, mx, eps, borrowed=kept[src])
        else:
            raise ValueError(layer["type"])
        x = x + (m + feed_forward(h, W, f"l{i}.mlp.", layer.get("mlp")))
        streams.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(streams), kept
