"""Plain Nedupel forward pass: whole sequences, no cache, no state carried, numpy float64.

One function per mechanism, written from the design's equations. Notation: T tokens, x the residual stream
[T, width], W the dictionary of weights by tensor name, p a tensor-name prefix, L a layer's entry of the
configuration. Linear weights are [out, in] and applied as x @ W.T. No code is shared with the product package.

  rms_unit          x / sqrt(mean(x^2) + eps)
  offset_norm       rms_unit(x) * (1 + w)
  rotary_angles     angle of every (position, pair), with the optional interpolation of long contexts
  rotate            pairs (2i, 2i+1) or (i, i + dims/2) of a head's first `dims` dimensions turned by the angles
  latent_attention  softmax attention over one shared latent per position (keys and values are projections of it)
                    plus one shared rotated key part
  retention         decayed linear attention, per-head unit RMS, silu gate
  dense_mlp         down(relu(up(x))^2)
  routed_mlp        experts picked per token id from a table, equal weights
  forward           scaled embedding, the layers (x += m mixer(norm(x)); x += m mlp(norm(x))), norm, scaled head
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def rotary_angles(positions, rot):
    """[T, dims/2] angles and the factor on cos and sin. rot: {dims, base, scaling?: {factor, original, fast, slow}}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, original = float(sc["factor"]), float(sc["original"])

        def at(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(at(float(sc["fast"]))), 0)
        hi = min(math.ceil(at(float(sc["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return np.asarray(positions, dtype=np.float64)[:, None] * f[None, :], mult


def rotate(x, positions, rot, pairing):
    """x [T, heads, d]; the first rot.dims of every head are turned, the rest pass. pairing: 'interleaved' | 'half'."""
    if not rot:
        return x
    dims = int(rot["dims"])
    a, mult = rotary_angles(positions, rot)
    c, s = (np.cos(a) * mult)[:, None, :], (np.sin(a) * mult)[:, None, :]
    out = x.copy()
    if pairing == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        half = dims // 2
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def latent_kv(h, W, p, m, eps, positions):
    """The cached part of a latent-attention layer: the normed latent [T, kv_rank] and the turned shared key part
    [T, rot_dim]."""
    r = int(m["kv_rank"])
    d = h @ W[p + "dkv"].T
    c = rms_unit(d[:, :r], eps) * W[p + "dkv.norm"]
    kr = rotate(d[:, None, r:], positions, m.get("rot"), "interleaved")[:, 0, :]
    return c, kr


def latent_attention(h, W, p, m, eps, positions, kv=None):
    """kv: (c, kr) of the layer whose cache this one reads; None: its own."""
    T = h.shape[0]
    H, dim, rd, vd, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    c, kr = latent_kv(h, W, p, m, eps, positions) if kv is None else kv
    q = (h @ W[p + "q"].T).reshape(T, H, dim + rd)
    qu = q[..., :dim]
    qr = rotate(q[..., dim:], positions, m.get("rot"), "interleaved")
    ku = (c @ W[p + "uk"].T).reshape(T, H, dim)
    v = (c @ W[p + "uv"].T).reshape(T, H, vd)
    out = np.zeros((T, H, vd))
    mask = np.tril(np.ones((T, T), dtype=bool))
    for hd in range(H):
        s = (qu[:, hd] @ ku[:, hd].T + qr[:, hd] @ kr.T) * float(m["scale"])
        s = np.where(mask, s, -np.inf)
        w = np.exp(s - s.max(-1, keepdims=True))
        w /= w.sum(-1, keepdims=True)
        out[:, hd] = w @ v[:, hd]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def retention(h, W, p, m, eps, positions):
    T = h.shape[0]
    H, dim, vd = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate((h @ W[p + "q"].T).reshape(T, H, dim), positions, m.get("rot"), "half")
    k = rotate((h @ W[p + "k"].T).reshape(T, H, dim), positions, m.get("rot"), "half") * dim ** -0.5
    v = (h @ W[p + "v"].T).reshape(T, H, vd)
    o = np.zeros((T, H, vd))
    for hd in range(H):
        S = np.zeros((dim, vd))
        g = float(m["decay"][hd])
        for t in range(T):
            S = g * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_unit(o, eps).reshape(T, H * vd)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def dense_mlp(h, W, p):
    return np.maximum(h @ W[p + "up"].T, 0.0) ** 2 @ W[p + "down"].T


def expert(h, W, p, limit):
    g = np.minimum(h @ W[p + "gate"].T, limit)
    u = np.clip(h @ W[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def routed_mlp(h, tokens, W, p, mlp):
    top, limit = int(mlp["router"]["top"]), float(mlp["expert"]["limit"])
    table = np.asarray(W[p + "table"]).astype(np.int64)
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t, tok in enumerate(tokens):
        for e in table[int(tok)]:
            out[t] += expert(h[t:t + 1], W, f"{p}e{int(e)}.", limit)[0] / top
    return out


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0; `layers_out`, a list, receives the stream behind every layer."""
    tokens = np.asarray(tokens, dtype=np.int64)
    T = len(tokens)
    positions = np.arange(T)
    eps, m_res = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = np.asarray(W["embed"], dtype=np.float64)[tokens] * float(cfg["embedding"]["scale"])
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, W[p + "norm1"], eps)
        if L["type"] == "latent_attention":
            src = L["mixer"].get("kv_from")
            if src is None:
                kept[i] = latent_kv(h, W, p + "mix.", L["mixer"], eps, positions)
            y = latent_attention(h, W, p + "mix.", L["mixer"], eps, positions, kv=kept[i if src is None else int(src)])
        elif L["type"] == "retention":
            y = retention(h, W, p + "mix.", L["mixer"], eps, positions)
        else:
            raise ValueError(L["type"])
        x = x + m_res * y
        mlp = L.get("mlp")
        if mlp is not None:
            h = offset_norm(x, W[p + "norm2"], eps)
            y = dense_mlp(h, W, p + "mlp.") if mlp["kind"] == "dense" else routed_mlp(h, tokens, W, p + "mlp.", mlp)
            x = x + m_res * y
        if layers_out is not None:
            layers_out.append(x.copy())
    return offset_norm(x, W["final.norm"], eps) @ np.asarray(W["head"], dtype=np.float64).T * float(cfg["logit_scale"])
