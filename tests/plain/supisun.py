"""Plain Supisun forward pass: whole sequences, no cache, no state carried, numpy float64.

One function per mechanism, written from the design's equations. Notation: T tokens, x the residual stream
[T, width], W the dictionary of weights by tensor name, p a tensor-name prefix. Linear weights are [out, in]
and applied as x @ W.T. No code is shared with the product package.

  causal_conv     y_t = sum_j w[:, j] * x_(t - taps + 1 + j)  (+ bias), zeros before the start
  layer_norm      (x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations
  rms_unit        x / sqrt(mean(x^2) + eps)
  rotate_half     pairs (i, i + dims/2) of the first `dims` dimensions turned by p * base^(-2i/dims)
  attention       whole-projection q/k norm, rotation, unit-RMS values, value mixing, chunked causal softmax
  mamba1          gated selective scan
  delta           gated delta rule
  dense_mlp       down(gelu_erf(up(x)))
  forward         embedding + positions, the layers (x += LN(mixer(x + conv(x))); x += LN(mlp(x))), LN, head
"""
from __future__ import annotations

import math

import numpy as np


def _erf(x: np.ndarray) -> np.ndarray:
    return np.vectorize(math.erf, otypes=[np.float64])(x)


def silu(x):
    return x / (1.0 + np.exp(-x))


def softplus(x):
    return np.logaddexp(0.0, x)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def gelu_erf(x):
    return 0.5 * x * (1.0 + _erf(x / math.sqrt(2.0)))


def causal_conv(x, w, bias=None):
    T, C = x.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += w[:, j][None, :] * padded[j:j + T]
    return y if bias is None else y + bias[None, :]


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rotate_half(x, dims, base):
    """x [T, heads, dim]; position of row t is t."""
    if not dims:
        return x
    T = x.shape[0]
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.arange(T)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(T, chunk=None):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    vis = j <= i
    if chunk:
        vis &= (i // chunk) == (j // chunk)
    return vis


def attention(W, p, m, h, eps, shared, chunk_override=None):
    T = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    q = rms_unit(q, eps) * W[p + "q.norm"]                 # one RMS over the whole projection
    k = rms_unit(k, eps) * W[p + "k.norm"]
    q, k, v = q.reshape(T, H, dim), k.reshape(T, G, dim), v.reshape(T, G, vd)
    rot = m.get("rot") or {}
    q, k = rotate_half(q, rot.get("dims", 0), rot.get("base", 1.0)), rotate_half(k, rot.get("dims", 0), rot.get("base", 1.0))
    v = rms_unit(v, eps)                                   # per head
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = float(W[p + "vmix"])
            v = (1.0 - lam) * v + lam * shared["v_first"]
    chunk = chunk_override if chunk_override is not None else (m.get("mask") or {}).get("size")
    vis = visible(T, chunk)
    out = np.zeros((T, H, vd))
    for hh in range(H):
        g = hh // (H // G)
        s = np.where(vis, (q[:, hh] @ k[:, g].T) * m["scale"], -np.inf)
        s = np.exp(s - s.max(-1, keepdims=True))
        out[:, hh] = (s / s.sum(-1, keepdims=True)) @ v[:, g]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def mamba1(W, p, m, h):
    T = h.shape[0]
    I, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :I], xz[:, I:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    dbc = x @ W[p + "x"].T
    dt = softplus(dbc[:, :R] @ W[p + "dt"].T + W[p + "dt.b"])
    Bm, Cm = dbc[:, R:R + N], dbc[:, R + N:]
    A = -np.exp(W[p + "A_log"])
    S = np.zeros((I, N))
    y = np.zeros((T, I))
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * Bm[t][None, :]
        y[t] = S @ Cm[t] + W[p + "D"] * x[t]
    return (y * silu(z)) @ W[p + "o"].T


def delta(W, p, m, h, eps):
    T = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dim)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dim)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, vd)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[p + "b"].T)
    decay = np.exp(-np.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    gate = silu(h @ W[p + "g"].T).reshape(T, H, vd)
    o = np.zeros((T, H, vd))
    for hh in range(H):
        kv = hh // (H // G)
        S = np.zeros((dim, vd))
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, kv])
            S = S + np.outer(k[t, kv], u)
            o[t, hh] = S.T @ q[t, kv]
    o = rms_unit(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * vd) @ W[p + "o"].T


def dense_mlp(W, p, h):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


def forward(cfg, W, tokens, layers_out=None, chunk_override=None):
    """Logits [T, vocab] of one sequence run whole. `layers_out`, a list, receives the residual stream behind
    every layer. `chunk_override` replaces every attention layer's chunk size (a control for the tests)."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    tokens = np.asarray(tokens)
    T = len(tokens)
    x = W["embed"][tokens] + W["pos"][:T]
    shared = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = x + causal_conv(x, W[p + "canon1"])
        if L["type"] == "attention":
            y = attention(W, p + "mix.", L["mixer"], h, eps, shared, chunk_override)
        elif L["type"] == "mamba1":
            y = mamba1(W, p + "mix.", L["mixer"], h)
        else:
            y = delta(W, p + "mix.", L["mixer"], h, eps)
        x = x + layer_norm(y, W[p + "norm1"], W[p + "norm1.b"], eps)
        if L.get("mlp"):
            x = x + layer_norm(dense_mlp(W, p + "mlp.", x), W[p + "norm2"], W[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
