"""A plain, slow Fivesun in numpy float64: whole sequences, no cache, no batching, one function
per mechanism.  It is the oracle of the Fivesun tests and shares nothing with the package.

Notation: T tokens, rows of every array are tokens.  ``w`` maps checkpoint tensor names to float64
arrays, ``cfg`` is the config.json dictionary, ``p`` a tensor-name prefix, ``m`` a mixer's entry.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def logsigmoid(x):
    return -np.logaddexp(0.0, -x)


def unit_rms(x, eps):
    """Rows (last axis) divided by their root mean square, eps under the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


# ---------------------------------------------------------------- rotary positions
def rotary_frequencies(rot):
    """Per pair i of the first ``dims`` channels: base^(-2i/dims), divided by the factor (linear
    scaling), or blended between divided and kept by a ramp over i (the scaling with four numbers);
    returns (frequencies, factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor = float(sc["factor"])
    if "original" not in sc:
        return f / factor, 1.0

    def pair_at(turns):
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_at(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_at(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, size]: neighbouring channels (2i, 2i+1) of the first ``dims`` turn by position * f_i."""
    if not rot:
        return x
    f, mag = rotary_frequencies(rot)
    dims = int(rot["dims"])
    ang = positions[:, None].astype(np.float64) * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------- masks
def chunk_mask(T, size):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def window_mask(T, size):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def causal_mask(T):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return j <= i


def softmax_rows(scores, visible, sink=None):
    """Softmax over the visible keys of every row; ``sink`` (one number per row or None) is one more
    term of the denominator that has no value."""
    s = np.where(visible, scores, -np.inf)
    top = s.max(axis=-1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink[:, None])
    e = np.where(visible, np.exp(s - top), 0.0)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink[:, None] - top)
    return e / den


# ---------------------------------------------------------------- mixer: attention
def attention(h, w, p, m, eps, v_first=None):
    """Grouped-query attention with normed queries, keys and values, a chunked mask, a sink in the
    softmax, values blended with those of the first such layer, and a gate per head.
    Returns (output, the values this layer attends over)."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q = rotate(rms_norm(q, w[p + "q.norm"], eps), pos, m.get("rot"))
    k = rotate(rms_norm(k, w[p + "k.norm"], eps), pos, m.get("rot"))
    v = unit_rms(v, eps)
    if m.get("v_mix") and v_first is not None:
        lam = float(w[p + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    visible = chunk_mask(T, int(m["mask"]["size"])) if m.get("mask") else causal_mask(T)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        sc = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        pr = softmax_rows(sc, visible, np.full(T, float(w[p + "sink"][hd])))
        out[:, hd] = pr @ v[:, g]
    gate = sigmoid(h @ w[p + "g"].T)                      # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T, v


# ---------------------------------------------------------------- mixer: latent attention
def latent_attention(h, w, p, m, eps):
    """Keys and values expanded from one low-rank row per token; one rotated key part shared by the
    heads; a sliding window; a gate per output channel."""
    T = h.shape[0]
    H, d, dr, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, d + dr)
    q_flat, q_rot = q[..., :d], rotate(q[..., d:], pos, m.get("rot"))
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :R], w[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, None, R:], pos, m.get("rot"))[:, 0]          # [T, dr]
    k_flat = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    visible = window_mask(T, int(m["mask"]["size"])) if m.get("mask") else causal_mask(T)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        sc = (q_flat[:, hd] @ k_flat[:, hd].T + q_rot[:, hd] @ k_rot.T) * float(m["scale"])
        out[:, hd] = softmax_rows(sc, visible) @ v[:, hd]
    out = out.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---------------------------------------------------------------- mixer: matrix memory
def mlstm(h, w, p, m, eps):
    """A matrix memory per head with exponential input gate, sigmoid forget gate (both capped through a
    tanh) and a running maximum m that starts at 0 and keeps the exponentials in range."""
    T = h.shape[0]
    H, d, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ w[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    gi = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                 # log of the input gate
    gf = logsigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))     # log of the forget gate
    out = np.zeros((T, H, dv))
    for hd in range(H):
        S, n, mx = np.zeros((d, dv)), np.zeros(d), 0.0
        for t in range(T):
            m_new = max(gf[t, hd] + mx, gi[t, hd])
            keep, take = math.exp(gf[t, hd] + mx - m_new), math.exp(gi[t, hd] - m_new)
            S = keep * S + take * np.outer(k[t, hd], v[t, hd])
            n = keep * n + take * k[t, hd]
            mx = m_new
            out[t, hd] = (S.T @ q[t, hd]) / (max(abs(n @ q[t, hd]), math.exp(-mx)) + 1e-6)
    out = unit_rms(out, eps).reshape(T, H * dv) * w[p + "norm"]
    out = out * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---------------------------------------------------------------- feed-forward
def feed_forward(h, w, p):
    gate = np.maximum(h @ w[p + "gate"].T + w[p + "gate.b"], 0.0)
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (gate * up) @ w[p + "down"].T + w[p + "down.b"]


# ---------------------------------------------------------------- the model
def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence; with ``return_layers`` also the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    tokens = np.asarray(tokens)
    x = w["embed"][tokens] * float(cfg.get("embedding", {}).get("scale", 1.0))
    v_first, streams = None, []
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        h = rms_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "attention":
            y, v = attention(h, w, pre + "mix.", m, eps, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, pre + "mix.", m, eps)
        elif layer["type"] == "mlstm":
            y = mlstm(h, w, pre + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        y = y * sigmoid(h @ w[pre + "rg1"].T + w[pre + "rg1.b"])
        x = x + rms_norm(y, w[pre + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, w[pre + "norm2"], eps)
            y = feed_forward(h, w, pre + "mlp.")
            y = y * sigmoid(h @ w[pre + "rg2"].T + w[pre + "rg2.b"])
            x = x + rms_norm(y, w[pre + "norm2b"], eps)
        streams.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
