"""A plain, slow Fapudra in numpy float64: whole sequences, no cache, no batching, one function
per mechanism.  It is the oracle of the Fapudra tests and shares nothing with the package.

Notation: T tokens, W the model width, rows of every array are tokens.  ``w`` maps checkpoint
tensor names to float64 arrays, ``cfg`` is the config.json dictionary.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return np.logaddexp(0.0, x)


def unit_rms(x, eps):
    """Rows divided by their root mean square, eps under the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def causal_conv(x, taps_w, bias=None):
    """Per channel over time: y[t, c] = sum_j taps_w[c, j] x[t - (taps - 1) + j, c] (+ bias), zeros
    before the start; the last tap is the current token's."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j][None, :]
    if bias is not None:
        y = y + bias[None, :]
    return y


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu, with h_{-1} = 0."""
    prev = np.concatenate([np.zeros((1, h.shape[1])), h[:-1]], axis=0)
    return h + (prev - h) * mu[None, :]


# ---------------------------------------------------------------- state-space mixer
def mamba2(h, w, p, m, eps):
    H, P, N, G = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    inner = H * P
    T = h.shape[0]
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    Bm = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"][None, :])
    rate = np.exp(w[p + "A_log"])
    y = np.zeros((T, H, P))
    group_of = np.arange(H) // (H // G)
    S = np.zeros((H, N, P))                                    # one state matrix per head
    for t in range(T):
        S = np.exp(-rate * dt[t])[:, None, None] * S + dt[t][:, None, None] * Bm[t, group_of][:, :, None] * x[t][:, None, :]
        y[t] = np.einsum("hnp,hn->hp", S, Cm[t, group_of]) + w[p + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m.get("norm_groups", 1)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"][None, :]
    return y @ w[p + "o"].T


# ---------------------------------------------------------------- sigmoid attention
def distance_bucket(n, rows, far):
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def sigmoid_attention(h, w, p, m):
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    rel = w[p + "rel"]
    rows, far = rel.shape[0], m["bias_max"]
    mask = m.get("mask") or {}
    size, first = mask.get("size"), mask.get("keep_first", 0)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (j <= i) & ((i - j < size) | (j < first)) if size else (j <= i)
    bucket = np.array([distance_bucket(n, rows, far) for n in range(T)])[np.maximum(i - j, 0)]
    out = np.zeros((T, H, d))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] + rel[bucket, hd] + w[p + "pb"][hd]
        out[:, hd] = np.where(seen, sigmoid(s), 0.0) @ k[:, g]        # weights are not normalised over the keys
    out = out.reshape(T, H * d) * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---------------------------------------------------------------- delta rule with a decay per key channel
def channel_delta_rule(h, w, p, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"][None, :]).reshape(T, H, d)
    keep = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * step)
    o = np.zeros((T, H, dv))
    group_of = np.arange(H) // (H // G)
    S = np.zeros((H, d, dv))
    for t in range(T):
        kt, qt = k[t, group_of], q[t, group_of]
        S = keep[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - np.einsum("hdv,hd->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, qt)                  # the read-out sees this token's write
    o = unit_rms(o, eps) * w[p + "norm"][None, None, :]
    o = o.reshape(T, H * dv) * sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T)
    return o @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return (m.get("left_scale", 1.0) * sigmoid_attention(h, w, p + "left.", m["left"])
            + m.get("right_scale", 1.0) * channel_delta_rule(h, w, p + "right.", m["right"], eps))


# ---------------------------------------------------------------- mixture of experts
def route(h, w_router, r, gaps=None):
    """Per token the chosen experts and their weights: softmax over all experts; experts outside
    the best ``keep`` groups (a group's score is its best expert's) cannot be chosen.  ``gaps``: a
    list that receives, per token, how far (in logits) the closest call of the choice was."""
    z = h @ w_router.T
    z0 = z
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    E, top = r["experts"], r["top"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = grp["count"], grp["keep"]
    chosen, weights, margin = [], [], []
    for t in range(h.shape[0]):
        per = E // count
        best = np.array([s[t, g * per:(g + 1) * per].max() for g in range(count)])
        groups = np.argsort(-best, kind="stable")[:keep]
        allowed = np.full(E, -np.inf)
        for g in groups:
            allowed[g * per:(g + 1) * per] = s[t, g * per:(g + 1) * per]
        order = np.argsort(-allowed, kind="stable")
        idx = order[:top]
        chosen.append(idx)
        weights.append(s[t, idx] / (s[t, idx].sum() + 1e-20))
        gap = np.inf
        if keep < count:
            gz = np.sort(np.array([z0[t, g * per:(g + 1) * per].max() for g in range(count)]))[::-1]
            gap = min(gap, gz[keep - 1] - gz[keep])
        if top < keep * per:
            gap = min(gap, z0[t, order[top - 1]] - z0[t, order[top]])
        margin.append(gap)
    if gaps is not None:
        gaps.append(np.array(margin))
    return np.array(chosen), np.array(weights)


def expert(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def mixture(h, w, p, f, gaps=None):
    idx, wgt = route(h, w[p + "router"], f["router"], gaps)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t], wgt[t]):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.", f["expert"]["limit"])[0]
    return out


# ---------------------------------------------------------------- the model
def forward(cfg, w, tokens, layers_out=None, gaps=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the residual
    stream after every layer; ``gaps``: a list that receives, per layer with experts, every token's
    closest call in the choice of experts."""
    eps = cfg["norm"]["eps"]
    tokens = np.asarray(tokens)
    T = len(tokens)
    x = w["embed"][tokens] * (cfg.get("embedding") or {}).get("scale", 1.0) + w["pos"][:T]
    x = unit_rms(x, eps) * w["embed.norm"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = unit_rms(x, eps) * w[p + "norm1"]
        hm = token_shift(h, w[p + "shift"])
        if layer["type"] == "mamba2":
            a = mamba2(hm, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            a = parallel_mixer(hm, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        f = mixture(h, w, p + "mlp.", layer["mlp"], gaps) if layer.get("mlp") else 0.0
        x = x + (a + f)
        if layers_out is not None:
            layers_out.append(x.copy())
    y = unit_rms(x, eps) * w["final.norm"]
    logits = y @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return logits
