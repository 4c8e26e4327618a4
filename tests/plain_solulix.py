"""The Solulix decoder restated plainly: numpy, float64, whole sequences, no cache, one
function per mechanism.  It shares no code with the package; the tests compare the engine
with it.

Notation: ``h`` [T, width] is a sublayer's input, weights are stored [out, in] and applied
as ``x @ W.T``; ``w`` maps tensor names to float64 arrays; ``p`` is a layer's tensor prefix.
"""

from __future__ import annotations

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (weight None: bare)."""
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def short_conv(u, taps_w):
    """Causal convolution over time per channel.  u [T, C], taps_w [C, taps]; the last column
    weighs the token itself, the one before it the token before, zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), u], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j][None, :]
    return y


def visible(T, size, keep_first):
    """[T, T] mask: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def one_more_softmax(s, mask):
    """exp(s_j) / (1 + sum_j exp(s_j)) over the visible keys of each row."""
    s = np.where(mask, s, -np.inf)
    m = np.maximum(s.max(axis=1), 0.0)
    e = np.exp(s - m[:, None])
    return e / (e.sum(axis=1) + np.exp(-m))[:, None]


def attention_mixer(h, w, p, mx):
    """Grouped-query attention without positions: projections, a short convolution on each of
    q, k, v, scores times ``scale``, a sliding window that also keeps the first tokens, a softmax
    whose denominator counts one more."""
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = short_conv(h @ w[p + "q"].T, w[p + "q.conv"]).reshape(T, H, D)
    k = short_conv(h @ w[p + "k"].T, w[p + "k.conv"]).reshape(T, G, D)
    v = short_conv(h @ w[p + "v"].T, w[p + "v.conv"]).reshape(T, G, Dv)
    mask = visible(T, mx["mask"]["size"], mx["mask"]["keep_first"])
    out = np.zeros((T, H, Dv))
    for a in range(H):
        g = a // (H // G)
        prob = one_more_softmax((q[:, a] @ k[:, g].T) * mx["scale"], mask)
        out[:, a] = prob @ v[:, g]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def unit(x):
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + 1e-6)


def delta_mixer(h, w, p, mx, eps):
    """Gated delta rule with one decay per head and token."""
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, Dv)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = sigmoid(h @ w[p + "b"].T)                                                      # [T, H]
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :] * softplus(h @ w[p + "a"].T + w[p + "dt_bias"][None, :]))
    gate = silu(h @ w[p + "g"].T).reshape(T, H, Dv)
    out = np.zeros((T, H, Dv))
    for a in range(H):
        g = a // (H // G)
        S = np.zeros((D, Dv))
        for t in range(T):
            S = decay[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, a] = S.T @ q[t, g]
    out = rms_norm(out, w[p + "norm"], eps) * gate
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def squared_relu_expert(h, up, down):
    return (np.maximum(h @ up.T, 0.0) ** 2) @ down.T


def route(h, w, p, router):
    """Per token the chosen experts and their weights: [T, top] indices and weights."""
    z = h @ w[p + "router"].T
    z = z - z.max(axis=1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=1, keepdims=True)
    choice = s + w[p + "correction"][None, :]
    top = router["top"]
    idx = np.argsort(-choice, axis=1, kind="stable")[:, :top]
    picked = np.take_along_axis(s, idx, axis=1)
    weights = picked / (picked.sum(axis=1, keepdims=True) + 1e-20) * router["scale"]
    return idx, weights


def moe_ff(h, w, p, mlp):
    router = mlp["router"]
    E = router["experts"]
    idx, weights = route(h, w, p, router)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(idx[t], weights[t]):
            if e >= E:                  # an identity expert
                out[t] += g * h[t]
            else:
                out[t] += g * squared_relu_expert(h[t:t + 1], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])[0]
    if mlp.get("shared"):
        out += squared_relu_expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    order += [(i, None) for i in range(b, n)]
    return order


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] for one whole sequence (and the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = rms_norm(w["embed"][np.asarray(tokens)], w["embed.norm"], eps)
    x0 = x.copy()
    seen = []
    loop = cfg.get("loop")
    if loop and loop["start"] == loop["stop"]:
        loop = None
    for i, pass_no in layer_order({**cfg, "loop": loop}):
        if pass_no is not None:
            if pass_no > 0:
                x = x + x0
            x = x + w["loop.step"][pass_no][None, :]
        layer = cfg["layers"][i]
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            branch = attention_mixer(h, w, p + "mix.", layer["mixer"])
        else:
            branch = delta_mixer(h, w, p + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            branch = branch + (dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp))
        x = x + branch
        seen.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(seen)) if return_layers else logits
