"""The Rezusun decoder restated plainly: numpy, float64, whole sequences, no cache,
one function per mechanism.  It shares no code with the package; the tests compare
the engine with it.

Notation: ``h`` [T, width] is a sublayer's input, weights are stored [out, in] and
applied as ``x @ W.T``; ``w`` maps tensor names to float64 arrays.
"""

from __future__ import annotations

import math

import numpy as np


def linear(x, W, b=None):
    y = x @ W.T
    return y if b is None else y + b


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (weight None: bare)."""
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight, var the mean squared deviation; no bias."""
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * weight


def rotate_interleaved(x, positions, base, dims):
    """x [T, ..., D]: dimension 2i is paired with 2i + 1 for i < dims / 2; the pair at
    position p turns by the angle p * base^(-2i/dims); dimensions from ``dims`` on pass."""
    out = x.copy()
    i = np.arange(dims // 2)
    freq = base ** (-2.0 * i / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def sink_softmax_attention(q, k, v, scale, sink):
    """Causal attention of one head.  q [T, Dk], k [T, Dk], v [T, Dv]; the softmax's
    denominator holds exp(sink) once more: a key of score ``sink`` (unscaled) with no value."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
    m = np.maximum(s.max(axis=1), sink)
    e = np.exp(s - m[:, None])
    return (e @ v) / (e.sum(axis=1) + np.exp(sink - m))[:, None]


def latent_attention(h, w, p, mx, eps):
    """Attention whose queries, keys and values come from low-rank latents; one rotated key
    part is shared by all heads.  ``mx``: the mixer's sizes and constants."""
    T = h.shape[0]
    H, dim, rot, vdim, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    base, rdims = mx["rot"]["base"], mx["rot"]["dims"]
    pos = np.arange(T)
    cq = rms_norm(linear(h, w[p + "dq"]), w[p + "dq.norm"], eps)
    q = linear(cq, w[p + "uq"]).reshape(T, H, dim + rot)
    q_plain, q_rot = q[..., :dim], rotate_interleaved(q[..., dim:], pos, base, rdims)
    dkv = linear(h, w[p + "dkv"])
    c = rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_interleaved(dkv[:, rank:], pos, base, rdims)           # [T, rot], the same for every head
    k_plain = linear(c, w[p + "uk"]).reshape(T, H, dim)
    v = linear(c, w[p + "uv"]).reshape(T, H, vdim)
    out = np.zeros((T, H, vdim))
    for a in range(H):
        qa = np.concatenate([q_plain[:, a], q_rot[:, a]], axis=1)
        ka = np.concatenate([k_plain[:, a], k_rot], axis=1)
        out[:, a] = sink_softmax_attention(qa, ka, v[:, a], mx["scale"], w[p + "sink"][a])
    return linear(out.reshape(T, H * vdim), w[p + "o"])


def delta_state_scan(decay, remove, probe, key, value, read):
    """One head of the delta-rule family, token by token, state S [Dk, Dv] from zero:
    S <- diag(decay_t) S - remove_t (probe_t^T S) + key_t value_t^T with both products
    reading the state before the token; the token's output is S^T read_t afterwards."""
    T, Dk = key.shape
    S = np.zeros((Dk, value.shape[1]))
    out = np.zeros((T, value.shape[1]))
    for t in range(T):
        S = decay[t][:, None] * S - np.outer(remove[t], probe[t] @ S) + np.outer(key[t], value[t])
        out[t] = S.T @ read[t]
    return out


def general_delta(h, w, p, mx, eps):
    """Generalised delta rule: per-channel decay from a low-rank branch, a per-channel
    removal rate along the unit key, read-out by r, per-head RMS, weight, sigmoid gate."""
    T = h.shape[0]
    H, D = mx["heads"], mx["dim"]
    r = linear(h, w[p + "r"]).reshape(T, H, D)
    k = linear(h, w[p + "k"]).reshape(T, H, D)
    v = linear(h, w[p + "v"]).reshape(T, H, D)
    decay = np.exp(-math.exp(-0.5) * sigmoid(linear(np.tanh(linear(h, w[p + "w1"])), w[p + "w2"]) + w[p + "w0"]))
    decay = decay.reshape(T, H, D)
    a = sigmoid(linear(h, w[p + "a"], w[p + "a.b"])).reshape(T, H, D)
    unit = k / np.sqrt((k * k).sum(axis=-1, keepdims=True) + 1e-6)
    o = np.zeros((T, H, D))
    for j in range(H):
        o[:, j] = delta_state_scan(decay[:, j], a[:, j] * unit[:, j], unit[:, j], k[:, j], v[:, j], r[:, j])
    o = rms_norm(o, None, eps).reshape(T, H * D) * w[p + "norm"] * sigmoid(linear(h, w[p + "g"]))
    return linear(o, w[p + "o"])


def short_conv(x, taps_w):
    """Causal convolution over time per channel: x [T, C], taps_w [C, taps], the last
    column weighs the current token, zeros stand before the start."""
    T, C = x.shape
    n = taps_w.shape[1]
    padded = np.concatenate([np.zeros((n - 1, C)), x], axis=0)
    out = np.zeros((T, C))
    for j in range(n):
        out += padded[j:j + T] * taps_w[:, j][None, :]
    return out


def gated_delta_scan(g, beta, k, v, q):
    """One head of the gated delta rule exactly in the order it is stated: decay the
    state, take the error of its prediction for the key, write it, read with q."""
    T, Dk = k.shape
    S = np.zeros((Dk, v.shape[1]))
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def channel_delta(h, w, p, mx, eps):
    """Gated delta rule with a decay per head and key channel, short convolutions on q, k, v,
    grouped q/k heads, per-head RMS with one weight for all heads and a low-rank gate."""
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = silu(short_conv(linear(h, w[p + "q"]), w[p + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(linear(h, w[p + "k"]), w[p + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(linear(h, w[p + "v"]), w[p + "v.conv"])).reshape(T, H, Dv)
    q = q / np.sqrt((q * q).sum(axis=-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(linear(h, w[p + "b"]))                                        # [T, H]
    step = softplus(linear(linear(h, w[p + "a1"]), w[p + "a2"]) + w[p + "dt_bias"]).reshape(T, H, D)
    g = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * step)
    o = np.zeros((T, H, Dv))
    for j in range(H):
        kv = j // (H // G)
        o[:, j] = gated_delta_scan(g[:, j], beta[:, j], k[:, kv], v[:, j], q[:, kv])
    o = rms_norm(o, w[p + "norm"], eps)
    o = o.reshape(T, H * Dv) * sigmoid(linear(linear(h, w[p + "g1"]), w[p + "g2"]))
    return linear(o, w[p + "o"])


def dense_feed_forward(h, w, p):
    return linear(gelu_tanh(linear(h, w[p + "gate"], w[p + "gate.b"])) * linear(h, w[p + "up"], w[p + "up.b"]),
                  w[p + "down"], w[p + "down.b"])


MIXERS = {"latent_attention": latent_attention, "general_delta": general_delta, "channel_delta": channel_delta}


def layer_order(cfg):
    """The layers in the order they run: those of the loop ``times`` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, w, tokens, trace=None):
    """Logits [T, vocab] of one whole sequence.  ``trace``: a list that receives the
    residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    for i in layer_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        y = MIXERS[layer["type"]](layer_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        x = x + layer_norm(y, w[p + "norm1b"], eps) * w[p + "ls1"]
        if layer.get("mlp"):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward of kind {layer['mlp']['kind']!r}")
            y = dense_feed_forward(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
            x = x + layer_norm(y, w[p + "norm2b"], eps) * w[p + "ls2"]
        if trace is not None:
            trace.append(x.copy())
    return linear(layer_norm(x, w["final.norm"], eps), w["head"])
