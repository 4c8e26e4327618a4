"""Mixers that carry a matrix state per head from token to token (the delta-rule family).

Both mixers here make one product with all their input matrices stacked, turn the result
into the recurrence's vectors and step through the request's tokens in one kernel
(csrc/kernels/delta_rule.cu), and project the gated, normed read-out back to the model's
width.  The state lives in the request's slot as float32 and is zero for a request that
starts at position 0.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.specs import SlotStateSpec
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def _stack(mats, dtype_like):
    """Row-stacks matrices [n_i, in], each starting on a multiple of 8 rows (so that every
    segment of the product's rows starts 16-byte aligned); returns the matrix and the starts."""
    starts, rows, at = [], [], 0
    width = mats[0].shape[1]
    for m in mats:
        starts.append(at)
        rows.append(m)
        pad = _pad8(m.shape[0]) - m.shape[0]
        if pad:
            rows.append(torch.zeros((pad, width), dtype=m.dtype, device=m.device))
        at += _pad8(m.shape[0])
    return torch.cat(rows, dim=0).contiguous(), starts


def _modules(dtype):
    return ("delta_rule", "rowwise") + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))


@register("mixer", "general_delta")
class GeneralDelta(Part):
    """Generalised delta rule.  Per head, with r, k, v = W_r h, W_k h, W_v h (``dim`` each):
    decay ``w = exp(-e^{-1/2} sigmoid(W_w2 tanh(W_w1 h) + w0))`` and removal rate
    ``a = sigmoid(W_a h + b_a)`` per key channel, unit key ``u = k / sqrt(|k|^2 + 1e-6)``,

        S_t = diag(w) S_{t-1} - (a * u) (u^T S_{t-1}) + k v^T,        o_t = S_t^T r.

    Each head's o is divided by its root mean square, the heads are multiplied by ``norm``
    (one weight per head and channel) and by ``sigmoid(W_g h)``, then projected by W_o.
    params: hidden_size, heads, dim, decay_rank (rows of W_w1), eps."""

    @classmethod
    def weight_specs(cls, params):
        h, hd, lr = params["hidden_size"], params["heads"] * params["dim"], params["decay_rank"]
        return {"r": WeightSpec((hd, h)), "k": WeightSpec((hd, h)), "v": WeightSpec((hd, h)), "g": WeightSpec((hd, h)),
                "a": WeightSpec((hd, h)), "a_bias": WeightSpec((hd,), "bias"), "w1": WeightSpec((lr, h)),
                "w2": WeightSpec((hd, lr)), "w0": WeightSpec((hd,), "bias"), "norm": WeightSpec((hd,), "vector"),
                "o": WeightSpec((h, hd))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return _modules(dtype)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.heads, self.dim, self.eps = int(params["heads"]), int(params["dim"]), float(params["eps"])
        self.lr = int(params["decay_rank"])
        self.pad = ops.delta_key_pad(self.dim)
        if not self.pad or self.dim > 128:
            raise ValueError(f"general_delta: head size {self.dim} is refused (the scan keeps up to 128 key channels)")
        self.w_in, (self.at_r, self.at_k, self.at_v, self.at_g, self.at_a, self.at_w1) = _stack(
            [weights[n] for n in ("r", "k", "v", "g", "a", "w1")], ctx.dtype)
        self.w2, self.w0, self.a_bias = weights["w2"], weights["w0"], weights["a_bias"]
        self.norm, self.o = weights["norm"], weights["o"]

    def cache_spec(self):
        return SlotStateSpec((self.heads * self.dim * self.pad,), torch.float32)

    def activation_widths(self):
        hd = self.heads * self.dim
        return [self.w_in.shape[0], _pad8(self.lr), hd, 3 * hd, self.o.shape[0]]      # 3 hd: the read-outs in float32, and normed

    def forward(self, x, batch, cache):
        p = ops.linear(x, self.w_in)
        z = ops.linear(ops.tanh_slice(p, self.at_w1, self.lr), self.w2)
        y = ops.delta_scan("general", batch, cache.state, (p, self.at_r), (p, self.at_k), (p, self.at_v),
                           (p, self.at_g), (z, 0), (p, self.at_a), self.w0, self.a_bias, None, self.norm, True,
                           self.heads, self.heads, self.dim, self.dim, self.eps)
        return ops.linear(y, self.o)


@register("mixer", "channel_delta")
class ChannelDelta(Part):
    """Gated delta rule with a decay per head and key channel.  q, k (``kv_heads`` heads of ``dim``)
    and v (``heads`` heads of ``vdim``) each pass a short causal convolution over time per channel
    (``conv`` taps, the last for the token itself) and SiLU; q and k become unit vectors per head
    (q also times dim^-1/2); head j reads q/k head ``j // (heads / kv_heads)``.  With
    ``beta = sigmoid(W_b h)`` per head and ``g = exp(-exp(A_j) softplus(W_a2 W_a1 h + dt_bias))`` per head
    and key channel:

        S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.

    Each head's o is divided by its root mean square, multiplied by ``norm`` (``vdim`` wide, the
    same for all heads) and by ``sigmoid(W_g2 W_g1 h)``, then projected by W_o.  The request's
    state is the matrices and the last ``conv - 1`` inputs of the convolutions.
    params: hidden_size, heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank, eps."""

    @classmethod
    def weight_specs(cls, params):
        h, H, G, D, Dv = (params[k] for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        taps, ra, rg = params["conv"], params["decay_rank"], params["gate_rank"]
        return {"q": WeightSpec((G * D, h)), "k": WeightSpec((G * D, h)), "v": WeightSpec((H * Dv, h)),
                "q_conv": WeightSpec((G * D, taps), "bias"), "k_conv": WeightSpec((G * D, taps), "bias"),
                "v_conv": WeightSpec((H * Dv, taps), "bias"), "b": WeightSpec((H, h)),
                "A_log": WeightSpec((H,), "bias"), "norm": WeightSpec((Dv,), "vector"),
                "a1": WeightSpec((ra, h)), "a2": WeightSpec((H * D, ra)), "dt_bias": WeightSpec((H * D,), "bias"),
                "g1": WeightSpec((rg, h)), "g2": WeightSpec((H * Dv, rg)), "o": WeightSpec((h, H * Dv))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return _modules(dtype)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.heads, self.kv_heads = int(params["heads"]), int(params["kv_heads"])
        self.dim, self.vdim, self.taps = int(params["dim"]), int(params["vdim"]), int(params["conv"])
        self.eps = float(params["eps"])
        self.ra, self.rg = int(params["decay_rank"]), int(params["gate_rank"])
        if self.heads % self.kv_heads:
            raise ValueError(f"channel_delta: {self.heads} heads cannot share {self.kv_heads} query/key heads evenly")
        self.pad = ops.delta_key_pad(self.dim)
        if not self.pad or self.dim > 128 or self.vdim > 256 or (self.dim > 64 and self.vdim > 128):
            raise ValueError(f"channel_delta: head sizes {self.dim} x {self.vdim} are refused by the scan kernel")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"channel_delta: {self.taps} convolution taps are refused (1 to 16)")
        gd, hv = self.kv_heads * self.dim, self.heads * self.vdim
        # q, k, v lie side by side without padding: the convolution runs over them as one block of channels
        qkv = torch.cat([weights["q"], weights["k"], weights["v"]], dim=0)
        self.w_in, (_, self.at_b, self.at_a1, self.at_g1) = _stack(
            [qkv, weights["b"], weights["a1"], weights["g1"]], ctx.dtype)
        self.channels = 2 * gd + hv
        self.conv_w = torch.cat([weights["q_conv"], weights["k_conv"], weights["v_conv"]], dim=0).contiguous()
        self.a2, self.g2 = weights["a2"], weights["g2"]
        self.A_log, self.dt_bias, self.norm, self.o = weights["A_log"], weights["dt_bias"], weights["norm"], weights["o"]
        self.matrix_floats = self.heads * self.vdim * self.pad

    def cache_spec(self):
        return SlotStateSpec((self.matrix_floats + (self.taps - 1) * self.channels,), torch.float32)

    def activation_widths(self):
        hv = self.heads * self.vdim
        return [self.w_in.shape[0], self.channels, self.heads * self.dim, hv, 3 * hv, self.o.shape[0]]

    def forward(self, x, batch, cache):
        p = ops.linear(x, self.w_in)
        decay = ops.linear(p[:, self.at_a1:self.at_a1 + self.ra], self.a2)
        gate = ops.linear(p[:, self.at_g1:self.at_g1 + self.rg], self.g2)
        tails = cache.state[:, self.matrix_floats:] if self.taps > 1 else None
        c = ops.conv_silu(p, 0, self.channels, self.conv_w, tails, batch)
        gd = self.kv_heads * self.dim
        y = ops.delta_scan("gated", batch, cache.state, (c, 0), (c, gd), (c, 2 * gd), (gate, 0), (decay, 0),
                           (p, self.at_b), self.dt_bias, None, self.A_log, self.norm, False,
                           self.heads, self.kv_heads, self.dim, self.vdim, self.eps)
        return ops.linear(y, self.o)


@register("mixer", "gated_delta")
class GatedDelta(Part):
    """Gated delta rule with one decay per head.  q, k (``kv_heads`` heads of ``dim``) and v (``heads``
    heads of ``vdim``) each pass a short causal convolution over time per channel (``conv`` taps, the
    last for the token itself) and SiLU; q and k become unit vectors per head (q also times dim^-1/2);
    head j reads q/k head ``j // (heads / kv_heads)``.  With ``beta = sigmoid(W_b h)`` and
    ``g = exp(-exp(A_j) softplus(W_a h + dt_bias))``, both one number per head:

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.

    Each head's o is divided by its root mean square, multiplied by ``norm`` (``vdim`` wide, the same
    for all heads) and by ``silu(W_g h)``, then projected by W_o.  The request's state is the
    matrices (float32) and the last ``conv - 1`` inputs of the convolutions.  One product makes every
    projection; the recurrence runs in the scan kernel that the other delta-rule mixers use.
    params: hidden_size, heads, kv_heads, dim, vdim, conv, eps."""

    @classmethod
    def weight_specs(cls, params):
        h, H, G, D, Dv, taps = (params[k] for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim", "conv"))
        return {"q": WeightSpec((G * D, h)), "k": WeightSpec((G * D, h)), "v": WeightSpec((H * Dv, h)),
                "q_conv": WeightSpec((G * D, taps), "bias"), "k_conv": WeightSpec((G * D, taps), "bias"),
                "v_conv": WeightSpec((H * Dv, taps), "bias"), "b": WeightSpec((H, h)), "a": WeightSpec((H, h)),
                "A_log": WeightSpec((H,), "bias"), "dt_bias": WeightSpec((H,), "bias"),
                "norm": WeightSpec((Dv,), "vector"), "g": WeightSpec((H * Dv, h)), "o": WeightSpec((h, H * Dv))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return _modules(dtype)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.heads, self.kv_heads = int(params["heads"]), int(params["kv_heads"])
        self.dim, self.vdim, self.taps = int(params["dim"]), int(params["vdim"]), int(params["conv"])
        self.eps = float(params["eps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"gated_delta: {self.heads} heads cannot share {self.kv_heads} query/key heads evenly")
        self.pad = ops.delta_key_pad(self.dim)
        if not self.pad or self.dim > 128 or self.vdim > 256 or (self.dim > 64 and self.vdim > 128):
            raise ValueError(f"gated_delta: head sizes {self.dim} x {self.vdim} are refused by the scan kernel")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"gated_delta: {self.taps} convolution taps are refused (1 to 16)")
        gd, hv = self.kv_heads * self.dim, self.heads * self.vdim
        qkv = torch.cat([weights["q"], weights["k"], weights["v"]], dim=0)
        self.w_in, (_, self.at_b, self.at_a, self.at_g) = _stack([qkv, weights["b"], weights["a"], weights["g"]], ctx.dtype)
        self.channels = 2 * gd + hv
        self.conv_w = torch.cat([weights["q_conv"], weights["k_conv"], weights["v_conv"]], dim=0).contiguous()
        self.A_log, self.dt_bias, self.norm, self.o = weights["A_log"], weights["dt_bias"], weights["norm"], weights["o"]
        self.matrix_floats = self.heads * self.vdim * self.pad

    def cache_spec(self):
        return SlotStateSpec((self.matrix_floats + (self.taps - 1) * self.channels,), torch.float32)

    def activation_widths(self):
        hv = self.heads * self.vdim
        return [self.w_in.shape[0], self.channels, hv, 3 * hv, self.o.shape[0]]

    def forward(self, x, batch, cache):
        p = ops.linear(x, self.w_in)
        tails = cache.state[:, self.matrix_floats:] if self.taps > 1 else None
        c = ops.conv_silu(p, 0, self.channels, self.conv_w, tails, batch)
        gd = self.kv_heads * self.dim
        y = ops.delta_scan("gated", batch, cache.state, (c, 0), (c, gd), (c, 2 * gd), (p, self.at_g), (p, self.at_a),
                           (p, self.at_b), self.dt_bias, None, self.A_log, self.norm, False,
                           self.heads, self.kv_heads, self.dim, self.vdim, self.eps,
                           decay_per_head=True, gate_act="silu")
        return ops.linear(y, self.o)
