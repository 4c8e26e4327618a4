"""Attention whose mask is a sliding window that keeps the sequence's first tokens, over
queries, keys and values that pass a short convolution first."""

from __future__ import annotations

import torch

from .. import ops
from ..cache.specs import PagedKVSpec, PagedWithStateSpec, SlotStateSpec
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("mixer", "conv_window_attention")
class ConvWindowAttention(Part):
    """Grouped-query attention without positions in its scores.

    q (``heads`` x ``dim``), k (``kv_heads`` x ``dim``) and v (``kv_heads`` x ``vdim``) come from one
    product with the row-stacked matrix; each channel then passes a causal convolution over time of
    ``conv`` taps (the last tap weighs the token itself, zeros before the sequence's start, no
    activation), whose last ``conv - 1`` inputs per request live in the request's state slot.  The
    convolved keys and values go to the request's pages, a row per token and key/value head holding
    [k | v].  Query i sees key j when ``j <= i and (i - j < window or j < keep_first)`` (``window`` None:
    every key up to i); scores are ``(q . k) * scale``; with ``one_more`` the softmax's denominator is
    ``1 + sum exp(s)``.  Query head h reads key/value head ``h // (heads / kv_heads)``.  Then W_o.
    Kernels: the general one (float32 arithmetic, any sizes, chunks of keys by absolute position) for
    float32, for steps of single tokens and for sizes the other refuses; for bfloat16 steps with runs
    of tokens and key and value size both 64 or 128 the tensor-core kernel of prompt portions.
    params: hidden_size, heads, kv_heads, dim, vdim, conv, scale, window, keep_first, one_more."""

    @classmethod
    def weight_specs(cls, params):
        h, H, G, D, Dv, taps = (params[k] for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim", "conv"))
        return {"q": WeightSpec((H * D, h)), "k": WeightSpec((G * D, h)), "v": WeightSpec((G * Dv, h)),
                "q_conv": WeightSpec((H * D, taps), "bias"), "k_conv": WeightSpec((G * D, taps), "bias"),
                "v_conv": WeightSpec((G * Dv, taps), "bias"), "o": WeightSpec((h, H * Dv))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        mods = ["window_attention", "delta_rule"]
        if dtype == torch.bfloat16 and params["dim"] == params["vdim"] and params["dim"] in (64, 128):
            mods.append("flash_attention")
        return tuple(mods) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.heads, self.kv_heads = int(params["heads"]), int(params["kv_heads"])
        self.dim, self.vdim, self.taps = int(params["dim"]), int(params["vdim"]), int(params["conv"])
        if self.heads % self.kv_heads:
            raise ValueError(f"conv_window_attention: {self.heads} query heads cannot be grouped over "
                             f"{self.kv_heads} key/value heads")
        if not (1 <= self.dim <= 256 and 1 <= self.vdim <= 256):
            raise ValueError(f"conv_window_attention: head sizes {self.dim} x {self.vdim} are refused (1 to 256)")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"conv_window_attention: {self.taps} convolution taps are refused (1 to 16)")
        self.scale = float(params["scale"])
        self.window = int(params["window"]) if params.get("window") else None
        self.keep_first = int(params.get("keep_first") or 0) if self.window else 0
        self.one_more = bool(params.get("one_more"))
        self.qkv = torch.cat([weights["q"], weights["k"], weights["v"]], dim=0).contiguous()
        self.conv_w = torch.cat([weights["q_conv"], weights["k_conv"], weights["v_conv"]], dim=0).contiguous()
        self.o = weights["o"]
        self.k_off = self.heads * self.dim
        self.v_off = self.k_off + self.kv_heads * self.dim
        self.channels = self.v_off + self.kv_heads * self.vdim

    def cache_spec(self):
        paged = PagedKVSpec(self.kv_heads, self.dim + self.vdim, self.window, planes=1, keep_first=self.keep_first)
        if self.taps == 1:
            return paged
        return PagedWithStateSpec(paged, SlotStateSpec(((self.taps - 1) * self.channels,), torch.float32))

    def activation_widths(self):
        return [self.channels, self.channels, self.heads * self.vdim, self.o.shape[0]]

    def _on_tensor_cores(self, page_size):
        return ops.flash_attention_rows_supported(self.dim, self.vdim, self.heads // self.kv_heads, page_size, self.ctx.dtype)

    def query_tile_heights(self):
        """Tokens per tile of the tensor-core kernel for prompt portions (bfloat16, key and value size
        64 or 128): the step's batch lays the tiles out for them."""
        if self.ctx.dtype != torch.bfloat16 or self.dim != self.vdim or self.dim not in (64, 128):
            return []
        g = self.heads // self.kv_heads
        return [ops.flash_tokens_per_tile(g, False), ops.flash_tokens_per_tile(g, True)]

    def forward(self, x, batch, cache):
        p = ops.linear(x, self.qkv)
        table = batch.block_tables[cache.group]
        # the convolution writes the new keys and values into their pages itself where the rows allow 16-byte accesses
        fused = cache.write and ops.conv_can_append(p, 0, self.channels, self.k_off, self.v_off, self.dim, self.vdim)
        c = ops.conv_silu(p, 0, self.channels, self.conv_w, cache.state, batch, act="none",
                          append=(cache.k, table, self.k_off, self.v_off, self.kv_heads, self.dim, self.vdim) if fused else None)
        if cache.write and not fused:
            ops.kv_rows_append(c, self.k_off, self.v_off, cache.k, table, batch, self.kv_heads, self.dim, self.vdim)
        if not batch.decode_only and self._on_tensor_cores(cache.page_size) and c.stride(0) % 8 == 0:
            a = ops.flash_attention_rows(c, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.scale,
                                         self.window or 0, self.keep_first, self.one_more)
        else:
            a = ops.window_attention(c, 0, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.vdim,
                                     self.scale, self.window or 0, self.keep_first, self.one_more)
        return ops.linear(a, self.o)
