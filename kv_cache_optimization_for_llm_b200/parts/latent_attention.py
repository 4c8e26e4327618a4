"""Attention over a cached latent."""

from __future__ import annotations

import torch

from .. import ops
from ..cache.specs import PagedKVSpec
from ..weights.loader import WeightSpec
from .base import Part
from .delta_rule import _stack
from .registry import lookup, register


@register("mixer", "latent_attention")
class LatentAttention(Part):
    """Causal attention whose queries, keys and values come from low-rank latents.

    ``c_q = rms(W_dq h) * w_dq`` and ``q = W_uq c_q``, per head ``dim`` plain dimensions followed by
    ``rot_dim`` rotated ones.  ``W_dkv h`` gives ``kv_rank`` rows that, RMS-normed, are the latent c,
    and ``rot_dim`` more that are one rotated key part shared by all heads.  Per head the plain key
    is ``W_uk c`` and the value ``W_uv c``; score = (q_plain . k_plain + q_rot . k_rot) * scale; the
    softmax's denominator also holds ``exp(sink_h)``.  Only [c | rotated part] is cached, one
    row per token (a paged group of one plane).

    The key up-projection is applied to the queries instead (q_plain^T W_uk,h c = (W_uk,h^T q_plain)^T c),
    attention runs for all heads over the cached rows, and the value up-projection is applied
    to the attended latents; the output projection follows.
    params: hidden_size, heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, eps, position (PartSpec)."""

    @classmethod
    def weight_specs(cls, params):
        h, H, d, r, dv = (params[k] for k in ("hidden_size", "heads", "dim", "rot_dim", "vdim"))
        qr, kr = params["q_rank"], params["kv_rank"]
        return {"dq": WeightSpec((qr, h)), "dq_norm": WeightSpec((qr,), "vector"), "uq": WeightSpec((H * (d + r), qr)),
                "dkv": WeightSpec((kr + r, h)), "dkv_norm": WeightSpec((kr,), "vector"),
                "uk": WeightSpec((H * d, kr)), "uv": WeightSpec((H * dv, kr)), "sink": WeightSpec((H,), "bias"),
                "o": WeightSpec((h, H * dv))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("latent_attention",) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.heads, self.dim, self.rot, self.vdim = (int(params[k]) for k in ("heads", "dim", "rot_dim", "vdim"))
        self.q_rank, self.rank = int(params["q_rank"]), int(params["kv_rank"])
        self.scale, self.eps = float(params["scale"]), float(params["eps"])
        if self.rank > 512:
            raise ValueError(f"latent_attention: a latent of {self.rank} is refused (up to 512)")
        if ctx.dtype == torch.bfloat16 and (self.rank + self.rot) % 2:
            raise ValueError("latent_attention: in bfloat16 the cached row (kv_rank + rot_dim) must be even")
        self.w_in, (_, self.at_kv) = _stack([weights["dq"], weights["dkv"]], ctx.dtype)
        self.dq_norm, self.dkv_norm = weights["dq_norm"], weights["dkv_norm"]
        self.uq, self.o, self.sink = weights["uq"], weights["o"], weights["sink"]
        # per head: U_k^T [rank, dim] (absorbs the queries) and U_v [vdim, rank] (up-projects the attended latents)
        self.uk_t = weights["uk"].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = weights["uv"].view(self.heads, self.vdim, self.rank).contiguous()
        pos = params.get("position")
        self.position = None
        if pos is not None and self.rot:
            self.position = (ctx.make("position", pos) if ctx.make is not None
                             else lookup("position", pos.kind)(pos.params, {}, ctx))
            if self.position.rotary_dim > self.rot:
                raise ValueError(f"latent_attention: {self.position.rotary_dim} rotary dimensions in a part of {self.rot}")

    def cache_spec(self):
        return PagedKVSpec(1, self.rank + self.rot, None, planes=1)

    def activation_widths(self):
        H = self.heads
        return [self.w_in.shape[0], self.q_rank, H * (self.dim + self.rot), 3 * H * self.rank, 2 * H * self.vdim,
                self.o.shape[0]]

    def query_tile_heights(self):
        """Tokens per tile of the tensor-core attention (bfloat16, sizes it takes): the step's batch
        lays the tiles out for it."""
        if self.ctx.dtype != torch.bfloat16 or not ops.LATENT_TC or not ops.latent_attention_tc_supported(self.rank, self.rot):
            return []
        return [ops.latent_tokens_per_tile(self.heads)]

    def forward(self, x, batch, cache):
        d = ops.linear(x, self.w_in)
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        rdims = self.position.rotary_dim if self.position is not None else 0
        table = batch.block_tables[cache.group]
        cq = ops.latent_prep(d, self.q_rank, self.at_kv, self.rank, self.rot, rdims, self.dq_norm, self.dkv_norm,
                             self.eps, cos, sin, batch, table, cache.k, cache.write)
        q = ops.linear(cq, self.uq)
        per_head = self.dim + self.rot
        q_abs = ops.head_gemm(q, 0, per_head, self.uk_t)
        lat = ops.latent_attention(q_abs, q, self.dim, per_head, cos, sin, rdims, cache.k, table, batch, self.sink,
                                   self.scale, self.heads, self.rank, self.rot)
        return ops.linear(ops.head_gemm(lat, 0, self.rank, self.uv), self.o)
