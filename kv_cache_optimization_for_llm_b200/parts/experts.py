"""A feed-forward of many small experts of which every token uses a few."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """``experts`` feed-forward layers ``W_down relu(W_up h)^2`` (``expert_ff`` wide, no biases) of which a
    token uses ``top``.  The router's logits ``W_r h`` are float32; the scores are their softmax over
    all experts; the ``top`` experts with the largest ``score + correction`` are chosen and weighted with
    ``score / (sum of the chosen scores + 1e-20) * scale``.  The last ``identity`` outputs of the router
    are experts without matrices that hand their input on.  With ``shared_ff`` > 0 one more expert
    of the same form runs for every token with weight 1.

    All first matrices are stacked into one, and all second matrices side by side into another: a
    step is two products around an activation kernel that also multiplies each expert's features
    by the token's weight for it (0 where it was not chosen), so the second product's float32 sums
    add up exactly the chosen experts.  Every expert is computed for every token; what that costs
    against products over the chosen tokens only is ``experts / top`` times the experts' arithmetic
    in long steps and nothing in steps of a few tokens, which read every expert's matrices anyway.
    params: hidden_size, experts, identity, top, scale, expert_ff, shared_ff."""

    @classmethod
    def weight_specs(cls, params):
        h, E, I, F, S = (int(params[k]) for k in ("hidden_size", "experts", "identity", "expert_ff", "shared_ff"))
        specs = {"router": WeightSpec((E + I, h), "bias"), "correction": WeightSpec((E + I,), "bias")}
        for e in range(E):
            specs[f"up{e}"] = WeightSpec((F, h))
            specs[f"down{e}"] = WeightSpec((h, F))
        if S:
            specs["shared_up"] = WeightSpec((S, h))
            specs["shared_down"] = WeightSpec((h, S))
        return specs

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("experts",) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.hidden = int(params["hidden_size"])
        self.E, self.I, self.top = int(params["experts"]), int(params["identity"]), int(params["top"])
        self.F, self.S = int(params["expert_ff"]), int(params.get("shared_ff") or 0)
        self.scale = float(params["scale"])
        if not 1 <= self.top <= min(32, self.E + self.I):
            raise ValueError(f"routed_experts: {self.top} of {self.E + self.I} experts per token is refused (1 to 32)")
        ups = [weights[f"up{e}"] for e in range(self.E)] + ([weights["shared_up"]] if self.S else [])
        downs = [weights[f"down{e}"] for e in range(self.E)] + ([weights["shared_down"]] if self.S else [])
        self.width = self.E * self.F + self.S
        # the products' inner sizes are padded to multiples of 8 (16-byte rows), the padding being zeros
        self.pad = (-self.width) % 8
        if ups:
            up = torch.cat(ups, dim=0)
            down = torch.cat(downs, dim=1)
            if self.pad:
                up = torch.cat([up, up.new_zeros((self.pad, up.shape[1]))], dim=0)
                down = torch.cat([down, down.new_zeros((down.shape[0], self.pad))], dim=1)
            self.up, self.down = up.contiguous(), down.contiguous()
        else:
            self.up = self.down = None
        self.router, self.correction = weights["router"], weights["correction"]
        # The router's products are float32 sums of float32 products.  Where the compute type holds the router's
        # weights exactly (a checkpoint stored in that type), the step's matrix product kernels make them (tensor
        # cores add up bfloat16 products exactly in float32); otherwise the routing kernel does, on float32 weights.
        self.router_in_compute_type = None
        lowp = self.router.to(ctx.dtype)
        if self.hidden % 8 == 0 and torch.equal(lowp.float(), self.router):
            self.router_in_compute_type = lowp.contiguous()

    def activation_widths(self):
        w = self.width + self.pad
        return [4 * (self.E + self.I) + 2, w, w, self.hidden]

    def forward(self, x, batch):
        logits = None
        if self.router_in_compute_type is not None:
            logits = ops.linear(x, self.router_in_compute_type, out_dtype=torch.float32)
        gate, identity_weight = ops.route(x, self.router, self.correction, self.E, self.I, self.top, self.scale, logits)
        if self.up is not None:
            a = ops.expert_act(ops.linear(x, self.up), gate, self.E, self.F, self.S + self.pad)
            y = ops.linear(a, self.down)
        else:
            y = ops.new(tuple(x.shape), x.dtype, x.device)
            y.zero_()
        if identity_weight is not None:
            ops.row_axpy(y, x, identity_weight)
        return y
