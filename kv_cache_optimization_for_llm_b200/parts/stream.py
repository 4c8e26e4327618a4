"""Parts that stand in the schedule in front of a layer and change what is pending on the
residual stream."""

from __future__ import annotations

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("stream", "pass_start")
class PassStart(Part):
    """The start of pass ``index`` through a run of layers that repeats with the same weights:
    row ``index`` of a learned table [passes, size] joins the stream, and so does, when
    ``add_embedding`` is set, the embedding's output once more.  Nothing is launched here: both
    are added to what is pending, and the next norm sums everything in its own kernel.
    params: size, passes, index, add_embedding."""

    @classmethod
    def weight_specs(cls, params):
        return {"steps": WeightSpec((params["passes"], params["size"]), "bias")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("rowwise",)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        index = int(params["index"])
        if not 0 <= index < int(params["passes"]):
            raise ValueError(f"pass_start: pass {index} of {params['passes']}")
        self.vector = weights["steps"][index].contiguous()
        self.needs_embedding = bool(params.get("add_embedding"))

    def forward(self, residual, delta, embedded):
        if delta is None:
            pending = ops.PendingSum()
        elif isinstance(delta, ops.PendingSum):
            pending = delta
        elif isinstance(delta, ops.Folded):
            pending = ops.PendingSum()      # that branch has added its output to the residual itself
        elif isinstance(delta, ops.PostNormed):
            pending = ops.PendingSum((delta.materialize(),))
        else:
            pending = ops.PendingSum((delta,))
        return pending.plus(rows=embedded if self.needs_embedding else None, vector=self.vector)
