"""Parts that act on the residual stream between two layers."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, ResidualStream, WeightDecl, param, register_part


@register_part("transition", "stream_reentry")
class StreamReentry(Part):
    """x <- W [x ; x0] + step[n]: the stream re-enters through a product with the embedding output x0 beside it
    (W is [hidden, 2 hidden], x first), then row n of a [passes, hidden] table is added. Used before each pass
    over a stretch of layers that runs several times; ``n`` is the pass. The stream's pending addend is taken in
    first (float32); the product reads both halves in the run's dtype and writes float32; the table stays float32.
    The second half of the product's input is the same for every pass of a step and is written once.
    Parameters: ``hidden``, ``passes``, ``weight`` and ``step`` (the tensors' full names)."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.passes = param(spec, "passes", int)
        self.weight_name = param(spec, "weight", str)
        self.step_name = param(spec, "step", str)

    def weights(self):
        return {self.weight_name: WeightDecl((self.hidden, 2 * self.hidden)),
                self.step_name: WeightDecl((self.passes, self.hidden), precision="float32")}

    def bind(self, tensors):
        self.w_in = tensors[self.weight_name].contiguous()
        self.w_step = tensors[self.step_name].float().contiguous()

    def forward(self, stream: ResidualStream, ctx, embedding, arg: int) -> ResidualStream:
        if not 0 <= arg < self.passes:
            raise ValueError(f"stream_reentry: pass {arg} of {self.passes}")
        t, dt, dev = stream.total.shape[0], self.env.dtype, self.w_in.device
        both = ctx.buffer("reentry.in", (t, 2 * self.hidden), dt, dev)
        key = ("reentry.embedded", id(self))
        ops.stream_concat(both, stream.total, stream.pending, stream.pending_scale, embedding.table, ctx.token_ids,
                          first=True, second=key not in ctx.step_cache, stream=ctx.stream)
        ctx.step_cache[key] = True
        total = ctx.buffer("reentry.out", (t, self.hidden), torch.float32, dev)
        ops.linear(both, self.w_in, out=total, stream=ctx.stream)
        ops.add_row_vector(total, self.w_step[arg], stream=ctx.stream)
        return ResidualStream(total)
