"""Dense gated feed-forward."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightDecl, param, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down(silu(gate(x)) * up(x)), no biases (miniserve/model/qwen3.py:128-131). The gate and
    up matrices are stacked at load so that one product makes both
    (miniserve/model/fused.py:41-95 does the same). Parameters: ``hidden``, ``intermediate``."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.inter = param(spec, "intermediate", int)

    def weights(self):
        return {
            "gate_proj.weight": WeightDecl((self.inter, self.hidden)),
            "up_proj.weight": WeightDecl((self.inter, self.hidden)),
            "down_proj.weight": WeightDecl((self.hidden, self.inter)),
        }

    def stacks(self):
        return {"gate_up_proj.weight": ("gate_proj.weight", "up_proj.weight")}

    def bind(self, tensors):
        self.w_gate_up = self.joined(tensors, "gate_up_proj.weight", self.stacks()["gate_up_proj.weight"])
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, ctx) -> torch.Tensor:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        act = ctx.buffer("mlp.act", (t, self.inter), dt, dev)
        if dt == torch.bfloat16:
            # one kernel with the activation in its epilogue where there is one (decode steps, wide prompt steps)
            fused = ops.silu_mul_is_fused(x, self.w_gate_up, act)
            scratch = None if fused else ctx.buffer("mlp.gate_up", (t, 2 * self.inter), dt, dev)
            ops.linear_silu_mul(x, self.w_gate_up, act, scratch=scratch, stream=ctx.stream)
        else:
            gate_up = ops.linear(x, self.w_gate_up, stream=ctx.stream, out=ctx.buffer("mlp.gate_up", (t, 2 * self.inter), dt, dev))
            ops.silu_mul(act, gate_up, stream=ctx.stream)
        return ops.linear(act, self.w_down, stream=ctx.stream, out=ctx.buffer("mlp.down", (t, self.hidden), dt, dev))


@register_part("feed_forward", "dense_mlp")
class DenseMLP(Part):
    """down(act(up(x))), no gate and no biases. Parameters: ``hidden``, ``intermediate``, ``activation``
    (``gelu_tanh``: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); ``relu_squared``: max(z, 0)^2), ``names``
    (up / down -> tensor names). ``features`` stops before the down projection, for a block that joins it with
    another part's output projection."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.inter = param(spec, "intermediate", int)
        self.activation = spec.get("activation", "gelu_tanh")
        if self.activation not in ("gelu_tanh", "relu_squared"):
            raise ValueError(f"dense_mlp knows the activations 'gelu_tanh' and 'relu_squared', not {self.activation!r}")
        self.feature_width = self.inter
        names = dict(spec.get("names") or {})
        self.names = {"up": names.get("up", "up_proj.weight"), "down": names.get("down", "down_proj.weight")}

    def weights(self):
        return {self.names["up"]: WeightDecl((self.inter, self.hidden)),
                self.names["down"]: WeightDecl((self.hidden, self.inter))}

    def bind(self, tensors):
        self.w_up = tensors[self.names["up"]].contiguous()
        self.w_down = tensors[self.names["down"]].contiguous()

    def features(self, x, ctx, out: torch.Tensor) -> None:
        """``out`` [T, intermediate] (a view whose rows may be part of wider ones) = act(up(x))."""
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        up = ops.linear(x, self.w_up, stream=ctx.stream, out=ctx.buffer("mlp.up", (t, self.inter), dt, dev))
        if self.activation == "relu_squared":
            ops.relu_squared(out, up, stream=ctx.stream)
        else:
            ops.gelu_tanh(up, up, stream=ctx.stream)
            out.copy_(up)

    def forward(self, x, ctx) -> torch.Tensor:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        if self.activation == "relu_squared":
            act = ctx.buffer("mlp.act", (t, self.inter), dt, dev)
            self.features(x, ctx, act)
            return ops.linear(act, self.w_down, stream=ctx.stream, out=ctx.buffer("mlp.down", (t, self.hidden), dt, dev))
        # the activation in the product's epilogue where there is such a kernel (decode steps)
        act = ops.linear_gelu_tanh(x, self.w_up, ctx.buffer("mlp.act", (t, self.inter), dt, dev), stream=ctx.stream)
        return ops.linear(act, self.w_down, stream=ctx.stream, out=ctx.buffer("mlp.down", (t, self.hidden), dt, dev))
