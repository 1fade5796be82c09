"""Position encodings that act on q and k inside the attention mixer."""

from __future__ import annotations

import torch

from .base import Part, param, register_part


@register_part("position", "rope_neox")
class RotaryNeox(Part):
    """Rotate-half rotary encoding: inv_freq[j] = 1 / theta^(2j / rotary_dim), computed on the
    CPU in float32 from an int64 arange exactly as the reference does
    (miniserve/model/qwen3.py:98-101); the kernel multiplies by the position and takes
    cos/sin in float32. Parameters: ``head_dim``, ``theta``, optional ``rotary_dim``."""
    shape_static = True
    pairing = "halves"  # channel i turns together with channel i + rotary_dim / 2

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = param(spec, "head_dim", int)
        self.theta = param(spec, "theta", float)
        rotary = spec.get("rotary_dim")
        self.rotary_dim = self.head_dim if rotary is None else int(rotary)  # 0: nothing is rotated
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and at most head_dim={self.head_dim}")
        self.inv_freq = self._frequencies().to(env.device)

    def _frequencies(self) -> torch.Tensor:
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float32) / self.rotary_dim
        return 1.0 / (self.theta ** exponent)

    def kernel_table(self) -> tuple[torch.Tensor | None, int]:
        return self.inv_freq, self.rotary_dim

    def step_table(self, ctx) -> torch.Tensor | None:
        """cos/sin of every token of this step, made once per step and shared by all layers
        whose encoding has the same frequencies (the reference's fused path keeps the same
        float32 table, miniserve/model/fused.py:183-184)."""
        from .. import ops

        key = ("rope_table", type(self).__name__, self.theta, self.rotary_dim)
        if self.rotary_dim == 0:
            return None
        table = ctx.step_cache.get(key)
        if table is None:
            table = ops.rope_table(ctx.positions, self.inv_freq, ctx.num_tokens, self.rotary_dim, stream=ctx.stream)
            ctx.step_cache[key] = table
        return table


@register_part("position", "rope_pairs")
class RotaryPairs(RotaryNeox):
    """Rotary encoding over adjacent channels: (x[2i], x[2i+1]) turns by position * theta^(-2i / rotary_dim),
    for i < rotary_dim / 2; channels from ``rotary_dim`` on pass unchanged. The frequencies are worked out in
    float64 and rounded once; the angle and its cosine and sine are float32 on the device. Same parameters
    as ``rope_neox``; only the general q|k|v kernel (``ops.qkv_prepare``) takes this pairing."""
    pairing = "adjacent"

    def _frequencies(self) -> torch.Tensor:
        i = torch.arange(0, self.rotary_dim // 2, dtype=torch.float64)
        return (float(self.theta) ** (-2.0 * i / self.rotary_dim)).to(torch.float32)


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q and k pass through unrotated."""
    shape_static = True
    pairing = "halves"

    def kernel_table(self):
        return None, 0

    def step_table(self, ctx):
        return None
