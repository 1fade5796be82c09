"""Position encodings that act on q and k inside the attention mixer."""

from __future__ import annotations

import math

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


@register_part("position", "rope_yarn")
class RotaryYarn(RotaryNeox):
    """Rotate-half rotary encoding whose frequencies were rescaled for contexts longer than the ``original`` one:
    with f_i = theta^(-2i / rotary_dim), pair i turns by f_i / factor * r_i + f_i * (1 - r_i), where r_i rises
    linearly from 0 to 1 between the pair that makes ``fast`` turns over ``original`` positions (rounded down) and
    the one that makes ``slow`` turns (rounded up): fast pairs keep their frequency, slow ones have it divided by
    ``factor``. Cosine and sine are both multiplied by 0.1 ln(factor) + 1. Frequencies are worked out in float64 and
    rounded once; the angle and its cosine and sine are float32 on the device. The factor on cos/sin exists only in
    the step's table, so mixers use the kernels that read the table (``table_only``).
    Parameters: those of ``rope_neox`` and ``factor``, ``original``, ``fast``, ``slow``."""
    table_only = True

    def __init__(self, spec, env):
        self.factor = param(spec, "factor", float)
        self.original = param(spec, "original", float)
        self.fast = param(spec, "fast", float)
        self.slow = param(spec, "slow", float)
        if self.factor <= 0 or self.original <= 0 or self.fast <= 0 or self.slow <= 0:
            raise ValueError("rope_yarn: factor, original, fast and slow must be positive")
        self.magnitude = 0.1 * math.log(self.factor) + 1.0
        super().__init__(spec, env)

    def _pair_with_turns(self, turns: float) -> float:
        return self.rotary_dim * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

    def _frequencies(self) -> torch.Tensor:
        i = torch.arange(0, self.rotary_dim // 2, dtype=torch.float64)
        f = float(self.theta) ** (-2.0 * i / self.rotary_dim)
        lo = max(math.floor(self._pair_with_turns(self.fast)), 0)
        hi = min(math.ceil(self._pair_with_turns(self.slow)), self.rotary_dim - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return (f / self.factor * ramp + f * (1.0 - ramp)).to(torch.float32)

    def step_table(self, ctx) -> torch.Tensor | None:
        from .. import ops

        if self.rotary_dim == 0:
            return None
        key = ("rope_table", type(self).__name__, self.theta, self.rotary_dim, self.factor, self.original, self.fast, self.slow)
        table = ctx.step_cache.get(key)
        if table is None:
            table = ops.rope_table_scaled(ctx.positions, self.inv_freq, self.magnitude, ctx.num_tokens, self.rotary_dim, stream=ctx.stream)
            ctx.step_cache[key] = table
        return table


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q and k pass through unrotated."""
    shape_static = True
    pairing = "halves"

    def kernel_table(self):
        return None, 0

    def step_table(self, ctx):
        return None
