"""Several mixers side by side on the same input, their outputs added with fixed weights."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, build_part, register_part


@register_part("mixer", "parallel")
class ParallelMixers(Part):
    """y = sum_i scale_i * mixer_i(x): every branch reads the same normed input and keeps a cache or state
    of its own (the cache manager hands this part a tuple of views, one per branch). When every branch
    can stop before its output projection (``features`` and ``w_o``), the branches write their scaled
    features side by side into one row and ONE product with the output matrices joined along their
    inputs makes the sum; otherwise the branches' outputs are added one by one.
    Parameters: ``branches``: a sequence of (tensor-name prefix, mixer PartSpec, scale)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        branches = spec["branches"]
        if not branches:
            raise ValueError("a parallel mixer needs at least one branch")
        self.prefixes = [str(p) for p, _, _ in branches]
        self.mixers = [build_part("mixer", s, env) for _, s, _ in branches]
        self.scales = [float(c) for _, _, c in branches]
        self.joint = all(hasattr(m, "features") and hasattr(m, "feature_width") for m in self.mixers)
        if self.joint and any(getattr(m, "general", True) is False for m in self.mixers):
            self.joint = False  # an attention branch on its own fused path has no such stop
        self.w_o = None

    @property
    def shape_static(self) -> bool:
        return all(getattr(m, "shape_static", False) for m in self.mixers)

    def sub_parts(self):
        return dict(zip(self.prefixes, self.mixers))

    def cache_need(self):
        return tuple(m.cache_need() for m in self.mixers)

    def bind_all(self, tensors, prefix: str = "") -> None:
        super().bind_all(tensors, prefix)
        if self.joint:
            w_o = torch.cat([m.w_o for m in self.mixers], dim=1)  # [hidden, sum of feature widths]
            self.feature_width = w_o.shape[1]
            if w_o.shape[1] % 8:  # the product wants rows of whole 16 bytes: zero columns, which meet zero features
                w_o = torch.cat((w_o, torch.zeros((w_o.shape[0], -w_o.shape[1] % 8), dtype=w_o.dtype, device=w_o.device)), dim=1)
            self.w_o = w_o.contiguous()

    def forward(self, x: torch.Tensor, ctx, cache):
        t, dt, dev = x.shape[0], self.env.dtype, x.device
        if self.joint:
            feat = ctx.buffer("par.feat", (t, self.w_o.shape[1]), dt, dev)
            at = 0
            for m, c, scale in zip(self.mixers, cache, self.scales):
                m.features(x, ctx, c, feat[:, at:at + m.feature_width], scale)
                at += m.feature_width
            if at < feat.shape[1]:
                feat[:, at:].zero_()
            return ops.linear(feat, self.w_o, stream=ctx.stream, out=ctx.buffer("par.proj", (t, self.w_o.shape[0]), dt, dev))
        total = None
        for i, (m, c, scale) in enumerate(zip(self.mixers, cache, self.scales)):
            y = m.forward(x, ctx, c)
            if total is None:
                total = ctx.buffer("par.sum", tuple(y.shape), dt, dev)
                ops.axpby(total, y, y, scale, 0.0, stream=ctx.stream)
            else:
                ops.axpby(total, total, y, 1.0, scale, stream=ctx.stream)
        return total
