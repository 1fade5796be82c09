"""Arrangements of mixer, feed-forward and norms into one layer."""

from __future__ import annotations

from ..config.spec import LayerSpec
from .base import BuildEnv, Part, ResidualStream, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Part):
    """h += mixer(norm1(h)); h += feed_forward(norm2(h)) (miniserve/model/qwen3.py:212-216).
    The adds are fused into the norm that follows them, so the block hands its last addend
    on as ``pending``. Parameters: ``names`` maps mixer / feed_forward / norm1 / norm2 to their
    tensor-name prefixes inside the layer. A layer without a feed-forward (``LayerSpec.feed_forward`` None)
    has neither it nor norm2, and hands the mixer's output on as the pending addend."""
    shape_static = True

    def __init__(self, spec, env: BuildEnv, layer: LayerSpec | None = None):
        super().__init__(spec, env)
        if layer is None:
            raise ValueError("a block is built from its LayerSpec (use build_block)")
        names = dict(spec.get("names") or {})
        self.has_ff = layer.feed_forward is not None
        self.names = {k: names[k] for k in ("mixer", "norm1") + (("feed_forward", "norm2") if self.has_ff else ())}
        self.mixer = build_part("mixer", layer.mixer, env)
        self.norm1 = build_part("norm", layer.norms["norm1"], env)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, env) if self.has_ff else None
        self.norm2 = build_part("norm", layer.norms["norm2"], env) if self.has_ff else None

    def sub_parts(self):
        out = {self.names["mixer"]: self.mixer, self.names["norm1"]: self.norm1}
        if self.has_ff:
            out.update({self.names["feed_forward"]: self.feed_forward, self.names["norm2"]: self.norm2})
        return out

    def forward(self, stream: ResidualStream, ctx, cache) -> ResidualStream:
        total = stream.total
        x = self.norm1.forward(total, stream.pending, ctx)
        a = self.mixer.forward(x, ctx, cache)
        if not self.has_ff:
            return ResidualStream(total, a)
        x = self.norm2.forward(total, a, ctx)
        return ResidualStream(total, self.feed_forward.forward(x, ctx))



def build_block(layer: LayerSpec, env: BuildEnv) -> Part:
    from .base import _REGISTRY

    try:
        cls = _REGISTRY["block"][layer.block.kind]
    except KeyError:
        raise ValueError(f"no block arrangement named {layer.block.kind!r}; registered: {sorted(_REGISTRY['block'])}") from None
    return cls(layer.block, env, layer)
