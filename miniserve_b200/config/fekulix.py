"""Typed configuration of the Fekulix decoder, read from its config.json.

config.json carries ``architecture``, ``width``, ``vocab``, ``logit_scale``, ``norm.eps`` and ``layers``:
one entry per layer with ``type`` (``parallel`` or ``channel_delta``), the mixer's sizes and constants
under ``mixer``, the feed-forward under ``mlp`` (``{"kind": "dense", "ff": n}`` or null), and optionally
``weights_of``: the index of the layer whose tensors this one runs with (a cache and state of its own).
The ranks of the low-rank projections are not in config.json; they are the first dimension of the
tensors ``a1`` / ``g1`` (``complete`` fills them in from the checkpoint's shapes; a configuration made by
hand, for random weights, names them as ``decay_rank`` / ``gate_rank`` in the mixer's entry).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

LAYER_TYPES = ("parallel", "channel_delta")


@dataclass(frozen=True)
class FekulixLayer:
    type: str
    mixer: Mapping[str, Any]
    ff: int | None  # None: no feed-forward
    weights_of: int | None


@dataclass(frozen=True)
class FekulixConfig:
    width: int
    vocab: int
    eps: float
    logit_scale: float
    layers: tuple[FekulixLayer, ...]
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FekulixConfig":
        missing = [k for k in ("width", "vocab", "layers", "norm") if k not in raw]
        if missing:
            raise KeyError(f"config.json lacks {missing}")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            kind = entry.get("type")
            if kind not in LAYER_TYPES:
                raise NotImplementedError(f"layer {i}: type {kind!r} is not one of {LAYER_TYPES}")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not supported")
            of = entry.get("weights_of")
            if of is not None:
                of, seen = int(of), {i}
                while 0 <= of < len(raw["layers"]) and of not in seen and raw["layers"][of].get("weights_of") is not None:
                    seen.add(of)  # a layer that borrows from a borrower runs with the tensors at the end of the chain
                    of = int(raw["layers"][of]["weights_of"])
                if not 0 <= of < len(raw["layers"]) or of in seen:
                    raise ValueError(f"layer {i}: weights_of={entry.get('weights_of')} must lead to another layer that has tensors of its own")
                if raw["layers"][of].get("type") != kind:
                    raise ValueError(f"layer {i} ({kind}) cannot run with the weights of layer {of} ({raw['layers'][of].get('type')})")
            layers.append(FekulixLayer(kind, entry["mixer"], int(mlp["ff"]) if mlp is not None else None, of))
        cfg = cls(width=int(raw["width"]), vocab=int(raw["vocab"]), eps=float(raw["norm"]["eps"]),
                  logit_scale=float(raw.get("logit_scale", 1.0)), layers=tuple(layers), raw=raw)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.width < 1 or self.vocab < 1 or not self.layers:
            raise ValueError("width, vocab and the number of layers must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "parallel":
                left, right = m["left"], m["right"]
                if int(left["heads"]) % int(left["kv_heads"]):
                    raise ValueError(f"layer {i}: {left['heads']} heads are not a multiple of {left['kv_heads']} kv heads")
                rot = int(left["rot"]["dims"])
                if rot % 2 or rot > int(left["dim"]):
                    raise ValueError(f"layer {i}: rot.dims={rot} must be even and at most dim={left['dim']}")
                if "decay_rank" not in right:
                    raise KeyError(f"layer {i}: the rank of the decay's projection is unknown (no checkpoint, no 'decay_rank')")
            else:
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ValueError(f"layer {i}: {m['heads']} heads are not a multiple of {m['kv_heads']} query/key heads")
                for key in ("decay_rank", "gate_rank"):
                    if key not in m:
                        raise KeyError(f"layer {i}: the rank {key!r} is unknown (no checkpoint, and not in the mixer's entry)")


def complete_from_shapes(raw: Mapping[str, Any], shapes: Mapping[str, tuple]) -> dict[str, Any]:
    """The ranks of the low-rank projections, read off the checkpoint's tensor shapes."""
    raw = copy.deepcopy(dict(raw))
    for i, entry in enumerate(raw.get("layers", [])):
        src, hops = i, 0
        while raw["layers"][src].get("weights_of") is not None and hops <= len(raw["layers"]):
            src, hops = int(raw["layers"][src]["weights_of"]), hops + 1
        m = entry.get("mixer", {})
        if entry.get("type") == "parallel":
            name = f"l{src}.mix.right.a1"
            if "decay_rank" not in m.get("right", {}) and name in shapes:
                m["right"]["decay_rank"] = int(shapes[name][0])
        elif entry.get("type") == "channel_delta":
            for key, tensor in (("decay_rank", "a1"), ("gate_rank", "g1")):
                name = f"l{src}.mix.{tensor}"
                if key not in m and name in shapes:
                    m[key] = int(shapes[name][0])
            name = f"l{src}.mix.q.conv"
            if "conv" not in m and name in shapes:  # the taps are the convolution tensor's second dimension
                m["conv"] = int(shapes[name][1])
    return raw
