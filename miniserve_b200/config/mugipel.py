"""Typed configuration of the Mugipel decoder, read from its config.json.

config.json carries ``architecture``, ``width``, ``vocab``, ``norm.eps``, ``residual_mult``, ``layers`` and
optionally ``loop``. A layer entry has ``type`` (``attention`` or ``latent_attention``), the mixer's sizes and
constants under ``mixer`` and the feed-forward under ``mlp`` (``{"kind": "dense", "ff": n}`` or null).
``loop`` = ``{"start": a, "stop": b, "times": n}``: layers a .. b-1 run n times in a row with the same tensors
and a cache of their own each time; before every pass the stream re-enters through a product with the
embedding beside it (tensors ``loop.in``, ``loop.step``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

LAYER_TYPES = ("attention", "latent_attention")


@dataclass(frozen=True)
class MugipelLayer:
    type: str
    mixer: Mapping[str, Any]
    ff: int | None  # None: no feed-forward


@dataclass(frozen=True)
class MugipelLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MugipelConfig:
    width: int
    vocab: int
    eps: float
    residual_mult: float
    layers: tuple[MugipelLayer, ...]
    loop: MugipelLoop | None
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MugipelConfig":
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
            layers.append(MugipelLayer(kind, entry["mixer"], int(mlp["ff"]) if mlp is not None else None))
        loop = raw.get("loop")
        if loop is not None:
            loop = MugipelLoop(int(loop["start"]), int(loop["stop"]), int(loop["times"]))
        cfg = cls(width=int(raw["width"]), vocab=int(raw["vocab"]), eps=float(raw["norm"]["eps"]),
                  residual_mult=float(raw.get("residual_mult", 1.0)), layers=tuple(layers), loop=loop, raw=raw)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.width < 1 or self.vocab < 1 or not self.layers:
            raise ValueError("width, vocab and the number of layers must be positive")
        if self.loop is not None:
            lp = self.loop
            if not 0 <= lp.start < lp.stop <= len(self.layers) or lp.times < 1:
                raise ValueError(f"loop {lp.start}..{lp.stop} x {lp.times} does not fit {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "attention":
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ValueError(f"layer {i}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
                rot = m.get("rot")
                if rot is not None and (int(rot["dims"]) % 2 or int(rot["dims"]) > int(m["dim"])):
                    raise ValueError(f"layer {i}: rot.dims={rot['dims']} must be even and at most dim={m['dim']}")
                mask = m.get("mask")
                if mask is not None and int(mask["size"]) < 1:
                    raise ValueError(f"layer {i}: mask.size={mask['size']} must be positive")
            else:
                for key in ("heads", "dim", "vdim", "kv_rank"):
                    if int(m[key]) < 1:
                        raise ValueError(f"layer {i}: {key}={m[key]} must be positive")

    def run_layers(self) -> list[tuple[int, int | None]]:
        """The order in which layers run: (layer, number of the pass if this run opens a pass of the loop else None)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        order: list[tuple[int, int | None]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            order += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return order + [(i, None) for i in range(lp.stop, n)]
