"""Helpers of the Mugipel tests: small configurations, a model folder with random weights written from the
checkpoint format alone (names and shapes are stated here, not taken from the product), and the oracle's logits.
The runner that steps the product's own model, cache manager and step function is the one of the Fekulix tests."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch

from tests.fekulix_util import Runner, _RoundedProducts, rel_err  # noqa: F401  (shared, architecture-free)
from tests.plain import mugipel_plain as plain


def attention_layer(heads=4, kv_heads=2, dim=32, vdim=16, rot=8, base=100.0, scaling=True, scale=0.3, softcap=20.0, chunk=24, ff=96):
    rotd = None
    if rot:
        rotd = {"base": base, "dims": rot}
        if scaling:
            rotd["scaling"] = {"factor": 4.0, "fast": 8.0, "original": 64, "slow": 0.5} if scaling is True else dict(scaling)
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if rotd:
        mixer["rot"] = rotd
    if softcap:
        mixer["softcap"] = softcap
    if chunk:
        mixer["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": mixer, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def latent_layer(heads=3, dim=16, vdim=24, rank=40, scale=0.35, ff=64):
    return {"type": "latent_attention", "mixer": {"dim": dim, "heads": heads, "kv_rank": rank, "scale": scale, "vdim": vdim},
            "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def config(layers, width=64, vocab=97, eps=1e-5, mult=0.7, loop=None):
    raw = {"architecture": "Mugipel", "layers": copy.deepcopy(layers), "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab,
           "width": width}
    if loop:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    return raw


def config_a():
    """Both mixers; the last two layers run three times; a layer without feed-forward inside the loop."""
    return config([attention_layer(), latent_layer(), attention_layer(heads=2, kv_heads=2, dim=24, vdim=24, rot=24, chunk=40, ff=None),
                   latent_layer(heads=2, dim=32, vdim=8, rank=16)], loop=(2, 4, 3))


def config_b():
    """Sizes that are no multiples of 8 or 16 where the format allows; the loop starts at the first layer and
    covers everything, once; one kv head under five query heads; no rotation, cap or mask in one layer; a block
    mask shorter than a page; a multiplier of one."""
    return config([
        latent_layer(heads=5, dim=12, vdim=20, rank=36, scale=0.5, ff=52),
        attention_layer(heads=5, kv_heads=1, dim=20, vdim=12, rot=0, softcap=None, chunk=None, scale=0.4, ff=44),
        attention_layer(heads=3, kv_heads=3, dim=16, vdim=40, rot=6, base=37.0, scaling={"factor": 1.5, "fast": 4.0, "original": 16,
                                                                                        "slow": 1.0}, softcap=3.0, chunk=5, ff=36),
    ], width=36, vocab=61, eps=1e-6, mult=1.0, loop=(0, 3, 1))


def config_c():
    """No loop at all; rotation without rescaling; a latent as large as a head of 128; six heads in two groups;
    a block mask that is no multiple of the page."""
    return config([
        attention_layer(heads=6, kv_heads=2, dim=48, vdim=32, rot=32, base=1000.0, scaling=None, softcap=8.0, chunk=50, ff=80),
        latent_layer(heads=2, dim=40, vdim=40, rank=128, scale=0.2, ff=None),
        attention_layer(heads=2, kv_heads=1, dim=64, vdim=64, rot=16, chunk=None, ff=72),
    ], width=56, vocab=83, mult=0.4)


def config_d():
    """Larger and rounder: a width of 288, eight heads in four groups with the whole head of 80 rotated and a smaller
    value size, a latent of 72 in a head of 80, the latent layer first, the first two layers run three times."""
    return config([
        latent_layer(heads=4, dim=32, vdim=96, rank=72, scale=0.2, ff=320),
        attention_layer(heads=8, kv_heads=4, dim=80, vdim=48, rot=80, base=5000.0, scaling={"factor": 8.0, "fast": 16.0, "original": 128,
                                                                                           "slow": 2.0}, softcap=15.0, chunk=128, ff=320),
        attention_layer(heads=4, kv_heads=4, dim=64, vdim=64, rot=32, chunk=96, softcap=None, ff=192),
        latent_layer(heads=8, dim=48, vdim=32, rank=64, scale=0.15, ff=None),
    ], width=288, vocab=640, mult=0.5, loop=(0, 2, 3))


def tensor_shapes(raw) -> dict[str, tuple]:
    """Names and shapes of a checkpoint of this configuration."""
    w = raw["width"]
    out = {"embed": (raw["vocab"], w), "final.norm": (w,)}
    if raw.get("loop"):
        out["loop.in"], out["loop.step"] = (w, 2 * w), (raw["loop"]["times"], w)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (w,)
        if layer["mlp"] is not None:
            out[p + "mlp.up"], out[p + "mlp.down"] = (layer["mlp"]["ff"], w), (w, layer["mlp"]["ff"])
        q, h, dk, dv = p + "mix.", m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            g = m["kv_heads"]
            out.update({q + "q": (h * dk, w), q + "k": (g * dk, w), q + "v": (g * dv, w), q + "sink": (h,), q + "g": (h * dv, w),
                        q + "o": (w, h * dv)})
        else:
            r = m["kv_rank"]
            out.update({q + "q": (h * dk, w), q + "dkv": (r, w), q + "dkv.norm": (r,), q + "uk": (h * dk, r), q + "uv": (h * dv, r),
                        q + "g": (h * dv, w), q + "o": (w, h * dv)})
    return out


def random_weights(raw, seed: int, sharpen: float = 2.5) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices about 1/sqrt(fan-in) so that activations are of size one, the query and key side
    times ``sharpen`` so that attention is peaked, norm weights around zero, sinks around zero."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(raw).items():
        leaf = name.rsplit(".", 1)[-1]
        if name == "loop.step":
            t = 0.3 * torch.randn(shape, generator=gen)
        elif len(shape) == 2:
            t = torch.randn(shape, generator=gen) * (1.2 / shape[1] ** 0.5)
            if leaf in ("q", "k", "uk"):
                t = t * sharpen ** 0.5
        elif leaf == "sink":
            t = torch.randn(shape, generator=gen)
        elif name.endswith("dkv.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        else:  # norm weights, stored as the distance from one
            t = 0.2 * torch.randn(shape, generator=gen)
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, raw, seed: int, sharpen: float = 2.5) -> Path:
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw, indent=1))
    save_file(random_weights(raw, seed, sharpen), str(folder / "model.safetensors"))
    return folder


def oracle(folder, dtype=torch.float64):
    cfg, w = plain.read_config(folder), plain.read_weights(folder, dtype)
    return lambda ids: plain.all_logits(cfg, w, ids)


def rounding_noise(folder, ids) -> float:
    """rel_err of the oracle against itself when every matrix product's result is rounded to bfloat16:
    what rounding alone costs on this model and these tokens (the engine rounds in more places)."""
    cfg, w = plain.read_config(folder), plain.read_weights(folder, torch.float64)
    exact = plain.all_logits(cfg, w, ids)
    rounded = {k: (v.as_subclass(_RoundedProducts) if v.dim() == 2 and k not in ("embed", "loop.step") else v) for k, v in w.items()}
    return rel_err(torch.as_tensor(plain.all_logits(cfg, rounded, ids)).as_subclass(torch.Tensor), exact)
