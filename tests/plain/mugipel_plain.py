"""Plain, slow restatement of the Mugipel decoder, used only as the tests' oracle.

Whole sequences, no cache, no batching, one function per mechanism, nothing imported from the
product package. Everything runs in the dtype of the tensors it is given (the tests hand it
float64 or float32).

Notation: T tokens, W model width, H query heads, G key/value heads, dk key size, dv value size,
R the latent's size. Linear weights are [out, in] and applied as ``x @ w.T``.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- files

def read_config(model_dir) -> dict:
    return json.loads((Path(model_dir) / "config.json").read_text())


def read_weights(model_dir, dtype=torch.float64) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return {k: (v.to(dtype) if v.is_floating_point() else v)
            for k, v in load_file(str(Path(model_dir) / "model.safetensors")).items()}


# --------------------------------------------------------------------------- small pieces

def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the distance of the scale from one."""
    return unit_rms(x, eps) * (1.0 + w)


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def feed_forward(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return relu_squared(h @ up.T) @ down.T


# --------------------------------------------------------------------------- rotation

def yarn_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[torch.Tensor, float]:
    """(frequency of each of the dims/2 pairs, the factor on cos and sin). Without ``scaling`` the
    frequencies are base^(-2i/dims) and the factor is one. With it, pairs that turn fast keep their
    frequency, pairs that turn slowly have it divided by ``factor``, and a linear ramp over the pair
    index joins the two; where the ramp starts and ends follows from how many turns a pair makes
    over ``original`` positions."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_with_turns(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_with_turns(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_with_turns(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, scaling: dict | None) -> torch.Tensor:
    """x [T, heads, d]: channel i < dims/2 turns together with channel i + dims/2 by position * f_i;
    channels from ``dims`` on pass unchanged."""
    if dims == 0:
        return x
    f, mag = yarn_frequencies(dims, base, scaling)
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    c = (torch.cos(ang) * mag).to(x.dtype)[:, None, :]
    s = (torch.sin(ang) * mag).to(x.dtype)[:, None, :]
    half = dims // 2
    a, b = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# --------------------------------------------------------------------------- attention

def visible(t: int, chunk: int | None) -> torch.Tensor:
    """[T, T] bool: query i sees key j <= i, and with ``chunk`` only keys of its own block of ``chunk``
    positions counted from the sequence's start."""
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_attention(q, k, v, scale: float, mask: torch.Tensor, softcap: float | None = None,
                      sink: torch.Tensor | None = None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]. Scores q.k * scale, squashed to
    softcap * tanh(score / softcap) if ``softcap``; ``sink`` [H]: the denominator of head h has one
    more term exp(sink_h) that carries no value (it is neither scaled nor squashed)."""
    t, h, _ = q.shape
    g = k.shape[1]
    out = torch.zeros((t, h, v.shape[2]), dtype=q.dtype)
    for head in range(h):
        kv = head // (h // g)
        s = (q[:, head] @ k[:, kv].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[head].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[head] - m)
        out[:, head] = (e / den) @ v[:, kv]
    return out


def attention_mixer(h: torch.Tensor, w: dict, p: str, m: dict, positions: torch.Tensor) -> torch.Tensor:
    """The 'attention' mixer on its normed input h [T, W]; ``w[p + name]`` are its tensors."""
    t = h.shape[0]
    hq, g, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).view(t, hq, dk)
    k = (h @ w[p + "k"].T).view(t, g, dk)
    v = (h @ w[p + "v"].T).view(t, g, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_halves(q, positions, int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        k = rotate_halves(k, positions, int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    chunk = int(m["mask"]["size"]) if m.get("mask") else None
    a = softmax_attention(q, k, v, float(m["scale"]), visible(t, chunk), m.get("softcap"), w.get(p + "sink"))
    a = a.reshape(t, hq * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return a @ w[p + "o"].T


def latent_attention_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The 'latent_attention' mixer: keys and values of every head are made from one small normed
    vector per token (the only thing a cache would hold); no positions; causal; ordinary softmax."""
    t = h.shape[0]
    hq, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).view(t, hq, dk)
    c = unit_rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).view(t, hq, dk)
    v = (c @ w[p + "uv"].T).view(t, hq, dv)
    a = softmax_attention(q, k, v, float(m["scale"]), visible(t, None))
    a = a.reshape(t, hq * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return a @ w[p + "o"].T


# --------------------------------------------------------------------------- the model

def run_order(cfg: dict) -> list[tuple[int, int | None]]:
    """[(layer, number of the pass if this run opens a pass of the loop else None)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def layer_streams(cfg: dict, w: dict, ids) -> torch.Tensor:
    """The residual stream after every layer run: [runs, T, W]."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x0 = w["embed"][ids]
    x = x0
    outs = []
    for layer, opens in run_order(cfg):
        entry = cfg["layers"][layer]
        p = f"l{layer}."
        if opens is not None:
            x = torch.cat((x, x0), dim=-1) @ w["loop.in"].T + w["loop.step"][opens]
        h = offset_norm(x, w[p + "norm1"], eps)
        if entry["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", entry["mixer"], positions)
        elif entry["type"] == "latent_attention":
            y = latent_attention_mixer(h, w, p + "mix.", entry["mixer"], eps)
        else:
            raise NotImplementedError(entry["type"])
        if entry.get("mlp") is not None:
            y = y + feed_forward(h, w[p + "mlp.up"], w[p + "mlp.down"])
        x = x + mult * y
        outs.append(x)
    return torch.stack(outs)


def all_logits(cfg: dict, w: dict, ids) -> torch.Tensor:
    """Logits at every position: [T, vocab]. The output matrix is the embedding table."""
    x = layer_streams(cfg, w, ids)[-1]
    return offset_norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ w["embed"].T
