"""Plain, slow restatement of the Fekulix decoder, used only as the tests' oracle.

Whole sequences, no cache, no batching, token-by-token recurrences, one function per mechanism,
nothing imported from the product package. Everything runs in the dtype of the tensors it is
given (the tests hand it float64 or float32).

Notation: T tokens, W model width, H heads, G key/value (or query/key) heads, dk key size,
dv value size. Linear weights are [out, in] and applied as ``x @ w.T``.
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

    return {k: v.to(dtype) for k, v in load_file(str(Path(model_dir) / "model.safetensors")).items()}


# --------------------------------------------------------------------------- small pieces

def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def dynamic_tanh(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """tanh(alpha x) w + b: a norm that takes no statistics."""
    return torch.tanh(alpha * x) * w + b


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: channels (2i, 2i+1), i < dims/2, turn by the angle position * base^(-2i/dims);
    channels from ``dims`` on pass unchanged."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps]; y[t, c] = sum_j w[c, j] x[t - (taps - 1 - j), c], zeros before the start."""
    t, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < t:
            y[back:] += x[:t - back] * w[:, j]
    return y


# --------------------------------------------------------------------------- mixers

def sink_attention(q, k, v, scale: float) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]. Causal; the weights of row t are
    exp(s_j) / (1 + sum_j exp(s_j)): one more term in the denominator that carries no value."""
    t, h, _ = q.shape
    g = k.shape[1]
    out = torch.zeros(t, h, v.shape[2], dtype=q.dtype)
    for head in range(h):
        kv = head // (h // g)
        s = (q[:, head] @ k[:, kv].T) * scale
        s = s.masked_fill(torch.ones(t, t, dtype=torch.bool).triu(1), float("-inf"))
        m = torch.clamp(s.max(dim=1, keepdim=True).values, min=0.0)
        e = torch.exp(s - m)
        p = e / (torch.exp(-m) + e.sum(dim=1, keepdim=True))
        out[:, head] = p @ v[:, kv]
    return out


def softmax_branch(h, positions, w, p, c, eps):
    """The 'left' mixer. ``w(name)`` gives a tensor of the branch, ``c`` its config entry."""
    t = h.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ w("q").T).view(t, H, dk)
    k = (h @ w("k").T).view(t, G, dk)
    v = (h @ w("v").T).view(t, G, dv)
    q = unit_rms(q, eps) * w("q.norm")
    k = unit_rms(k, eps) * w("k.norm")
    q = rotate_pairs(q, positions, c["rot"]["dims"], c["rot"]["base"])
    k = rotate_pairs(k, positions, c["rot"]["dims"], c["rot"]["base"])
    o = sink_attention(q, k, v, c["scale"])
    gate = torch.sigmoid(h @ w("g").T)  # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(t, H * dv) @ w("o").T


def decay_recurrence(q, k, v, a):
    """q, k, a [T, H, dk], v [T, H, dv]. S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    t, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=q.dtype)
    out = torch.zeros(t, H, dv, dtype=q.dtype)
    for i in range(t):
        S = a[i][:, :, None] * S + k[i][:, :, None] * v[i][:, None, :]
        out[i] = torch.einsum("hkv,hk->hv", S, q[i])
    return out


def linear_branch(h, w, c, eps):
    """The 'right' mixer: linear attention with a decay per key channel."""
    t = h.shape[0]
    H, dk, dv = c["heads"], c["dim"], c["vdim"]
    q = (h @ w("q").T).view(t, H, dk) * dk ** -0.5
    k = (h @ w("k").T).view(t, H, dk)
    v = (h @ w("v").T).view(t, H, dv)
    z = (h @ w("a1").T) @ w("a2").T + w("a2.b")
    a = (torch.sigmoid(z) ** (1.0 / c["tau"])).view(t, H, dk)
    o = decay_recurrence(q, k, v, a)
    o = unit_rms(o, eps) * w("norm")
    o = o.reshape(t, H * dv) * silu(h @ w("g").T)
    return o @ w("o").T


def parallel_mixer(h, positions, w, c, eps):
    left = softmax_branch(h, positions, lambda n: w("left." + n), None, c["left"], eps)
    right = linear_branch(h, lambda n: w("right." + n), c["right"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


def delta_recurrence(q, k, v, beta, g):
    """q, k, g [T, H, dk], v [T, H, dv], beta [T, H]. Per head and token:
    S <- g S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    t, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=q.dtype)
    out = torch.zeros(t, H, dv, dtype=q.dtype)
    for i in range(t):
        S = g[i][:, :, None] * S
        u = beta[i][:, None] * (v[i] - torch.einsum("hkv,hk->hv", S, k[i]))
        S = S + k[i][:, :, None] * u[:, None, :]
        out[i] = torch.einsum("hkv,hk->hv", S, q[i])
    return out


def channel_delta_mixer(h, w, c, eps):
    t = h.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(causal_conv(h @ w("q").T, w("q.conv"))).view(t, G, dk)
    k = silu(causal_conv(h @ w("k").T, w("k.conv"))).view(t, G, dk)
    v = silu(causal_conv(h @ w("v").T, w("v.conv"))).view(t, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ w("b").T)  # [T, H]
    step = torch.nn.functional.softplus((h @ w("a1").T) @ w("a2").T + w("dt_bias")).view(t, H, dk)
    g = torch.exp(-torch.exp(w("A_log"))[None, :, None] * step)
    o = delta_recurrence(q, k, v, beta, g)
    gate = torch.sigmoid((h @ w("g1").T) @ w("g2").T).view(t, H, dv)
    o = unit_rms(o, eps) * w("norm") * gate
    return o.reshape(t, H * dv) @ w("o").T


def dense_ff(h, w):
    return gelu_tanh(h @ w("up").T) @ w("down").T


# --------------------------------------------------------------------------- the model

def layer_outputs(cfg: dict, weights: dict, ids) -> tuple[torch.Tensor, torch.Tensor]:
    """(residual stream after every layer run [runs, T, W], logits [T, vocab])."""
    eps = cfg["norm"]["eps"]
    x = weights["embed"][torch.as_tensor(list(ids), dtype=torch.long)]
    positions = torch.arange(x.shape[0])
    after = []

    def norm(name, y):
        return dynamic_tanh(y, weights[name], weights[name + ".b"], weights[name + ".alpha"])

    for i, layer in enumerate(cfg["layers"]):
        src = i
        while cfg["layers"][src].get("weights_of") is not None:  # a layer may run with another layer's tensors
            src = cfg["layers"][src]["weights_of"]
        pre = f"l{src}."
        w = lambda n, pre=pre: weights[pre + "mix." + n]
        h = norm(pre + "norm1", x)
        if layer["type"] == "parallel":
            x = x + parallel_mixer(h, positions, w, layer["mixer"], eps)
        elif layer["type"] == "channel_delta":
            x = x + channel_delta_mixer(h, w, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            x = x + dense_ff(norm(pre + "norm2", x), lambda n, pre=pre: weights[pre + "mlp." + n])
        after.append(x)
    logits = norm("final.norm", x) @ weights["head"].T * cfg["logit_scale"]
    return torch.stack(after), logits


def all_logits(cfg: dict, weights: dict, ids) -> torch.Tensor:
    return layer_outputs(cfg, weights, ids)[1]
