"""The Mugipel decoder as data: its configuration mapped onto parts.

Layers in which the mixer and the feed-forward read one normed input and their sum enters the stream times a
constant; an RMS norm whose weight is stored as its distance from one; two kinds of mixer, ``attention``
(grouped heads, part of each head rotated by halves with frequencies rescaled for longer contexts, capped
scores, a mask by blocks of positions, a learned sink per head, a sigmoid gate per channel) and
``latent_attention`` (keys and values of all heads made from one small normed vector per token, the only thing
cached; no positions); a dense feed-forward with squared ReLU or none; a stretch of layers that runs several
times with the same tensors, the stream re-entering before each pass through a product with the embedding
beside it; logits through the embedding table. Tensor names are the checkpoint's: ``embed``, ``loop.in``,
``loop.step``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``, ``final.norm``.
"""

from __future__ import annotations

from ..config.mugipel import MugipelConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _position(c) -> PartSpec:
    rot = c.get("rot")
    if not rot or int(rot["dims"]) == 0:
        return PartSpec("none")
    params = dict(head_dim=int(c["dim"]), theta=float(rot["base"]), rotary_dim=int(rot["dims"]))
    # without rescaling: a factor of one leaves every frequency and the factor on cos and sin as they are
    scaling = rot.get("scaling") or {"factor": 1.0, "original": 1.0, "fast": 1.0, "slow": 1.0}
    params.update(factor=float(scaling["factor"]), original=float(scaling["original"]), fast=float(scaling["fast"]),
                  slow=float(scaling["slow"]))
    return PartSpec("rope_yarn", params)


def _attention(width: int, c) -> PartSpec:
    mask = c.get("mask")
    return PartSpec("gqa_attention", dict(
        hidden=width, heads=int(c["heads"]), kv_heads=int(c["kv_heads"]), head_dim=int(c["dim"]), value_dim=int(c["vdim"]),
        qk_norm=False, scale=float(c["scale"]), softcap=float(c["softcap"]) if c.get("softcap") else None,
        chunk=int(mask["size"]) if mask else None, sink="learned", out_gate="channel_sigmoid", position=_position(c),
        names=dict(q="q", k="k", v="v", o="o", gate="g", sink="sink")))


def _latent(width: int, eps: float, c) -> PartSpec:
    return PartSpec("latent_attention", dict(
        hidden=width, heads=int(c["heads"]), head_dim=int(c["dim"]), value_dim=int(c["vdim"]), latent=int(c["kv_rank"]),
        scale=float(c["scale"]), eps=eps,
        names=dict(q="q", down="dkv", norm="dkv.norm", up_k="uk", up_v="uv", gate="g", o="o")))


def mugipel_model_spec(cfg: MugipelConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.eps, unit_offset=True, name=""))
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer = _attention(cfg.width, layer.mixer) if layer.type == "attention" else _latent(cfg.width, cfg.eps, layer.mixer)
        ffn = None
        names = dict(mixer="mix.", norm1="norm1")
        if layer.ff is not None:
            ffn = PartSpec("dense_mlp", dict(hidden=cfg.width, intermediate=layer.ff, activation="relu_squared",
                                             names=dict(up="up", down="down")))
            names["feed_forward"] = "mlp."
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("parallel_residual", dict(names=names, residual_mult=cfg.residual_mult)),
                                mixer=mixer, feed_forward=ffn, norms=dict(norm1=norm)))
    transitions = ()
    if cfg.loop is not None:
        transitions = (PartSpec("stream_reentry", dict(hidden=cfg.width, passes=cfg.loop.times, weight="loop.in", step="loop.step")),)
    run_order = tuple(RunEntry(layer, transition=None if opens is None else 0, transition_arg=opens or 0)
                      for layer, opens in cfg.run_layers())
    return ModelSpec(
        architecture="Mugipel", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=cfg.width, name="embed")),
        layers=tuple(layers), run_order=run_order, final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear_head", dict(vocab=cfg.vocab, hidden=cfg.width, tied=True, tied_to="embed", name="head")),
        transitions=transitions)


MUGIPEL = register_architecture(Architecture("Mugipel", MugipelConfig.from_dict, mugipel_model_spec), replace=True)
