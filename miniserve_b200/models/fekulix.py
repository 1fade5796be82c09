"""The Fekulix decoder as data: its configuration mapped onto parts.

Pre-norm layers whose norm is Dynamic Tanh; two kinds of mixer, ``parallel`` (softmax attention with a
sink, per-head output gate, q/k norm and partial rotary over adjacent channels, beside linear attention
with a per-channel decay; their outputs added with fixed weights) and ``channel_delta`` (the gated delta
rule behind short convolutions); a dense tanh-GELU feed-forward or none; a layer may run with another
layer's tensors and a cache of its own (the run order names the owning layer); the logits are scaled.
Tensor names are the checkpoint's: ``embed``, ``l<i>.norm1[.b|.alpha]``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.fekulix import FekulixConfig, complete_from_shapes
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

NORM_NAMES = dict(weight="", bias=".b", alpha=".alpha")


def _softmax_branch(width: int, eps: float, c) -> PartSpec:
    return PartSpec("gqa_attention", dict(
        hidden=width, heads=int(c["heads"]), kv_heads=int(c["kv_heads"]), head_dim=int(c["dim"]), value_dim=int(c["vdim"]),
        qk_norm=True, qk_norm_eps=eps, scale=float(c["scale"]), sink=True, out_gate="head_sigmoid",
        position=PartSpec("rope_pairs", dict(head_dim=int(c["dim"]), theta=float(c["rot"]["base"]), rotary_dim=int(c["rot"]["dims"]))),
        names=dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", gate="g")))


def _linear_branch(width: int, eps: float, c) -> PartSpec:
    return PartSpec("decay_linear_attention", dict(
        hidden=width, heads=int(c["heads"]), key_dim=int(c["dim"]), value_dim=int(c["vdim"]), tau=float(c["tau"]),
        decay_rank=int(c["decay_rank"]), eps=eps,
        names=dict(q="q", k="k", v="v", g="g", o="o", norm="norm", a1="a1", a2="a2", a_bias="a2.b")))


def _mixer(width: int, eps: float, layer) -> PartSpec:
    m = layer.mixer
    if layer.type == "parallel":
        return PartSpec("parallel", dict(branches=(
            ("left.", _softmax_branch(width, eps, m["left"]), float(m["left_scale"])),
            ("right.", _linear_branch(width, eps, m["right"]), float(m["right_scale"])))))
    return PartSpec("gated_delta_rule", dict(
        hidden=width, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), key_dim=int(m["dim"]), value_dim=int(m["vdim"]),
        conv=int(m["conv"]), decay_rank=int(m["decay_rank"]), gate_rank=int(m["gate_rank"]), eps=eps, unit_eps=1e-6,
        names=dict(q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", beta="b", a_log="A_log",
                   norm="norm", a1="a1", a2="a2", dt_bias="dt_bias", g1="g1", g2="g2", o="o")))


def fekulix_model_spec(cfg: FekulixConfig) -> ModelSpec:
    norm = PartSpec("dynamic_tanh", dict(size=cfg.width, names=NORM_NAMES))
    layers: list[LayerSpec] = []
    index_of: dict[int, int] = {}  # config layer -> index among the layers that have tensors
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        ffn = None
        if layer.ff is not None:
            ffn = PartSpec("dense_mlp", dict(hidden=cfg.width, intermediate=layer.ff, activation="gelu_tanh",
                                             names=dict(up="up", down="down")))
        names = dict(mixer="mix.", norm1="norm1")
        norms = dict(norm1=norm)
        if ffn is not None:
            names.update(feed_forward="mlp.", norm2="norm2")
            norms["norm2"] = norm
        index_of[i] = len(layers)
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm", dict(names=names)),
                                mixer=_mixer(cfg.width, cfg.eps, layer), feed_forward=ffn, norms=norms))
    run_order = tuple(RunEntry(index_of[layer.weights_of if layer.weights_of is not None else i])
                      for i, layer in enumerate(cfg.layers))
    return ModelSpec(
        architecture="Fekulix", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=cfg.width, name="embed")),
        layers=tuple(layers), run_order=run_order, final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear_head", dict(vocab=cfg.vocab, hidden=cfg.width, tied=False, name="head", scale=cfg.logit_scale)))


FEKULIX = register_architecture(
    Architecture("Fekulix", FekulixConfig.from_dict, fekulix_model_spec, complete=complete_from_shapes), replace=True)
