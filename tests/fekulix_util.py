"""Helpers of the Fekulix tests: small configurations, a model folder with random weights written
from the checkpoint format alone (names and shapes are stated here, not taken from the product), the
oracle's logits, and a runner that steps the product's own model, cache manager and step function."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch

from tests.plain import fekulix_plain as plain


def parallel_layer(heads=4, kv_heads=2, dim=32, vdim=16, rot=8, base=100.0, scale=0.25, r_heads=2, r_dim=24, r_vdim=40,
                   tau=4.0, left_scale=0.7, right_scale=1.3, ff=96, decay_rank=8, weights_of=None):
    layer = {"type": "parallel",
             "mixer": {"left": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": {"base": base, "dims": rot},
                                "scale": scale, "vdim": vdim},
                       "left_scale": left_scale,
                       "right": {"dim": r_dim, "heads": r_heads, "tau": tau, "vdim": r_vdim, "decay_rank": decay_rank},
                       "right_scale": right_scale},
             "mlp": {"ff": ff, "kind": "dense"} if ff else None}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, ff=None, decay_rank=8, gate_rank=16, weights_of=None):
    layer = {"type": "channel_delta",
             "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim,
                       "decay_rank": decay_rank, "gate_rank": gate_rank},
             "mlp": {"ff": ff, "kind": "dense"} if ff else None}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def config(layers, width=64, vocab=97, eps=1e-5, logit_scale=1.5):
    return {"architecture": "Fekulix", "layers": copy.deepcopy(layers), "logit_scale": logit_scale, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def config_a():
    """Both mixers, a layer without feed-forward, both kinds run twice with shared tensors."""
    return config([parallel_layer(), delta_layer(), parallel_layer(weights_of=0), delta_layer(weights_of=1)])


def config_b():
    """Sizes that are no multiples of 8 or 16 where the format allows, one kv head, one linear head,
    the whole key rotated, ranks 5, 3 and 7, two taps, and a convolution of a single tap."""
    return config([
        parallel_layer(heads=3, kv_heads=1, dim=16, vdim=40, rot=16, base=37.0, scale=0.4, r_heads=1, r_dim=40, r_vdim=8,
                       tau=9.0, left_scale=1.0, right_scale=1.0, ff=40, decay_rank=5),
        delta_layer(heads=2, kv_heads=2, dim=40, vdim=12, conv=2, ff=56, decay_rank=3, gate_rank=7),
        delta_layer(heads=3, kv_heads=1, dim=8, vdim=16, conv=1, ff=None, decay_rank=8, gate_rank=8),
    ], width=48, vocab=61, eps=1e-6, logit_scale=0.5)


def config_c():
    """A width and feed-forward sizes that are no multiples of 8, key sizes that are no multiples of 8
    (the recurrence stages them element by element), five heads, a layer that borrows from a borrower."""
    return config([
        delta_layer(heads=5, kv_heads=5, dim=12, vdim=20, conv=4, ff=52, decay_rank=6, gate_rank=10),
        parallel_layer(heads=5, kv_heads=5, dim=24, vdim=24, rot=6, base=1000.0, scale=0.3, r_heads=3, r_dim=20, r_vdim=12,
                       tau=2.0, left_scale=0.5, right_scale=2.0, ff=None, decay_rank=4),
        delta_layer(weights_of=0, heads=5, kv_heads=5, dim=12, vdim=20, conv=4, ff=52, decay_rank=6, gate_rank=10),
        delta_layer(weights_of=2, heads=5, kv_heads=5, dim=12, vdim=20, conv=4, ff=52, decay_rank=6, gate_rank=10),
    ], width=36, vocab=53, eps=1e-5, logit_scale=3.0)


def tensor_shapes(raw) -> dict[str, tuple]:
    """Names and shapes of a checkpoint of this configuration."""
    w = raw["width"]
    out = {"embed": (raw["vocab"], w), "head": (raw["vocab"], w)}

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (w,), (w,), ()

    norm("final.norm")
    for i, layer in enumerate(raw["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        norm(p + "norm1")
        if layer["mlp"] is not None:
            norm(p + "norm2")
            out[p + "mlp.up"], out[p + "mlp.down"] = (layer["mlp"]["ff"], w), (w, layer["mlp"]["ff"])
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            q = p + "mix.left."
            out.update({q + "q": (a["heads"] * a["dim"], w), q + "k": (a["kv_heads"] * a["dim"], w),
                        q + "v": (a["kv_heads"] * a["vdim"], w), q + "q.norm": (a["dim"],), q + "k.norm": (a["dim"],),
                        q + "g": (a["heads"], w), q + "o": (w, a["heads"] * a["vdim"])})
            q = p + "mix.right."
            out.update({q + "q": (b["heads"] * b["dim"], w), q + "k": (b["heads"] * b["dim"], w),
                        q + "v": (b["heads"] * b["vdim"], w), q + "g": (b["heads"] * b["vdim"], w),
                        q + "o": (w, b["heads"] * b["vdim"]), q + "norm": (b["vdim"],), q + "a1": (b["decay_rank"], w),
                        q + "a2": (b["heads"] * b["dim"], b["decay_rank"]), q + "a2.b": (b["heads"] * b["dim"],)})
        else:
            q, h, g, dk, dv = p + "mix.", m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({q + "q": (g * dk, w), q + "q.conv": (g * dk, m["conv"]), q + "k": (g * dk, w),
                        q + "k.conv": (g * dk, m["conv"]), q + "v": (h * dv, w), q + "v.conv": (h * dv, m["conv"]),
                        q + "b": (h, w), q + "A_log": (h,), q + "norm": (dv,), q + "a1": (m["decay_rank"], w),
                        q + "a2": (h * dk, m["decay_rank"]), q + "dt_bias": (h * dk,), q + "g1": (m["gate_rank"], w),
                        q + "g2": (h * dv, m["gate_rank"]), q + "o": (w, h * dv)})
    return out


def random_weights(raw, seed: int, sharpen: float = 3.0) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices about 1/sqrt(fan-in) so that activations are of size one, norm scales
    about one, the q/k norm scales times ``sharpen`` so that attention is peaked, decays spread out."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(raw).items():
        leaf = name.rsplit(".", 1)[-1]
        if len(shape) == 2 and not name.endswith(".conv"):
            t = torch.randn(shape, generator=gen) * (1.2 / shape[1] ** 0.5)
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=gen) * 0.6
        elif leaf == "alpha":
            t = 0.6 + 0.2 * torch.rand(shape, generator=gen)
        elif leaf in ("b", "dt_bias"):  # biases (a norm's, a decay's)
            t = 0.3 * torch.randn(shape, generator=gen)
        elif leaf == "A_log":
            t = torch.randn(shape, generator=gen) * 0.5 - 0.5
        else:  # norm scales
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
            if name.endswith("q.norm") or name.endswith("k.norm"):
                t = t * sharpen
        out[name] = t.to(torch.bfloat16)
    return out


def stored_config(raw) -> dict:
    """config.json as a checkpoint carries it: without the ranks, which the tensors' shapes give."""
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
        layer["mixer"].get("right", {}).pop("decay_rank", None)
    return raw


def write_model(folder, raw, seed: int, sharpen: float = 3.0) -> Path:
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(stored_config(raw), indent=1))
    save_file(random_weights(raw, seed, sharpen), str(folder / "model.safetensors"))
    return folder


def oracle(folder, dtype=torch.float64):
    cfg, w = plain.read_config(folder), plain.read_weights(folder, dtype)
    return lambda ids: plain.all_logits(cfg, w, ids)


class Runner:
    """Steps the product's model through its cache manager and step function, as the trace runner does."""

    def __init__(self, folder, dtype: str, max_tokens: int = 512, page_size: int = 16, max_requests: int = 4, poison=True):
        from miniserve_b200.cache import CacheManager
        from miniserve_b200.engine.loader import load_model
        from miniserve_b200.engine.step import StepFunction

        _, _, self.model = load_model(folder, dtype, "cuda:0")
        self.cache = CacheManager(self.model.entry_caches, max(1, -(-max_tokens // page_size)), page_size, max_requests,
                                  dtype=self.model.dtype, device=self.model.device, poison=poison, poison_on_free=poison)
        self.step_fn = StepFunction(self.model, self.cache)
        self.live: dict = {}

    def step(self, entries, end=()) -> torch.Tensor:
        """entries: (id, tokens, want); returns float32 logits [wanted, vocab] on the CPU."""
        from miniserve_b200.engine.step import StepRow

        rows = []
        for rid, tokens, want in entries:
            if rid not in self.live:
                self.live[rid] = self.cache.new_request()
            want = list(range(len(tokens))) if want == "all" else want
            rows.append(StepRow(self.live[rid], list(tokens), list(want)))
        logits = self.step_fn.run(rows)
        self.step_fn.check_status()
        for rid in end:
            self.cache.release(self.live.pop(rid))
        return logits.float().cpu()

    def feed(self, rid, ids, sizes, end=True) -> torch.Tensor:
        """One request alone in portions of the given sizes (the last size repeats); logits everywhere."""
        outs, i, k = [], 0, 0
        while i < len(ids):
            n = min(sizes[min(k, len(sizes) - 1)], len(ids) - i)
            k += 1
            outs.append(self.step([(rid, ids[i:i + n], "all")], end=[rid] if end and i + n == len(ids) else []))
            i += n
        return torch.cat(outs)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest per-position distance of the logits (mean taken off), over the oracle's spread."""
    d = got.double() - want.double()
    d = d - d.mean(dim=-1, keepdim=True)
    spread = (want.double() - want.double().mean(dim=-1, keepdim=True)).pow(2).mean().sqrt()
    return (d.pow(2).mean(dim=-1).sqrt().max() / spread).item()


class _RoundedProducts(torch.Tensor):
    """A matrix whose products come back rounded to bfloat16 (and widened again)."""

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        args = [a.as_subclass(torch.Tensor) if isinstance(a, _RoundedProducts) else a for a in args]
        out = func(*args, **(kwargs or {}))
        name = getattr(func, "__name__", "")
        if name in ("matmul", "__matmul__", "__rmatmul__"):
            return out.bfloat16().to(out.dtype)
        if isinstance(out, torch.Tensor) and name in ("__get__", "t", "transpose"):
            return out.as_subclass(_RoundedProducts)
        return out


def rounding_noise(folder, ids) -> float:
    """rel_err of the oracle against itself when every matrix product's result is rounded to bfloat16:
    what rounding alone costs on this model and these tokens (the engine rounds in more places)."""
    cfg, w = plain.read_config(folder), plain.read_weights(folder, torch.float64)
    exact = plain.all_logits(cfg, w, ids)
    rounded = {k: (v.as_subclass(_RoundedProducts) if v.dim() == 2 and not k.endswith(".conv") and k != "embed" else v)
               for k, v in w.items()}
    return rel_err(torch.as_tensor(plain.all_logits(cfg, rounded, ids)).as_subclass(torch.Tensor), exact)
