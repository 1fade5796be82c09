"""Mugipel without a GPU: configuration -> parts and run order, declared tensors against a statement of the
checkpoint format, refused configurations, the cache manager's single pool for a latent, and the oracle's
functions against other statements of the same formulas."""

import math

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.config.registry import resolve
from miniserve_b200.parts import PagedKV
from miniserve_b200.parts.decoder import DecoderModel
from tests import mugipel_util as mx
from tests.plain import mugipel_plain as plain


# --------------------------------------------------------------------------- configuration
@pytest.mark.parametrize("make", [mx.config_a, mx.config_b, mx.config_c, mx.config_d])
def test_declared_tensors_are_the_checkpoint_format(make):
    raw = make()
    _, cfg, spec = resolve(raw)
    model = DecoderModel(spec, torch.bfloat16, "cpu")
    decls = {k: tuple(v.shape) for k, v in model.weight_decls().items()}
    assert decls == mx.tensor_shapes(raw)
    assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"]


def test_run_order_repeats_the_looped_layers_with_caches_of_their_own():
    raw = mx.config_a()
    _, cfg, spec = resolve(raw)
    assert [(e.layer, e.transition, e.transition_arg) for e in spec.run_order] == [
        (0, None, 0), (1, None, 0), (2, 0, 0), (3, None, 0), (2, 0, 1), (3, None, 0), (2, 0, 2), (3, None, 0)]
    model = DecoderModel(spec, torch.float32, "cpu")
    assert [c.owner for c in model.entry_caches] == list(range(8))  # every run has its own cache
    assert plain.run_order(raw) == cfg.run_layers()
    # a loop from the first layer on opens its first pass before anything else has run; no loop: no transition
    _, cfg_b, spec_b = resolve(mx.config_b())
    assert spec_b.run_order[0].transition == 0 and all(e.transition is None for e in spec_b.run_order[1:])
    _, _, spec_c = resolve(mx.config_c())
    assert not spec_c.transitions and all(e.transition is None for e in spec_c.run_order)


def test_cache_needs_follow_the_mixers():
    _, _, spec = resolve(mx.config_a())
    model = DecoderModel(spec, torch.bfloat16, "cpu")
    needs = [c.need for c in model.entry_caches]
    assert needs[0] == PagedKV(2, 32, 24)  # keys and values in one head size; the block mask bounds what is kept
    assert needs[1] == PagedKV(1, 48, None, values=False)  # a latent of 40 numbers in a head of 48: one pool for keys and values
    assert needs[2] == PagedKV(2, 32, 40)  # head sizes in steps of 16
    assert needs[3] == PagedKV(1, 16, None, values=False)
    cache = CacheManager(model.entry_caches, 10, 8, 2, device=None)
    per_token = {g.need: g.bytes_per_token(2) for g in cache.groups}
    assert per_token[needs[1]] == 1 * 48 * 2 and per_token[needs[0]] == 2 * 2 * 32 * 2


@pytest.mark.parametrize("change, error", [
    (lambda r: r["layers"][0].update(type="window_attention"), NotImplementedError),
    (lambda r: r["layers"][0]["mlp"].update(kind="experts"), NotImplementedError),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), ValueError),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), ValueError),
    (lambda r: r["layers"][0]["mixer"]["mask"].update(size=0), ValueError),
    (lambda r: r.update(loop={"start": 2, "stop": 5, "times": 2}), ValueError),
    (lambda r: r.update(loop={"start": 1, "stop": 2, "times": 0}), ValueError),
    (lambda r: r.pop("norm"), KeyError),
])
def test_refused_configurations(change, error):
    raw = mx.config_a()
    change(raw)
    with pytest.raises(error):
        resolve(raw)


def test_a_latent_beyond_the_kernels_head_sizes_is_refused_with_a_message():
    raw = mx.config([mx.latent_layer(rank=600)])
    _, _, spec = resolve(raw)
    with pytest.raises(NotImplementedError, match="latent"):
        DecoderModel(spec, torch.bfloat16, "cpu")


# --------------------------------------------------------------------------- the oracle against other statements
def test_sink_is_one_more_key_without_a_value():
    torch.manual_seed(0)
    t, h, g, dk, dv = 9, 4, 2, 6, 5
    q, k, v = torch.randn(t, h, dk, dtype=torch.float64), torch.randn(t, g, dk, dtype=torch.float64), torch.randn(t, g, dv, dtype=torch.float64)
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0], dtype=torch.float64)
    got = plain.softmax_attention(q, k, v, 0.7, plain.visible(t, None), softcap=4.0, sink=sink)
    for i in range(t):
        for head in range(h):
            s = torch.stack([4.0 * torch.tanh((q[i, head] @ k[j, head // 2]) * 0.7 / 4.0) for j in range(i + 1)])
            p = torch.softmax(torch.cat((s, sink[head:head + 1])), 0)  # the sink: neither scaled nor capped
            want = sum(p[j] * v[j, head // 2] for j in range(i + 1))
            assert torch.allclose(got[i, head], want, atol=1e-12)
    # weights of a row add up to less than one
    ones = plain.softmax_attention(q, k, torch.ones(t, g, 1, dtype=torch.float64), 0.7, plain.visible(t, None), sink=sink)
    assert (ones < 1).all() and (ones > 0).all()


def test_block_mask_counts_from_the_start_of_the_sequence():
    m = plain.visible(11, 4)
    for i in range(11):
        for j in range(11):
            assert bool(m[i, j]) == (j <= i and j >= (i // 4) * 4)
    assert plain.visible(5, None).sum() == 15


def test_rescaled_frequencies_keep_fast_pairs_and_slow_down_slow_ones():
    dims, base = 32, 10000.0
    scaling = {"factor": 8.0, "fast": 32.0, "original": 256, "slow": 1.0}
    f, mag = plain.yarn_frequencies(dims, base, scaling)
    plain_f, one = plain.yarn_frequencies(dims, base, None)
    assert one == 1.0 and abs(mag - (0.1 * math.log(8.0) + 1.0)) < 1e-15
    turns = plain_f * 256 / (2 * math.pi)  # turns a pair makes over the original context
    assert torch.allclose(f[turns > 40], plain_f[turns > 40])  # well above `fast`: unchanged
    assert torch.allclose(f[turns < 0.7], plain_f[turns < 0.7] / 8.0)  # well below `slow`: divided by the factor
    assert ((f <= plain_f + 1e-18) & (f >= plain_f / 8.0 - 1e-18)).all()
    # rotation keeps lengths up to the factor on cos and sin, and leaves the channels behind `dims` alone
    x = torch.randn(5, 2, 40, dtype=torch.float64)
    y = plain.rotate_halves(x, torch.arange(5), dims, base, scaling)
    assert torch.equal(y[..., dims:], x[..., dims:])
    assert torch.allclose(y[..., :dims].norm(dim=-1), x[..., :dims].norm(dim=-1) * mag)
    assert torch.allclose(y[0, :, :dims], x[0, :, :dims] * mag)  # position 0 turns nothing
    # scores depend on the distance only
    a = plain.rotate_halves(x[:1].expand(5, -1, -1), torch.arange(5), dims, base, scaling)
    b = plain.rotate_halves(x[1:2].expand(5, -1, -1), torch.arange(5) + 3, dims, base, scaling)
    dots = (a * b).sum(-1)
    assert torch.allclose(dots, dots[:1].expand_as(dots))


def test_latent_attention_is_attention_over_the_latent_itself():
    """Folding the per-head key matrix onto the query and the per-head value matrix behind attention gives the
    same numbers: what the engine does with one cached vector per token."""
    torch.manual_seed(1)
    t, width = 12, 20
    m = {"dim": 6, "heads": 3, "kv_rank": 10, "scale": 0.4, "vdim": 7}
    w = {"q": torch.randn(18, width), "dkv": torch.randn(10, width), "dkv.norm": torch.rand(10) + 0.5, "uk": torch.randn(18, 10),
         "uv": torch.randn(21, 10), "g": torch.randn(21, width), "o": torch.randn(width, 21)}
    w = {"m." + k: v.double() for k, v in w.items()}
    h = torch.randn(t, width, dtype=torch.float64)
    want = plain.latent_attention_mixer(h, w, "m.", m, 1e-5)
    c = plain.unit_rms(h @ w["m.dkv"].T, 1e-5) * w["m.dkv.norm"]
    q = (h @ w["m.q"].T).view(t, 3, 6)
    q_folded = torch.einsum("thd,hdr->thr", q, w["m.uk"].view(3, 6, 10))
    over_c = plain.softmax_attention(q_folded, c[:, None, :], c[:, None, :], 0.4, plain.visible(t, None))
    vals = torch.einsum("thr,hvr->thv", over_c, w["m.uv"].view(3, 7, 10)).reshape(t, 21)
    got = (vals * torch.sigmoid(h @ w["m.g"].T)) @ w["m.o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_offset_norm_and_feed_forward():
    x = torch.randn(4, 10, dtype=torch.float64)
    w = torch.randn(10, dtype=torch.float64) * 0.1
    y = plain.offset_norm(x, w, 1e-6)
    assert torch.allclose(y / (1 + w), x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6))
    assert torch.allclose(plain.offset_norm(x, torch.zeros(10, dtype=torch.float64), 0.0).pow(2).mean(-1), torch.ones(4, dtype=torch.float64))
    up, down = torch.randn(6, 10, dtype=torch.float64), torch.randn(10, 6, dtype=torch.float64)
    z = x @ up.T
    assert torch.allclose(plain.feed_forward(x, up, down), (torch.where(z > 0, z * z, torch.zeros_like(z))) @ down.T)


def test_model_stream_re_enters_with_the_embedding_beside_it():
    raw = mx.config_a()
    w = {k: v.double() for k, v in mx.random_weights(raw, 3).items()}
    ids = [5, 9, 2, 77, 30, 1]
    streams = plain.layer_streams(raw, w, ids)
    assert streams.shape == (8, 6, raw["width"])
    # the first pass of the loop starts from W [x ; x0] + step[0] with x the stream after layer 1
    x0 = w["embed"][torch.tensor(ids)]
    entered = torch.cat((streams[1], x0), -1) @ w["loop.in"].T + w["loop.step"][0]
    h = plain.offset_norm(entered, w["l2.norm1"], raw["norm"]["eps"])
    y = plain.attention_mixer(h, w, "l2.mix.", raw["layers"][2]["mixer"], torch.arange(6))  # this layer has no feed-forward
    assert torch.allclose(streams[2], entered + raw["residual_mult"] * y, atol=1e-10)
    # a prefix of the tokens gives the same logits at those positions (causal everywhere)
    full, part = plain.all_logits(raw, w, ids), plain.all_logits(raw, w, ids[:4])
    assert torch.allclose(full[:4], part, atol=1e-9)
