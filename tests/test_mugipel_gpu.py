"""Mugipel on the GPU against the plain implementation: each mechanism alone, whole prompts against
token-by-token decoding and portions down to two tokens, unequal requests in one batch against each
alone, pages that are given back and used again, keys far away, at page borders and just inside and just
outside a block of the mask (in prompts and in decoding), the first tokens of a sequence, long decoding,
sizes that are no round numbers, the trace runner and greedy generation through the entry point."""

import math
import random

import pytest
import torch

from miniserve_b200 import ops
from miniserve_b200.cache.manager import KVEntryView
from miniserve_b200.config import LayerSpec, PartSpec
from miniserve_b200.parts import BuildEnv, ResidualStream, build_part
from miniserve_b200.parts.block import build_block
from tests import mugipel_util as mx
from tests.kernel_util import PagedBatch, make_context
from tests.plain import mugipel_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
F32, BF16 = 2e-5, 1e-1  # logits: distance over their spread (rel_err); bfloat16: see the model fixture
DTYPES = [torch.float32, torch.bfloat16]
HIDDEN = 48


def _ids(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def _close(got, want, dtype, scale=1.0):
    got, want = got.double().cpu(), want.double()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    err = (got - want).abs().max().item()
    assert err <= tol * scale * max(1.0, want.abs().max().item()), f"off by {err:.3e} (values up to {want.abs().max().item():.2f})"


def _bind(part, dtype, seed=0, std=0.3, change=None):
    """Random bfloat16-exact weights bound to the part; returns them as float64 by name."""
    gen = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, decl in part.all_weights().items():
        t = torch.randn(decl.shape, generator=gen) * std
        if decl.init == "ones_normal":
            t = 1.0 + t / 2
        tensors[name] = t.to(torch.bfloat16).float()
    if change:
        change(tensors)
    on_device = {k: v.to(torch.bfloat16).to(device=DEV, dtype=torch.float32 if part.all_weights()[k].precision == "float32" else dtype)
                 for k, v in tensors.items()}
    part.bind_all(on_device)
    return {k: v.to(torch.bfloat16).double() for k, v in tensors.items()}


@pytest.fixture(autouse=True)
def _seeded():
    torch.manual_seed(4321)
    torch.cuda.manual_seed(4321)


def _ctx(rows, page=8, kv_heads=1, d=16, dtype=torch.float32, share=None, seed=0, token_ids=None):
    pb = PagedBatch(rows, page, kv_heads, d, dtype, seed=seed, share=share)
    ctx = make_context(pb)
    if token_ids is not None:
        ctx.token_ids = torch.tensor(token_ids, dtype=torch.int32, device=DEV)
    return pb, ctx


# --------------------------------------------------------------------------- norm, feed-forward, rotation table, re-entry
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [72, 50, 1160])
def test_offset_norm_with_a_scaled_add_and_a_gather(dtype, size):
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=size, eps=1e-5, unit_offset=True, name="")), BuildEnv(dtype, DEV))
    w = _bind(norm, dtype, std=0.2)
    res, delta = torch.randn(11, size, device=DEV) * 3, torch.randn(11, size, device=DEV).to(dtype)
    total = res.double().cpu() + 0.6 * delta.double().cpu()
    _, ctx = _ctx([(0, 11)], dtype=dtype)
    out = norm.forward(res, delta, ctx, delta_scale=0.6)
    _close(out, plain.offset_norm(total, w[""], 1e-5), dtype)
    assert torch.allclose(res.double().cpu(), total, atol=2e-6)  # the sum went back into the stream, in float32
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    out = norm.forward(res, None, ctx, rows=rows, num_rows=2, write_residual=False)
    _close(out, plain.offset_norm(total[[7, 2]], w[""], 1e-5), dtype)
    # the weight stays float32 in bfloat16 runs too: 1 + 2^-10 is not rounded to 1 before it multiplies
    norm.bind({"": torch.full((size,), 2.0 ** -10, device=DEV)})
    x = torch.full((1, size), 256.0, device=DEV)
    got = norm.forward(x, None, ctx, rows=rows[:1] * 0, num_rows=1, write_residual=False)
    assert got.dtype == dtype and norm.w_weight.dtype == torch.float32
    if dtype == torch.float32:
        assert abs(got.mean().item() - (1.0 + 2.0 ** -10)) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, inter", [(40, 72), (36, 52)])
def test_squared_relu_feed_forward(dtype, hidden, inter):
    ffn = build_part("feed_forward", PartSpec("dense_mlp", dict(hidden=hidden, intermediate=inter, activation="relu_squared",
                                                                names=dict(up="up", down="down"))), BuildEnv(dtype, DEV))
    w = _bind(ffn, dtype)
    x = torch.randn(9, hidden, device=DEV).to(dtype)
    _, ctx = _ctx([(0, 9)], dtype=dtype)
    _close(ffn.forward(x, ctx), plain.feed_forward(x.double().cpu(), w["up"], w["down"]), dtype, 3.0)
    wide = torch.zeros(9, inter + 24, device=DEV, dtype=dtype)
    ffn.features(x, ctx, wide[:, 16:16 + inter])  # at a column offset of wider rows
    _close(wide[:, 16:16 + inter], plain.relu_squared(x.double().cpu() @ w["up"].T), dtype, 3.0)
    assert (wide[:, :16] == 0).all() and (wide[:, 16 + inter:] == 0).all()


@pytest.mark.parametrize("rot, base, scaling", [(8, 100.0, {"factor": 4.0, "fast": 8.0, "original": 64, "slow": 0.5}),
                                                (32, 300000.0, {"factor": 16.0, "fast": 24.0, "original": 1024, "slow": 2.0}),
                                                (6, 37.0, {"factor": 1.5, "fast": 4.0, "original": 16, "slow": 1.0})])
def test_rescaled_rotation_table(rot, base, scaling):
    pos = build_part("position", PartSpec("rope_yarn", dict(head_dim=rot + 8, theta=base, rotary_dim=rot, **scaling)),
                     BuildEnv(torch.float32, DEV))
    f, mag = plain.yarn_frequencies(rot, base, scaling)
    assert torch.allclose(pos.inv_freq.double().cpu(), f, rtol=1e-7)
    _, ctx = _ctx([(3, 5), (1000, 2)])
    table = pos.step_table(ctx).double().cpu()
    p = torch.tensor([3, 4, 5, 6, 7, 1000, 1001], dtype=torch.float64)
    ang = p[:, None] * f[None, :]
    assert torch.allclose(table[:, :rot // 2], torch.cos(ang) * mag, atol=2e-4)  # float32 angles at positions of a thousand
    assert torch.allclose(table[:, rot // 2:], torch.sin(ang) * mag, atol=2e-4)
    assert pos.step_table(ctx) is pos.step_table(ctx)  # made once per step


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_reentry(dtype):
    hidden, vocab, n = 40, 23, 7
    part = build_part("transition", PartSpec("stream_reentry", dict(hidden=hidden, passes=3, weight="in", step="step")), BuildEnv(dtype, DEV))
    emb = build_part("embedding", PartSpec("token_embedding", dict(vocab=vocab, hidden=hidden, name="embed")), BuildEnv(dtype, DEV))
    w = _bind(part, dtype)
    we = _bind(emb, dtype, seed=5)
    ids = _ids(n, vocab, 1)
    _, ctx = _ctx([(0, n)], dtype=dtype, token_ids=ids)
    total, pending = torch.randn(n, hidden, device=DEV), torch.randn(n, hidden, device=DEV).to(dtype)
    x = total.double().cpu() + 0.5 * pending.double().cpu()
    for arg in (0, 2):  # the second call of a step writes only the stream's half again
        out = part.forward(ResidualStream(total, pending, 0.5), ctx, emb, arg)
        assert out.pending is None and out.total.dtype == torch.float32
        want = torch.cat((x, we["embed"][torch.tensor(ids)]), -1) @ w["in"].T + w["step"][arg]
        _close(out.total, want, dtype, 3.0)
    with pytest.raises(ValueError):
        part.forward(ResidualStream(total), ctx, emb, 3)


# --------------------------------------------------------------------------- attention
def _attention(dtype, heads, kv_heads, dim, vdim, rot, scale=0.3, softcap=6.0, chunk=12, scaling=True):
    layer = mx.attention_layer(heads, kv_heads, dim, vdim, rot, 50.0, scaling, scale, softcap, chunk)["mixer"]
    from miniserve_b200.models.mugipel import _attention as spec_of

    return build_part("mixer", spec_of(HIDDEN, layer), BuildEnv(dtype, DEV)), layer


def _attention_ref(x, w, c, n=None):
    x = x.double().cpu()
    return plain.attention_mixer(x, {"m." + k: v for k, v in w.items()}, "m.", c, torch.arange(x.shape[0]))


def _portions(part, view, x, cuts, page, kv_heads, dtype, full):
    outs, at = [], 0
    for size in cuts:
        size = min(size, x.shape[0] - at)
        if size <= 0:
            break
        _, ctx = _ctx([(at, size)], page, kv_heads, part.cache_dim, dtype, share=full)
        outs.append(part.forward(x[at:at + size].contiguous(), ctx, view).clone())
        at += size
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot, page, chunk, softcap", [
    (4, 2, 32, 16, 8, 8, 12, 6.0), (5, 1, 16, 40, 16, 16, 7, 2.0), (2, 2, 24, 24, 0, 4, None, None), (6, 2, 48, 32, 32, 16, 50, None),
    (4, 2, 128, 128, 64, 16, 100, 5.0), (2, 1, 128, 64, 128, 32, None, 3.0)])  # head size 128: prompts on the tcgen05 kernel
def test_attention_whole_in_portions_and_decoded(dtype, heads, kv_heads, dim, vdim, rot, page, chunk, softcap):
    att, c = _attention(dtype, heads, kv_heads, dim, vdim, rot, softcap=softcap, chunk=chunk, scaling=rot != 16)
    w = _bind(att, dtype, change=lambda t: t["sink"].mul_(4.0))
    n = 61 if dim < 128 else 333
    x = torch.randn(n, HIDDEN, device=DEV).to(dtype) * 2
    ref = _attention_ref(x, w, c)
    pb, ctx = _ctx([(0, n)], page, kv_heads, att.cache_dim, dtype, seed=1)
    view = KVEntryView(0, pb.k_pool, pb.v_pool, page)
    out = att.forward(x, ctx, view)
    assert pb.status.item() == 0
    _close(out, ref, dtype, 2.0)
    full, _ = _ctx([(0, n)], page, kv_heads, att.cache_dim, dtype, seed=2)
    view = KVEntryView(0, full.k_pool, full.v_pool, page)
    _close(_portions(att, view, x, (page + 3, 2, 13, 2) + (1,) * n, page, kv_heads, dtype, full), ref, dtype, 2.0)
    # two unequal requests in one step (the second decodes a token behind what an earlier step left)
    both_pb, _ = _ctx([(0, 30), (0, n)], page, kv_heads, att.cache_dim, dtype, seed=7)
    view = KVEntryView(0, both_pb.k_pool, both_pb.v_pool, page)
    _, warm = _ctx([(0, 1), (0, n - 1)], page, kv_heads, att.cache_dim, dtype, share=both_pb)
    att.forward(torch.cat((x[:1], x[:n - 1])).contiguous(), warm, view)
    _, ctx = _ctx([(0, 30), (n - 1, 1)], page, kv_heads, att.cache_dim, dtype, share=both_pb)
    both = att.forward(torch.cat((x[:30], x[n - 1:])).contiguous(), ctx, view)
    _close(both[:30], ref[:30], dtype, 2.0)
    _close(both[30:], ref[n - 1:], dtype, 2.0)


def _needle_weights(tensors, heads, kv_heads, dim):
    """Head h's query matrix is minus its kv head's key matrix: a query scores far below everything against its own
    token's key, and far above everything against the key of a token whose input is minus its own (on the
    channels that are not rotated, which are most)."""
    k = tensors["k"].view(kv_heads, dim, -1)
    tensors["q"].copy_(-k.repeat_interleave(heads // kv_heads, dim=0).reshape(heads * dim, -1))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk, n, page, dim", [(16, 41, 8, 32), (20, 75, 16, 32), (512, 700, 16, 32), (2048, 1900, 16, 32),
                                                  (100, 777, 16, 128), (300, 1300, 32, 128), (4096, 2100, 16, 128)])
def test_a_key_just_inside_and_just_outside_the_block(dtype, chunk, n, page, dim):
    """The last query and one earlier token are made so that this pair scores far above everything else. With the
    earlier token at the first position of the last query's block its value must come back; one position before it
    must not, in a prompt and for a token decoded alone (the long cases cut the decoded token's keys several ways;
    head size 128 runs its prompts on the tcgen05 kernel, the longest one with its keys in several splits)."""
    heads, kv_heads, vdim = 4, 2, dim
    att, c = _attention(dtype, heads, kv_heads, dim, vdim, 8, scale=1.0, softcap=30.0, chunk=chunk)
    w = _bind(att, dtype, change=lambda t: _needle_weights(t, heads, kv_heads, dim))
    start = ((n - 1) // chunk) * chunk
    direction = (torch.randn(HIDDEN, device=DEV) * 3).to(dtype)
    for needle in (start, start - 1, start + 1, 0):
        if needle < 0:
            continue
        x = torch.randn(n, HIDDEN, device=DEV).to(dtype) * 0.1
        x[n - 1], x[needle] = direction, -direction
        ref = _attention_ref(x, w, c)
        blank = x.clone()
        blank[needle] = (torch.randn(HIDDEN, device=DEV) * 0.1).to(dtype)
        shows = (ref[n - 1] - _attention_ref(blank, w, c)[n - 1]).abs().max().item()
        assert (shows > 0.05) == (needle >= start), "the test's needle shows exactly when it is inside the block"
        full, _ = _ctx([(0, n)], page, kv_heads, att.cache_dim, dtype, seed=3)
        view = KVEntryView(0, full.k_pool, full.v_pool, page)
        _, ctx = _ctx([(0, n)], page, kv_heads, att.cache_dim, dtype, share=full)
        _close(att.forward(x, ctx, view), ref, dtype, 2.0)  # in a prompt
        _, ctx = _ctx([(n - 1, 1)], page, kv_heads, att.cache_dim, dtype, share=full)
        _close(att.forward(x[n - 1:].contiguous(), ctx, view), ref[n - 1:], dtype, 2.0)  # decoded alone over the same pages
        _, ctx = _ctx([(n - 3, 3)], page, kv_heads, att.cache_dim, dtype, share=full)
        _close(att.forward(x[n - 3:].contiguous(), ctx, view), ref[n - 3:], dtype, 2.0)  # a short portion


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink_takes_its_share_and_is_not_capped(dtype):
    """A large sink score empties the output; a very negative one gives the plain softmax. The cap would clip a
    sink of 9 to 2 if it were applied to it."""
    heads, kv_heads, dim, vdim = 2, 1, 16, 16
    att, c = _attention(dtype, heads, kv_heads, dim, vdim, 0, softcap=2.0, chunk=None)

    def sinks(t):
        t["sink"].copy_(torch.tensor([9.0, -30.0]))

    w = _bind(att, dtype, change=sinks)
    n = 20
    x = torch.randn(n, HIDDEN, device=DEV).to(dtype)
    ref = _attention_ref(x, w, c)
    pb, ctx = _ctx([(0, n)], 8, kv_heads, att.cache_dim, dtype)
    out = att.forward(x, ctx, KVEntryView(0, pb.k_pool, pb.v_pool, 8))
    _close(out, ref, dtype, 2.0)
    capped = dict(w)
    capped["sink"] = torch.tensor([2.0, -30.0], dtype=torch.float64)
    assert (_attention_ref(x, capped, c) - ref).abs().max() > 0.05


# --------------------------------------------------------------------------- latent attention
def _latent(dtype, heads, dim, vdim, rank, scale=0.35):
    layer = mx.latent_layer(heads, dim, vdim, rank, scale)["mixer"]
    from miniserve_b200.models.mugipel import _latent as spec_of

    return build_part("mixer", spec_of(HIDDEN, 1e-5, layer), BuildEnv(dtype, DEV)), layer


def _latent_ref(x, w, c):
    return plain.latent_attention_mixer(x.double().cpu(), {"m." + k: v for k, v in w.items()}, "m.", c, 1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, vdim, rank, page", [(3, 16, 24, 40, 8), (5, 12, 20, 36, 16), (2, 40, 40, 128, 16), (1, 64, 8, 16, 4),
                                                          (2, 16, 24, 300, 16)])  # a latent beyond the tensor-core kernels' head sizes
def test_latent_attention_whole_in_portions_and_decoded(dtype, heads, dim, vdim, rank, page):
    att, c = _latent(dtype, heads, dim, vdim, rank)
    w = _bind(att, dtype)
    n = 53
    x = torch.randn(n, HIDDEN, device=DEV).to(dtype) * 2
    ref = _latent_ref(x, w, c)
    pb, ctx = _ctx([(0, n)], page, 1, att.cache_dim, dtype, seed=1)
    pb.v_pool = pb.k_pool  # one pool serves as keys and values
    view = KVEntryView(0, pb.k_pool, pb.k_pool, page)
    out = att.forward(x, ctx, view)
    assert pb.status.item() == 0
    _close(out, ref, dtype, 3.0)
    stored = pb.read(0, pb.k_pool, n)[:, 0].double().cpu()  # what the cache holds is the normed latent, zero beyond its size
    latent = plain.unit_rms(x.double().cpu() @ w["dkv"].T, 1e-5) * w["dkv.norm"]
    _close(stored[:, :rank], latent, dtype, 2.0)
    assert (stored[:, rank:] == 0).all()
    full, _ = _ctx([(0, n)], page, 1, att.cache_dim, dtype, seed=2)
    view = KVEntryView(0, full.k_pool, full.k_pool, page)
    _close(_portions(att, view, x, (page + 3, 2, 13, 2) + (1,) * n, page, 1, dtype, full), ref, dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n, rank", [(700, 48), (1900, 128)])
def test_latent_attention_finds_a_far_key_among_hundreds(dtype, n, rank):
    heads, dim, vdim = 4, 32, 32
    att, c = _latent(dtype, heads, dim, vdim, rank, scale=1.0)

    def align(t):  # a token's query is minus its own key before the norm: q_h = -W_uk[h] W_down x
        t["q"].copy_(-(t["uk"] @ t["dkv"]).to(torch.bfloat16).float() * 0.5)

    w = _bind(att, dtype, change=align)
    needle = 5
    x = torch.randn(n, HIDDEN, device=DEV).to(dtype) * 0.1
    direction = (torch.randn(HIDDEN, device=DEV) * 2).to(dtype)
    x[n - 1], x[needle] = direction, -direction  # the needle's latent is minus the last token's: the one large score
    ref = _latent_ref(x, w, c)
    blank = x.clone()
    blank[needle] = (torch.randn(HIDDEN, device=DEV) * 0.1).to(dtype)
    assert (ref[n - 1] - _latent_ref(blank, w, c)[n - 1]).abs().max() > 0.05, "the test's needle does not show"
    full, _ = _ctx([(0, n)], 16, 1, att.cache_dim, dtype, seed=3)
    view = KVEntryView(0, full.k_pool, full.k_pool, 16)
    _, ctx = _ctx([(0, n - 1)], 16, 1, att.cache_dim, dtype, share=full)
    _close(att.forward(x[:n - 1].contiguous(), ctx, view), ref[:n - 1], dtype, 3.0)
    _, ctx = _ctx([(n - 1, 1)], 16, 1, att.cache_dim, dtype, share=full)
    _close(att.forward(x[n - 1:].contiguous(), ctx, view), ref[n - 1:], dtype, 3.0)


# --------------------------------------------------------------------------- the block
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ff", [56, None])
def test_parallel_residual_block(dtype, ff):
    raw = mx.config([mx.attention_layer(heads=2, kv_heads=1, dim=16, vdim=24, rot=8, chunk=9, ff=ff)], width=HIDDEN, mult=0.3)
    from miniserve_b200.config.registry import resolve

    _, _, spec = resolve(raw)
    block = build_block(spec.layers[0], BuildEnv(dtype, DEV))
    w = {"l0." + k: v for k, v in _bind(block, dtype).items()}
    assert block.joint == (ff is not None)
    n = 30
    total = torch.randn(n, HIDDEN, device=DEV)
    pending = torch.randn(n, HIDDEN, device=DEV).to(dtype)
    x = total.double().cpu() + 2.0 * pending.double().cpu()
    pb, ctx = _ctx([(0, n)], 8, 1, block.mixer.cache_dim, dtype)
    out = block.forward(ResidualStream(total, pending, 2.0), ctx, KVEntryView(0, pb.k_pool, pb.v_pool, 8))
    h = plain.offset_norm(x, w["l0.norm1"], 1e-5)
    y = plain.attention_mixer(h, w, "l0.mix.", raw["layers"][0]["mixer"], torch.arange(n))
    if ff:
        y = y + plain.feed_forward(h, w["l0.mlp.up"], w["l0.mlp.down"])
    assert out.pending_scale == 0.3
    _close(out.total, x, dtype)  # the earlier addend is in the stream, the block's own is handed on
    _close(out.pending, y, dtype, 4.0)


# --------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=["a", "b", "c", "d"])
def model(request, tmp_path_factory):
    raw = dict(a=mx.config_a, b=mx.config_b, c=mx.config_c, d=mx.config_d)[request.param]()
    folder = mx.write_model(tmp_path_factory.mktemp("mugipel_" + request.param), raw, seed=dict(a=11, b=12, c=13, d=14)[request.param])
    # bfloat16: the engine may be as far from the float64 truth as rounding alone takes the oracle (times 2.5: it
    # rounds in more places than the products), and at least 0.1; a lost key or a wrong page costs 0.3 to 1
    noise = mx.rounding_noise(folder, _ids(90, raw["vocab"], 20))
    return dict(folder=folder, raw=raw, oracle=mx.oracle(folder), page=dict(a=16, b=8, c=32, d=16)[request.param],
                tol={"float32": F32, "bfloat16": max(BF16, 2.5 * noise)})


def test_layer_streams_in_float32(model):
    """The residual stream after every layer run, against the oracle's (a looped layer counts each time)."""
    from miniserve_b200.cache import CacheManager
    from miniserve_b200.engine.loader import load_model
    from miniserve_b200.engine.step import StepFunction, StepRow

    ids = _ids(29, model["raw"]["vocab"], 8)
    w = plain.read_weights(model["folder"], torch.float64)
    want = plain.layer_streams(model["raw"], w, ids)
    _, _, net = load_model(model["folder"], "float32", "cuda:0")
    cache = CacheManager(net.entry_caches, 8, 16, 2, dtype=net.dtype, device=net.device)
    ctx = StepFunction(net, cache).prepare([StepRow(cache.new_request(), ids, [0])])
    stream = ResidualStream(net.embedding.forward(ctx))
    for i, e in enumerate(net.spec.run_order):
        if e.transition is not None:
            stream = net.transitions[e.transition].forward(stream, ctx, net.embedding, e.transition_arg)
        stream = net.layers[e.layer].forward(stream, ctx, cache.entry_views[i])
        x = stream.total.double().cpu() + stream.pending_scale * stream.pending.double().cpu()
        assert (x - want[i]).abs().max() < 1e-4 * max(1.0, want[i].abs().max()), f"after run {i} (layer {e.layer})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decoded_and_in_portions(model, dtype):
    vocab, tol = model["raw"]["vocab"], model["tol"][dtype]
    run = mx.Runner(model["folder"], dtype, max_tokens=256, page_size=model["page"])
    for n, seed in ((1, 1), (2, 2), (37, 3), (150, 4)):
        ids = _ids(n, vocab, seed)
        want = model["oracle"](ids)
        assert mx.rel_err(run.feed("w", ids, [n]), want) < tol
        if n > 2:
            assert mx.rel_err(run.feed("d", ids, [n - min(n - 1, 60), 1]), want) < tol  # the last 60 one by one, across block edges
            assert mx.rel_err(run.feed("c", ids, [7, 2, 24, 3, model["page"], 2, 5, 31, 2, 1, 1, 2, 9]), want) < tol
        assert run.cache.is_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages(model, dtype):
    """Up to four live requests, portions of some beside single tokens of others, a pool that holds only what is
    live: every page is used by several requests in turn (pages are filled with NaN when given back, and the
    layers with a block mask give pages back while a request runs)."""
    vocab, tol = model["raw"]["vocab"], model["tol"][dtype]
    seqs = {f"r{i}": _ids(n, vocab, 20 + i) for i, n in enumerate([90, 5, 64, 33, 1, 120, 17, 48])}
    want = {k: model["oracle"](v) for k, v in seqs.items()}
    run = mx.Runner(model["folder"], dtype, max_tokens=4 * 128, page_size=model["page"], max_requests=4)
    rng = random.Random(5)
    waiting, live, at, got = list(seqs), [], {}, {k: [] for k in seqs}
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        entries, ended = [], []
        order = sorted(live, key=lambda r: at[r] == 0 or len(seqs[r]) - at[r] > 40)  # decoding rows first
        for rid in order:
            left = len(seqs[rid]) - at[rid]
            n = 1 if left <= 40 and at[rid] > 0 else min(left, rng.choice([2, 3, 16, 29, 50]))
            if rng.random() < 0.15 and len(order) > 1:
                continue  # left out of this step
            entries.append((rid, seqs[rid][at[rid]:at[rid] + n], "all"))
            at[rid] += n
            if at[rid] == len(seqs[rid]):
                ended.append(rid)
        if not entries:
            continue
        logits = run.step(entries, end=ended)
        i = 0
        for rid, toks, _ in entries:
            got[rid].append(logits[i:i + len(toks)])
            i += len(toks)
        live = [r for r in live if r not in ended]
    for rid in seqs:
        assert mx.rel_err(torch.cat(got[rid]), want[rid]) < tol, rid
    assert run.cache.is_idle()


def test_long_decoding_in_float32(model):
    ids = _ids(400, model["raw"]["vocab"], 9)
    run = mx.Runner(model["folder"], "float32", max_tokens=448, page_size=model["page"])
    assert mx.rel_err(run.feed("long", ids, [3, 1]), model["oracle"](ids)) < 5 * F32


def test_trace_runner_replays_a_schedule(model, tmp_path):
    from tests.trace_util import Trace, run_trace

    vocab = model["raw"]["vocab"]
    a, b = _ids(50, vocab, 31), _ids(21, vocab, 32)
    tr = Trace()
    tr.step([("a", a[:30], [0, 29])])
    tr.step([("a", a[30:31], [0]), ("b", b[:19], "last")])
    tr.step([("b", b[19:20], [0]), ("a", a[31:], "all")], end=["a"])
    tr.step([("b", b[20:], [0])], end=["b"])
    tr.step([("c", b, "last")], end=["c"])  # in the pages that were given back
    out = run_trace(model["folder"], "float32", tr, tmp_path / "out", page_size=model["page"], vocab=vocab)
    want = {"a": model["oracle"](a), "b": model["oracle"](b), "c": model["oracle"](b)}
    assert len(out) == 2 + 2 + 1 + 19 + 1 + 1
    for (rid, pos, _), logits in out.items():
        assert mx.rel_err(logits[None], want[rid][pos:pos + 1]) < 5 * F32, (rid, pos)


@pytest.mark.parametrize("dtype, cuda_graph", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_greedy_generation_through_the_entry_point(model, dtype, cuda_graph):
    from miniserve_b200.engine import LLM, SamplingParams

    vocab = model["raw"]["vocab"]
    prompts = [_ids(n, vocab, 40 + n) for n in (5, 17, 33, 1, 9, 70)]
    llm = LLM(model["folder"], dtype=dtype, kv_pool_tokens=1024, page_size=model["page"], max_running=4,
              chunked_prefill_size=24, cuda_graph=cuda_graph)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=10))
    assert llm.engine.cache.is_idle()
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        seq = list(p)
        for t in o:  # teacher-forced: each chosen token is the oracle's best, or within rounding of it
            logits = model["oracle"](seq)[-1]
            assert (logits.max() - logits[t]).item() <= (1e-4 if dtype == "float32" else 0.15), (len(seq), t)
            seq.append(t)
