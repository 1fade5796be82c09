"""Fekulix on the GPU against the plain implementation: each mechanism alone, whole prompts against
token-by-token decoding and portions down to two tokens, unequal requests in one batch against each
alone, pages and state slots that are given back and used again, keys far away and at page borders,
the first tokens of a sequence, long decoding, sizes that are no round numbers, the trace runner and
greedy generation through the entry point."""

import random

import pytest
import torch

from miniserve_b200.cache.manager import KVEntryView, StateEntryView
from miniserve_b200.config import PartSpec
from miniserve_b200.parts import BuildEnv, build_part
from tests import fekulix_util as fx
from tests.kernel_util import PagedBatch, make_context
from tests.plain import fekulix_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
F32, BF16 = 2e-5, 1e-1  # logits: distance over their spread (rel_err); bfloat16: see the model fixture


def _ids(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def _close(got, want, dtype, scale=1.0):
    got, want = got.double().cpu(), want.double()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    err = (got - want).abs().max().item()
    assert err <= tol * scale * max(1.0, want.abs().max().item()), f"off by {err:.3e} (values up to {want.abs().max().item():.2f})"


def _bind(part, dtype, seed=0, std=0.3):
    """Random bfloat16-exact weights bound to the part; returns them as float64 by name."""
    gen = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, decl in part.all_weights().items():
        t = torch.randn(decl.shape, generator=gen) * std
        if decl.init == "ones_normal":
            t = 1.0 + t / 2
        t = t.to(torch.bfloat16)
        tensors[name] = t.to(device=DEV, dtype=torch.float32 if decl.precision == "float32" else dtype)
    part.bind_all(tensors)
    return {k: v.double().cpu() for k, v in tensors.items()}


@pytest.fixture(autouse=True)
def _seeded():
    torch.manual_seed(1234)
    torch.cuda.manual_seed(1234)


def _ctx(rows, page=8, kv_heads=1, d=16, dtype=torch.float32, slots=None, share=None, seed=0):
    pb = PagedBatch(rows, page, kv_heads, d, dtype, seed=seed, share=share)
    ctx = make_context(pb)
    ctx.state_slot = torch.tensor(slots if slots is not None else list(range(len(rows))), dtype=torch.int32, device=DEV)
    return pb, ctx


DTYPES = [torch.float32, torch.bfloat16]


# --------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_dynamic_tanh_with_add_and_gather(dtype):
    norm = build_part("norm", PartSpec("dynamic_tanh", dict(size=72, names=dict(weight="", bias=".b", alpha=".alpha"))),
                      BuildEnv(dtype, DEV))
    w = _bind(norm, dtype)
    res, delta = torch.randn(11, 72, device=DEV) * 3, (torch.randn(11, 72, device=DEV)).to(dtype)
    total = res.double().cpu() + delta.double().cpu()
    _, ctx = _ctx([(0, 11)], dtype=dtype)
    out = norm.forward(res, delta, ctx)
    _close(out, plain.dynamic_tanh(total, w[""], w[".b"], w[".alpha"]), dtype)
    assert torch.allclose(res.double().cpu(), total, atol=1e-6)  # the sum went back into the stream
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    out = norm.forward(res, None, ctx, rows=rows, num_rows=2, write_residual=False)
    _close(out, plain.dynamic_tanh(total[[7, 2]], w[""], w[".b"], w[".alpha"]), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward(dtype):
    ffn = build_part("feed_forward", PartSpec("dense_mlp", dict(hidden=40, intermediate=72, names=dict(up="up", down="down"))),
                     BuildEnv(dtype, DEV))
    w = _bind(ffn, dtype)
    x = torch.randn(9, 40, device=DEV).to(dtype)
    _, ctx = _ctx([(0, 9)], dtype=dtype)
    _close(ffn.forward(x, ctx), plain.dense_ff(x.double().cpu(), lambda n: w[n]), dtype, 3.0)


def _attention(dtype, heads, kv_heads, dim, vdim, rot, scale=0.3, hidden=48):
    c = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=dict(dims=rot, base=50.0), scale=scale)
    spec = PartSpec("gqa_attention", dict(
        hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=dim, value_dim=vdim, qk_norm=True, qk_norm_eps=1e-5, scale=scale,
        sink=True, out_gate="head_sigmoid", position=PartSpec("rope_pairs", dict(head_dim=dim, theta=50.0, rotary_dim=rot)),
        names=dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", gate="g")))
    return build_part("mixer", spec, BuildEnv(dtype, DEV)), c


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot, page", [(4, 2, 32, 16, 8, 8), (3, 1, 16, 40, 16, 16), (2, 2, 24, 24, 0, 4)])
def test_sink_attention_whole_in_portions_and_decoded(dtype, heads, kv_heads, dim, vdim, rot, page):
    att, c = _attention(dtype, heads, kv_heads, dim, vdim, rot)
    w = _bind(att, dtype)
    for k in ("q.norm", "k.norm"):  # peaked attention: a key that is lost or misplaced moves the output
        getattr(att, "w_" + k.replace(".", "_")).mul_(3.0)
        w[k] = w[k] * 3.0
    n = 45
    x = torch.randn(n, 48, device=DEV).to(dtype)
    ref = plain.softmax_branch(x.double().cpu(), torch.arange(n), lambda name: w[name], None, c, 1e-5)
    pb, ctx = _ctx([(0, n)], page, kv_heads, att.cache_dim, dtype, seed=1)
    view = KVEntryView(0, pb.k_pool, pb.v_pool, page)
    out = att.forward(x, ctx, view)
    assert pb.status.item() == 0
    _close(out, ref, dtype, 2.0)
    # the sink is in the result: without it the weights of a row would add up to one
    no_sink = plain.softmax_branch(x.double().cpu()[:1], torch.arange(1), lambda name: w[name], None, c, 1e-5)
    assert (out[0].double().cpu() - no_sink[0]).abs().max() < 1e-1 and ref[0].abs().max() > 0
    # portions over the same pages (cut inside a page), then single tokens
    full, _ = _ctx([(0, n)], page, kv_heads, att.cache_dim, dtype, seed=2)
    view = KVEntryView(0, full.k_pool, full.v_pool, page)
    outs, at = [], 0
    for size in (page + 3, 2, 13, 2) + (1,) * n:
        size = min(size, n - at)
        if size <= 0:
            break
        _, ctx = _ctx([(at, size)], page, kv_heads, att.cache_dim, dtype, share=full)
        outs.append(att.forward(x[at:at + size].contiguous(), ctx, view).clone())
        at += size
    _close(torch.cat(outs), ref, dtype, 2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, n", [(2, 1, 32, 32, 700), (4, 2, 128, 64, 1900), (2, 2, 48, 80, 1700)])
def test_sink_attention_finds_a_far_key_among_hundreds(dtype, heads, kv_heads, dim, vdim, n):
    """One early key and the last query are scaled so that this pair's score stands out; its value
    must come back, through pages, key splits and the sink. The longer cases cut the keys of the
    decoded token more than eight ways (partial results merged through scratch memory); head size 128
    takes the tensor-core kernels for the prompt."""
    att, c = _attention(dtype, heads, kv_heads, dim, vdim, 8, scale=1.0 if dim == 32 else 0.3)
    w = _bind(att, dtype)
    needle = 5
    x = torch.randn(n, 48, device=DEV).to(dtype) * 0.2
    x[n - 1] = x[needle] = (torch.randn(48, device=DEV) * 2).to(dtype)  # the same direction: after the norm q and k line up
    ref = plain.softmax_branch(x.double().cpu(), torch.arange(n), lambda name: w[name], None, c, 1e-5)
    full, _ = _ctx([(0, n)], 16, kv_heads, att.cache_dim, dtype, seed=3)
    view = KVEntryView(0, full.k_pool, full.v_pool, 16)
    _, ctx = _ctx([(0, n - 1)], 16, kv_heads, att.cache_dim, dtype, share=full)
    head = att.forward(x[:n - 1].contiguous(), ctx, view)
    _close(head, ref[:n - 1], dtype, 2.0)
    _, ctx = _ctx([(n - 1, 1)], 16, kv_heads, att.cache_dim, dtype, share=full)
    out = att.forward(x[n - 1:].contiguous(), ctx, view)
    _close(out, ref[n - 1:], dtype, 2.0)


def _state_views(part):
    need = part.cache_need()
    needs = need if isinstance(need, tuple) else (need,)
    views = tuple(StateEntryView(torch.full((5, *nd.shape), float("nan"), dtype=nd.dtype, device=DEV), tuple(nd.shape)) for nd in needs)
    return views if isinstance(need, tuple) else views[0]


def _portions(part, views, x, cuts, slot, dtype):
    outs, at = [], 0
    for size in cuts:
        size = min(size, x.shape[0] - at)
        if size <= 0:
            break
        _, ctx = _ctx([(at, size)], dtype=dtype, slots=[slot])
        outs.append(part.forward(x[at:at + size].contiguous(), ctx, views).clone())
        at += size
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dk, dv, rank", [(2, 24, 40, 8), (1, 40, 8, 5), (3, 16, 16, 16), (1, 72, 136, 4)])
def test_decay_linear_attention(dtype, heads, dk, dv, rank):
    c = dict(heads=heads, dim=dk, vdim=dv, tau=5.0)
    spec = PartSpec("decay_linear_attention", dict(hidden=48, heads=heads, key_dim=dk, value_dim=dv, tau=5.0, decay_rank=rank, eps=1e-5,
                                                   names=dict(q="q", k="k", v="v", g="g", o="o", norm="norm", a1="a1", a2="a2", a_bias="a2.b")))
    part = build_part("mixer", spec, BuildEnv(dtype, DEV))
    w = _bind(part, dtype)
    n = 70
    x = torch.randn(n, 48, device=DEV).to(dtype)
    ref = plain.linear_branch(x.double().cpu(), lambda name: w[name], c, 1e-5)
    views = _state_views(part)
    _close(_portions(part, views, x, (n,), 1, dtype), ref, dtype, 3.0)
    # the same slot again (state of the request before is still there), in portions down to two tokens, then token by token
    _close(_portions(part, views, x, (33, 2, 9, 2) + (1,) * n, 1, dtype), ref, dtype, 3.0)
    # two requests of unequal length in one step, in other slots
    _, ctx = _ctx([(0, 21), (0, n)], dtype=dtype, slots=[4, 0])
    both = part.forward(torch.cat((x[:21], x)), ctx, views)
    _close(both[21:], ref, dtype, 3.0)
    _close(both[:21], ref[:21], dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dk, dv", [(2, 24, 40), (1, 20, 136)])
def test_decay_linear_attention_over_segments_of_a_long_portion(dtype, heads, dk, dv):
    """A step of 512 tokens or more walks every row in eight segments at once and mends the outputs and the
    state afterwards: against the token-by-token oracle, whole, behind an earlier portion (a state to start
    from), beside a short row (segments that are empty), and then decoded on from the state it left."""
    c = dict(heads=heads, dim=dk, vdim=dv, tau=3.0)
    spec = PartSpec("decay_linear_attention", dict(hidden=48, heads=heads, key_dim=dk, value_dim=dv, tau=3.0, decay_rank=8, eps=1e-5,
                                                   names=dict(q="q", k="k", v="v", g="g", o="o", norm="norm", a1="a1", a2="a2", a_bias="a2.b")))
    part = build_part("mixer", spec, BuildEnv(dtype, DEV))
    w = _bind(part, dtype)
    n = 700
    x = torch.randn(n, 48, device=DEV).to(dtype)
    ref = plain.linear_branch(x.double().cpu(), lambda name: w[name], c, 1e-5)
    views = _state_views(part)
    _close(_portions(part, views, x, (n,), 1, dtype), ref, dtype, 3.0)
    _close(_portions(part, views, x, (37, 600, 2) + (1,) * n, 1, dtype), ref, dtype, 3.0)
    _, ctx = _ctx([(0, 5), (0, 690)], dtype=dtype, slots=[4, 0])
    both = part.forward(torch.cat((x[:5], x[:690])), ctx, views)
    _close(both[:5], ref[:5], dtype, 3.0)
    _close(both[5:], ref[:690], dtype, 3.0)
    _, ctx = _ctx([(690, 10)], dtype=dtype, slots=[0])
    _close(part.forward(x[690:].contiguous(), ctx, views), ref[690:], dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, groups, dk, dv, taps, ranks", [(4, 2, 16, 24, 3, (8, 16)), (2, 2, 40, 12, 2, (3, 7)),
                                                               (3, 1, 8, 16, 1, (8, 8)), (2, 1, 32, 72, 5, (4, 4))])
def test_gated_delta_rule(dtype, heads, groups, dk, dv, taps, ranks):
    c = dict(heads=heads, kv_heads=groups, dim=dk, vdim=dv, conv=taps)
    spec = PartSpec("gated_delta_rule", dict(
        hidden=48, heads=heads, kv_heads=groups, key_dim=dk, value_dim=dv, conv=taps, decay_rank=ranks[0], gate_rank=ranks[1],
        eps=1e-5, names=dict(q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", beta="b", a_log="A_log",
                             norm="norm", a1="a1", a2="a2", dt_bias="dt_bias", g1="g1", g2="g2", o="o")))
    part = build_part("mixer", spec, BuildEnv(dtype, DEV))
    w = _bind(part, dtype)
    n = 60
    x = torch.randn(n, 48, device=DEV).to(dtype)
    ref = plain.channel_delta_mixer(x.double().cpu(), lambda name: w[name], c, 1e-5)
    views = _state_views(part)
    _close(_portions(part, views, x, (n,), 2, dtype), ref, dtype, 3.0)
    # portions shorter than the convolution's history, single tokens from the very first one, the slot used before
    _close(_portions(part, views, x, (1, 1, 2, 1, 3, 2, 17, 2) + (1,) * n, 2, dtype), ref, dtype, 3.0)
    _, ctx = _ctx([(0, n), (0, 7)], dtype=dtype, slots=[3, 1])
    both = part.forward(torch.cat((x, x[:7])), ctx, views)
    _close(both[:n], ref, dtype, 3.0)
    _close(both[n:], ref[:7], dtype, 3.0)


# --------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=["a", "b", "c"])
def model(request, tmp_path_factory):
    raw = dict(a=fx.config_a, b=fx.config_b, c=fx.config_c)[request.param]()
    folder = fx.write_model(tmp_path_factory.mktemp("fekulix_" + request.param), raw, seed=dict(a=11, b=12, c=13)[request.param])
    # bfloat16: the engine may be as far from the float64 truth as rounding alone takes the oracle (times 2.5: it
    # rounds in more places than the products), and at least 0.1; a lost key, a stale state or a wrong slot costs 0.3 to 1
    noise = fx.rounding_noise(folder, _ids(90, raw["vocab"], 20))
    return dict(folder=folder, raw=raw, oracle=fx.oracle(folder), page=dict(a=16, b=8, c=32)[request.param],
                tol={"float32": F32, "bfloat16": max(BF16, 2.5 * noise)})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decoded_and_in_portions(model, dtype):
    vocab, tol = model["raw"]["vocab"], model["tol"][dtype]
    run = fx.Runner(model["folder"], dtype, max_tokens=256, page_size=model["page"])
    for n, seed in ((1, 1), (2, 2), (37, 3), (150, 4)):
        ids = _ids(n, vocab, seed)
        want = model["oracle"](ids)
        assert fx.rel_err(run.feed("w", ids, [n]), want) < tol
        if n > 2:
            assert fx.rel_err(run.feed("d", ids, [n - min(n - 1, 40), 1]), want) < tol  # the last 40 one by one
            assert fx.rel_err(run.feed("c", ids, [7, 2, 24, 3, model["page"], 2, 5, 31, 2, 1, 1, 2, 9]), want) < tol
        assert run.cache.is_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(model, dtype):
    """Up to four live requests, portions of some beside single tokens of others, a pool that holds
    only what is live: every page and slot is used by several requests in turn (pages are filled
    with NaN when given back, state slots keep the old request's state)."""
    vocab, tol = model["raw"]["vocab"], model["tol"][dtype]
    seqs = {f"r{i}": _ids(n, vocab, 20 + i) for i, n in enumerate([90, 5, 64, 33, 1, 120, 17, 48])}
    want = {k: model["oracle"](v) for k, v in seqs.items()}
    run = fx.Runner(model["folder"], dtype, max_tokens=4 * 128, page_size=model["page"], max_requests=4)
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
        assert fx.rel_err(torch.cat(got[rid]), want[rid]) < tol, rid
    assert run.cache.is_idle()


def test_long_decoding_in_float32(model):
    ids = _ids(400, model["raw"]["vocab"], 9)
    run = fx.Runner(model["folder"], "float32", max_tokens=448, page_size=model["page"])
    assert fx.rel_err(run.feed("long", ids, [3, 1]), model["oracle"](ids)) < 5 * F32


def test_trace_runner_replays_a_schedule(model, tmp_path):
    from tests.trace_util import Trace, run_trace

    vocab = model["raw"]["vocab"]
    a, b = _ids(50, vocab, 31), _ids(21, vocab, 32)
    tr = Trace()
    tr.step([("a", a[:30], [0, 29])])
    tr.step([("a", a[30:31], [0]), ("b", b[:19], "last")])
    tr.step([("b", b[19:20], [0]), ("a", a[31:], "all")], end=["a"])
    tr.step([("b", b[20:], [0])], end=["b"])
    tr.step([("c", b, "last")], end=["c"])  # in the pages and the slot that were given back
    out = run_trace(model["folder"], "float32", tr, tmp_path / "out", page_size=model["page"], vocab=vocab)
    want = {"a": model["oracle"](a), "b": model["oracle"](b), "c": model["oracle"](b)}
    assert len(out) == 2 + 2 + 1 + 19 + 1 + 1
    for (rid, pos, _), logits in out.items():
        assert fx.rel_err(logits[None], want[rid][pos:pos + 1]) < 5 * F32, (rid, pos)


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
